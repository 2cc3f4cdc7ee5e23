"""Launcher with the flags of light_dist_gnn/main.py:24-33 (--nprocs --epoch --backend --dataset) plus --layers,
--hidden and --rep (1.5D replication factor).  One process per GPU, spawned on this host."""
import argparse
import os

import torch

import dist_train
import dist_utils


def process_wrapper(rank, args, func):
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29500')
    os.environ.setdefault('NCCL_SOCKET_IFNAME', 'lo')
    env = dist_utils.DistEnv(rank, args.nprocs, args.backend, rep=getattr(args, 'rep', 1))
    try:
        func(env, args)
    finally:
        env.shutdown()


if __name__ == '__main__':
    num_GPUs = torch.cuda.device_count()
    parser = argparse.ArgumentParser()
    parser.add_argument('--nprocs', type=int, default=max(num_GPUs, 1))
    parser.add_argument('--epoch', type=int, default=20)
    parser.add_argument('--backend', type=str, default='nccl')
    parser.add_argument('--dataset', type=str, default='rmat_plumbing')
    parser.add_argument('--layers', type=int, default=3)
    parser.add_argument('--hidden', type=int, default=256)
    parser.add_argument('--rep', type=int, default=1)
    args = parser.parse_args()
    torch.multiprocessing.spawn(process_wrapper, (args, dist_train.main), args.nprocs)
