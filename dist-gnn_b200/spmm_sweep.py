"""Standalone distributed SpMM sweep: seeded R-MAT adjacency x dense fp32 operand, 1D broadcast-SpMM.

    python dist-gnn_b200/spmm_sweep.py --nodes 1048576 --degree 16 --widths 16,64,256,512 --iters 5
    python -m torch.distributed.run --nproc-per-node N ... dist-gnn_b200/spmm_sweep.py ...      (N ranks, one per GPU)

For every width it prints one JSON line: device time of the local products (CUDA events around every product),
algorithmic GB/s  (8*nnz + 4*(m+1) + 4*F*touched + 4*F*m*(1+[beta!=0])) / t  against the measured HBM peak, the no-reuse
gather GB/s, and with more than one rank the broadcast bus GB/s and the broadcast/compute overlap of the stage loop.
The same command with small sizes is what the profiler captures are taken from.
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)

import torch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--nodes', type=int, default=1 << 20)
    ap.add_argument('--degree', type=int, default=16, help='average directed degree before self loops')
    ap.add_argument('--widths', default='16,64,256,512')
    ap.add_argument('--iters', type=int, default=5)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--seed', type=int, default=0)
    ap.add_argument('--beta', type=float, default=0.0, help='0: overwrite C (first stage), 1: accumulate')
    ap.add_argument('--no-permute', action='store_true')
    args = ap.parse_args()

    import spmm_cpp
    from coo_graph import graph_utils, synthetic
    from dist_utils import DistEnv
    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29556')
    os.environ.setdefault('DIST_GNN_LOG_ROOT', '/tmp/dist_gnn_bench_logs')
    env = DistEnv(rank, world, 'nccl')
    dev = env.device
    N = args.nodes
    ei = synthetic.rmat_edge_index(N, N * args.degree, args.seed, permute=not args.no_permute, device=dev)
    A = graph_utils.sym_normalization(ei, N)
    del ei
    n = (N + world - 1) // world
    row_block = graph_utils.sparse_2d_split(A, n, split_dim=0)[rank]
    del A
    row_block = graph_utils._coo(row_block.indices(), row_block.values(), (n, n * world))
    parts = graph_utils.sparse_2d_split(row_block, n, split_dim=1)
    del row_block
    plans = [spmm_cpp.SpmmPlan.from_coo(p) for p in parts]
    peak = 6546.9
    peaks_file = os.path.join(os.path.dirname(HERE), 'MEASURED_PEAKS.json')
    if os.path.exists(peaks_file):
        with open(peaks_file) as f:
            peak = float(json.load(f)['hbm_gbs'])
    for width in (int(w) for w in args.widths.split(',')):
        x = torch.randn(n, width, device=dev)
        z = torch.zeros(n, width, device=dev)
        line = {'nodes': N, 'degree': args.degree, 'width': width, 'ranks': world, 'rank': rank,
                'nnz_rank': sum(p.stats()['nnz'] for p in plans)}
        if world == 1:
            for _ in range(args.warmup):
                plans[0].spmm(x, z, 1.0, args.beta)
            spmm_cpp.profile_begin()
            for _ in range(args.iters):
                plans[0].spmm(x, z, 1.0, args.beta)
            prof = spmm_cpp.profile_end()
        else:
            recv = env.recv_buffers(n, width)
            roots = list(range(world))
            for _ in range(args.warmup):
                spmm_cpp.bcast_spmm(env.comm, roots, plans, x, recv, z)
            spmm_cpp.profile_begin()
            for _ in range(args.iters - 1):
                spmm_cpp.bcast_spmm(env.comm, roots, plans, x, recv, z)
            spmm_cpp.bcast_spmm(env.comm, roots, plans, x, recv, z, timed=True)
            prof = spmm_cpp.profile_end()
            t = env.comm.last_times()
            msg = n * width * 4
            line.update(bcast_bus_gbs=round(world * msg / (t['comm_ms'] * 1e-3) / 1e9, 2), comm_ms=round(t['comm_ms'], 4),
                        loop_ms=round(t['total_ms'], 4), loop_spmm_ms=round(t['spmm_ms'], 4),
                        overlap=round((t['comm_ms'] + t['spmm_ms'] - t['total_ms']) / max(min(t['comm_ms'], t['spmm_ms']), 1e-9), 4))
        sec = prof['spmm_ms'] * 1e-3
        line.update(spmm_ms=round(prof['spmm_ms'] / args.iters, 4), alg_gbs=round(prof['alg_bytes'] / sec / 1e9, 2),
                    frac_of_hbm_peak=round(prof['alg_bytes'] / sec / 1e9 / peak, 4), gather_gbs=round(prof['gather_bytes'] / sec / 1e9, 2),
                    gflops=round(prof['flops'] / sec / 1e9, 2), kernel_launches=prof['kernel_launches'])
        for r in range(world):
            if r == rank:
                print(json.dumps(line), flush=True)
            if world > 1:
                env.barrier_all()
    env.shutdown()


if __name__ == '__main__':
    main()
