"""Compare the stage-loop schedules of the distributed SpMM on the benchmark graph: one graph build and one process
group, then for every variant a few timed epochs and one timed distributed SpMM per operand width.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29711 \\
        dist-gnn_b200/stage_sweep.py --variants peer_compact:1,peer_copy:1,feature_chunks:1:128,reference:4
    ... dist-gnn_b200/stage_sweep.py --rep 2 --layers 4 --variants reference:1,reference:2        (1.5D, config 3)

A variant is  stage_order:stage_group[:chunk_width].  Rank 0 prints one JSON line per variant: epoch ms (CUDA events,
max over ranks) and per width the transfer rate, transfer / product / loop times and the overlap, as bench.py reports
them (it uses bench.py's own graph builder and stage-loop measurement).
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
for p in (HERE, os.path.dirname(HERE)):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--variants', default='peer_compact:1,peer_copy:1,local_first:1,feature_chunks:1:128,reference:1,reference:2,reference:4')
    ap.add_argument('--config', default='sparse2m')
    ap.add_argument('--rep', type=int, default=1)
    ap.add_argument('--layers', type=int, default=0)
    ap.add_argument('--steps', type=int, default=4)
    ap.add_argument('--widths', default='256,100,47')
    a = ap.parse_args()
    import torch.distributed as dist
    import torch.nn as nn
    import bench
    import spmm_cpp
    from coo_graph import synthetic
    from dist_train import local_loss
    from dist_utils import DistEnv
    from models import GCN
    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29711')
    os.environ.setdefault('DIST_GNN_LOG_ROOT', '/tmp/dist_gnn_bench_logs')
    if world < 2:
        raise SystemExit('stage_sweep compares multi-GPU schedules: launch it with torch.distributed.run on 2 or more GPUs')
    args = argparse.Namespace(config=a.config, layers=a.layers, seed=0, no_permute=False, rep=a.rep, gpus=world)
    env = DistEnv(rank, world, 'nccl', rep=a.rep)
    cfg = bench.workload_config(args)
    g = bench.build_rank_graph(cfg, args, env)
    dims = [cfg['feat_dim']] + [cfg['hidden']] * (cfg['layers'] - 1) + [cfg['num_classes']]
    model = GCN(g, env, hidden_dim=cfg['hidden'], num_layers=cfg['layers'], weights=synthetic.glorot_weights(dims, 0))
    optimizer = torch.optim.Adam(model.parameters(), lr=0.01)
    loss_func = nn.CrossEntropyLoss()

    def step():
        out = model(g.features)
        optimizer.zero_grad()
        loss = local_loss(g, out, loss_func)
        loss.backward()
        optimizer.step()
        return loss

    def fence():
        torch.cuda.synchronize()
        env.barrier_all()
        torch.cuda.synchronize()

    for variant in a.variants.split(','):
        parts = variant.split(':')
        env.stage_order, env.stage_group = parts[0], int(parts[1])
        if len(parts) > 2:
            env.chunk_width = int(parts[2])
        for _ in range(3):
            step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fence()
        e0.record()
        for _ in range(a.steps):
            loss = step()
        e1.record()
        fence()
        t = torch.tensor([e0.elapsed_time(e1) / a.steps], dtype=torch.float64, device=env.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=env.world_group)
        info = bench.measure_stage_loops(env, g, [int(w) for w in a.widths.split(',')], spmm_cpp)
        if rank == 0:
            print(json.dumps({'variant': variant, 'ranks': world, 'rep': a.rep, 'epoch_ms': round(t.item(), 3),
                              'loss': round(loss.item(), 6), 'loops': info}), flush=True)
    env.shutdown()


if __name__ == '__main__':
    main()
