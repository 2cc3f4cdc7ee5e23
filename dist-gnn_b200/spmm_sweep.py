"""Standalone distributed SpMM sweep: seeded R-MAT adjacency x dense fp32 operand, 1D broadcast-SpMM.

    python dist-gnn_b200/spmm_sweep.py --nodes 1000000 --degree 16 --widths 16,64,256,512 --iters 5
    python -m torch.distributed.run --nproc-per-node N ... dist-gnn_b200/spmm_sweep.py ...      (N ranks, one per GPU)
    python dist-gnn_b200/spmm_sweep.py --nodes 2449029 --edges 123718280 --widths 256 --block-of 8 [--packed]
        (one GPU: the products of rank 0 of an 8-rank partition, accumulating - what a stage loop runs between its
         transfers; --packed multiplies by the rows each block touches, as the compact peer loop does; --stage-group 4,2,1
         joins the remote blocks into products of 4, 2 and 1 arrivals)

The graph is the symmetrically normalised adjacency (self loops added) of a seeded R-MAT graph with `nodes` vertices and
about nodes * degree directed edges, built on the device.  For every width it prints one JSON line (the slowest rank's
figures): device time of the local products (CUDA events around every product), algorithmic GB/s
(8*nnz + 4*(m+1) + 4*F*touched + 4*F*m*(1+[beta!=0])) / t  against the measured HBM peak, the no-reuse gather GB/s, and
with more than one rank the transfer bus GB/s and the transfer/compute overlap of the stage loop the environment
selects (the model's own dispatcher).  Before the timings, a sample of rows of the distributed product is compared with a
float64 evaluation (dist_utils.selfcheck).  The same command with small sizes is what the profiler captures use.
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
    ap.add_argument('--nodes', type=int, default=1_000_000)
    ap.add_argument('--degree', type=int, default=16, help='average directed degree before self loops')
    ap.add_argument('--edges', type=int, default=0, help='directed edges (overrides nodes * degree)')
    ap.add_argument('--block-of', type=int, default=0, help='one GPU: time the stage products of rank 0 of this many ranks')
    ap.add_argument('--packed', action='store_true', help='with --block-of: operands hold only the rows each block touches')
    ap.add_argument('--widths', default='16,64,256,512')
    ap.add_argument('--iters', type=int, default=5)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--seed', type=int, default=0)
    ap.add_argument('--no-permute', action='store_true')
    ap.add_argument('--stage-order', default=None)
    ap.add_argument('--stage-group', default=None)
    ap.add_argument('--profiler-range', action='store_true', help='cudaProfilerStart/Stop around the timed products')
    args = ap.parse_args()

    import spmm_cpp
    from coo_graph import graph_utils, synthetic
    from dist_utils import DistEnv
    from dist_utils.selfcheck import sampled_rows_check
    from models import gcn
    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29556')
    os.environ.setdefault('DIST_GNN_LOG_ROOT', '/tmp/dist_gnn_bench_logs')
    env = DistEnv(rank, world, 'nccl', stage_order=args.stage_order, stage_group=args.stage_group)
    dev = env.device
    N = args.nodes
    ei = synthetic.rmat_edge_index(N, args.edges or N * args.degree, args.seed, permute=not args.no_permute, device=dev)
    A = graph_utils.sym_normalization(ei, N)
    del ei
    if args.block_of:
        if world != 1:
            raise SystemExit('--block-of emulates a rank of a larger partition on ONE GPU')
        emulate_rank(args, env, A, spmm_cpp, graph_utils)
        env.shutdown()
        return
    n = (N + world - 1) // world
    row_block = graph_utils.sparse_2d_split(A, n, split_dim=0)[rank]
    del A
    torch.cuda.empty_cache()
    row_block = graph_utils._coo(row_block.indices(), row_block.values(), (n, n * world))
    parts = graph_utils.sparse_2d_split(row_block, n, split_dim=1)
    stages = env.stages()
    peak = 6546.9
    peaks_file = os.path.join(os.path.dirname(HERE), 'MEASURED_PEAKS.json')
    if os.path.exists(peaks_file):
        with open(peaks_file) as f:
            peak = float(json.load(f)['hbm_gbs'])
    widths = [int(w) for w in args.widths.split(',')]
    check = sampled_rows_check(env, row_block, parts, [w for w in widths if w <= 256][-1:] or widths[:1])
    for width in widths:
        x = torch.randn(n, width, device=dev)
        z = torch.empty(n, width, device=dev)
        line = {'nodes': N, 'degree': args.degree, 'width': width, 'ranks': world, 'nnz_rank': int(row_block.values().numel()),
                'stage_order': env.stage_order if world > 1 else None, 'check_max_rel': check['max_rel'], 'check_ok': check['ok']}
        for _ in range(args.warmup):
            gcn._stage_loop(env, parts, x, z, stages, env.col_comm)
        torch.cuda.synchronize()
        env.barrier_all()
        spmm_cpp.profile_begin()
        if args.profiler_range:
            torch.cuda.profiler.start()
        for i in range(args.iters):
            gcn._stage_loop(env, parts, x, z, stages, env.col_comm, timed=(world > 1 and i == args.iters - 1))
        if args.profiler_range:
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        prof = spmm_cpp.profile_end()
        if world > 1:
            t = env.col_comm.last_times()
            moved = (world - 1) * n * width * 4
            if env.stage_order in ('peer_compact', 'peer_gather'):
                moved = sum(gcn.compact_exchange(env, parts, stages, owner_packs=env.stage_order == 'peer_compact')['stage_rows']) * width * 4
            line.update(moved_bytes=moved, bus_gbs=round(moved / (t['comm_ms'] * 1e-3) / 1e9, 2) if t['comm_ms'] > 0 else None,
                        comm_ms=round(t['comm_ms'], 4), loop_ms=round(t['total_ms'], 4), loop_spmm_ms=round(t['spmm_ms'], 4),
                        overlap=round((t['comm_ms'] + t['spmm_ms'] - t['total_ms']) / max(min(t['comm_ms'], t['spmm_ms']), 1e-9), 4))
        sec = max(prof['spmm_ms'] * 1e-3, 1e-12)
        line.update(spmm_ms=round(prof['spmm_ms'] / args.iters, 4), alg_gbs=round(prof['alg_bytes'] / sec / 1e9, 2),
                    frac_of_hbm_peak=round(prof['alg_bytes'] / sec / 1e9 / peak, 4), gather_gbs=round(prof['gather_bytes'] / sec / 1e9, 2),
                    gflops=round(prof['flops'] / sec / 1e9, 2), kernel_launches=prof['kernel_launches'])
        every = env.all_gather_object(line) if world > 1 else [line]
        if rank == 0:
            print(json.dumps(max(every, key=lambda l: l['spmm_ms'])), flush=True)
        del x, z
    env.shutdown()
    if not check['ok']:
        raise SystemExit(f'self-check failed: {check}')


def emulate_rank(args, env, A, spmm_cpp, graph_utils):
    """The local products rank 0 of a --block-of P partition runs in one distributed SpMM: block s multiplies operand s,
    the first overwrites z, the others accumulate.  No transfers (the operands are local random blocks)."""
    P, dev, N = args.block_of, env.device, A.size(0)
    n = (N + P - 1) // P
    row_block = graph_utils.sparse_2d_split(A, n, split_dim=0)[0]
    del A
    row_block = graph_utils._coo(row_block.indices(), row_block.values(), (n, n * P))
    parts = graph_utils.sparse_2d_split(row_block, n, split_dim=1)
    del row_block
    from models.gcn import group_sizes
    plans, rows_of = [spmm_cpp.SpmmPlan.from_coo(parts[0])], [n]         # the rank's own block, read in place
    spec = [int(v) for v in str(args.stage_group or 1).split(',')]
    first = 1
    for count in group_sizes(P - 1, spec if len(spec) > 1 else spec[0]):   # remote blocks, `count` arrivals per product
        row, col, val, base = [], [], [], 0
        for block in parts[first:first + count]:
            idx = block.indices()
            if args.packed:              # column ids become positions in the ascending list of touched columns
                touched = torch.unique(idx[1])
                row.append(idx[0]); col.append(torch.searchsorted(touched, idx[1].contiguous()) + base); val.append(block.values())
                base += int(touched.numel())
            else:
                row.append(idx[0]); col.append(idx[1] + base); val.append(block.values())
                base += n
        row, col, val = torch.cat(row), torch.cat(col), torch.cat(val)
        if count > 1:
            order = torch.sort(row * base + col).indices
            row, col, val = row[order], col[order], val[order]
        plans.append(spmm_cpp.SpmmPlan(row.to(torch.int32), col.to(torch.int32).contiguous(), val.contiguous(), n, base))
        rows_of.append(base)
        first += count
    del parts
    torch.cuda.empty_cache()
    for width in (int(w) for w in args.widths.split(',')):
        xs = [torch.randn(r, width, device=dev) for r in rows_of]
        z = torch.empty(n, width, device=dev)

        def loop():
            for s, plan in enumerate(plans):
                plan.spmm(xs[s], z, 1.0, 0.0 if s == 0 else 1.0)
        for _ in range(args.warmup):
            loop()
        torch.cuda.synchronize()
        spmm_cpp.profile_begin()
        if args.profiler_range:
            torch.cuda.profiler.start()
        for _ in range(args.iters):
            loop()
        if args.profiler_range:
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        prof = spmm_cpp.profile_end()
        sec = max(prof['spmm_ms'] * 1e-3, 1e-12)
        print(json.dumps({'nodes': N, 'emulated_rank': f'0 of {P}', 'packed': bool(args.packed), 'width': width, 'products': len(plans),
                          'operand_rows': rows_of, 'nnz_rank': sum(p.stats()['nnz'] for p in plans),
                          'spmm_ms': round(prof['spmm_ms'] / args.iters, 4), 'alg_bytes': prof['alg_bytes'] / args.iters,
                          'gather_gbs': round(prof['gather_bytes'] / sec / 1e9, 2), 'alg_gbs': round(prof['alg_bytes'] / sec / 1e9, 2)}), flush=True)
        del xs, z


if __name__ == '__main__':
    main()
