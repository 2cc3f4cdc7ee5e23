"""Benchmark of the broadcast-SpMM GCN epoch on the synthetic 2,449,029-node graph.

    python bench.py --gpus 1 --steps K --warmup W                 (one GPU)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...                          (the reference's CPU path, host cores)

A step is one training epoch as light_dist_gnn/dist_train.py:36-45 runs it: forward through the L DistGCNLayers
(2L distributed SpMMs per epoch counting backward), cross-entropy over the local train rows, backward, Adam.  The
graph, labels and split are regenerated from a seed on every rank (integer hash, identical everywhere); the same
total problem is split over N ranks, so scaling is "strong".  Rank 0 prints ONE JSON line.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, 'dist-gnn_b200')
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

METRIC, UNIT = 'gcn_epoch_ms', 'ms'
CPU_SAMPLE_PARTS = 16     # the CPU legs time one rank's share of a 16-way 1D row partition and scale by 16
DRAM_BYTES_PER_ENTRY_FLOAT = 1.57    # measured DRAM traffic of a product per (stored entry x float of width), see roofline


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--config', default='sparse2m', help='key of coo_graph.synthetic.CONFIGS')
    ap.add_argument('--rep', type=int, default=1, help='1.5D replication factor (1 = plain 1D)')
    ap.add_argument('--layers', type=int, default=0, help='override the number of GCN layers')
    ap.add_argument('--seed', type=int, default=0)
    ap.add_argument('--stage-group', type=int, default=0, help='stages fused into one product (0 = the default of DistEnv)')
    ap.add_argument('--stage-order', default=None, choices=['reference', 'local_first', 'feature_chunks', 'peer_copy', 'peer_compact'],
                    help='order of the products inside a distributed SpMM (default: that of DistEnv)')
    ap.add_argument('--chunk-width', type=int, default=0, help='column chunk width of the feature_chunks order (0 = default 64)')
    ap.add_argument('--dense', default=None, choices=['fp32', '3xtf32', 'tcgen05'],
                    help='dense transform: fp32 library GEMM, or three tensor-core TF32 passes with fp32 accumulation')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--profiler-range', action='store_true',
                    help='cudaProfilerStart/Stop around the device-resident timed steps (for ncu --profile-from-start off)')
    ap.add_argument('--no-permute', action='store_true', help='keep the raw R-MAT vertex order (skewed row blocks)')
    return ap.parse_args()


def workload_config(args):
    from coo_graph import synthetic
    cfg = dict(synthetic.CONFIGS[args.config])
    if args.layers:
        cfg['layers'] = args.layers
    return cfg


def describe(cfg, args, world):
    return (f"{args.config}: seeded R-MAT {cfg['num_nodes']:,} nodes / {cfg['directed_edges']:,} directed edges "
            f"(+self loops, sym-normalised fp32), {cfg['feat_dim']}-dim N(0,1) features, {cfg['num_classes']} classes, "
            f"{cfg['layers']}-layer GCN hidden {cfg['hidden']}, "
            + (f"1D row partition over {world} rank(s)" if args.rep == 1 else f"1.5D partition, {world} ranks, replication {args.rep}"))


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    FIELDS = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
              'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index):
        self.proc, self.gpu = None, gpu_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.gpu), f'--query-gpu={self.FIELDS}',
                                          '--format=csv,noheader,nounits', '-lms', '200'],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.summary = {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': [], 'samples': 0}
        if self.proc is None:
            return
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap')
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(',')]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])), mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith('active'):
                    reasons.add(name)
        if sm:
            self.summary = {'sm_mhz': statistics.median(sm), 'sm_max_mhz': max(mx), 'reasons': sorted(reasons), 'samples': len(sm)}


# ------------------------------------------------------------------------------------------------ our arm
def build_rank_graph(cfg, args, env):
    """This rank's Parted_COO_Graph, built in device memory from the seed; also the host copy of its feature block."""
    from coo_graph import COO_Graph, Parted_COO_Graph, synthetic
    dev = env.device
    d = synthetic.make_dataset(seed=args.seed, permute=not args.no_permute, device=dev, **cfg)
    full = COO_Graph.from_dict(args.config, d, device=dev)
    del d
    parts = env.world_size // env.rep
    g = Parted_COO_Graph.from_full(full, env.rank // env.rep, parts)
    g.adj = None                      # the stage loop only needs adj_parts; drop the joined copy and the full graph
    del full
    torch.cuda.empty_cache()
    return g


def run_ours(args):
    import torch.distributed as dist
    import torch.nn as nn
    import spmm_cpp
    from coo_graph import synthetic
    from dist_train import local_loss
    from dist_utils import DistEnv
    from models import GCN

    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29555')
    os.environ.setdefault('DIST_GNN_LOG_ROOT', '/tmp/dist_gnn_bench_logs')
    if world != args.gpus:
        raise SystemExit(f'--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}')
    if not torch.cuda.is_available():
        raise SystemExit('bench.py (impl ours) needs CUDA devices; there is no CPU path')
    env = DistEnv(rank, world, 'nccl', rep=args.rep, stage_group=args.stage_group or None, stage_order=args.stage_order)
    if args.chunk_width:
        env.chunk_width = args.chunk_width
    import models.gcn as gcn_module
    if args.dense:
        gcn_module.DENSE_MODE = args.dense
    cfg = workload_config(args)
    g = build_rank_graph(cfg, args, env)
    dims = [cfg['feat_dim']] + [cfg['hidden']] * (cfg['layers'] - 1) + [cfg['num_classes']]
    model = GCN(g, env, hidden_dim=cfg['hidden'], num_layers=cfg['layers'], weights=synthetic.glorot_weights(dims, args.seed))
    optimizer = torch.optim.Adam(model.parameters(), lr=0.01)
    loss_func = nn.CrossEntropyLoss()
    feat_host = g.features.cpu().pin_memory()            # e2e leg: the inputs start in pinned host memory

    def epoch_step():
        outputs = model(g.features)
        optimizer.zero_grad()
        loss = local_loss(g, outputs, loss_func)
        loss.backward()
        optimizer.step()
        return loss

    def fence():
        torch.cuda.synchronize()
        env.barrier_all()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        t = torch.tensor([x], dtype=torch.float64, device=env.device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=env.world_group)
        return float(t.item())

    for _ in range(max(args.warmup, 3)):
        epoch_step()
    # ---- device-resident leg: K epochs, inputs in HBM, CUDA events, max over ranks -------------------------------------
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fence()
    with ClockSampler(env.device.index) as clocks:
        spmm_cpp.profile_begin()
        if args.profiler_range:
            torch.cuda.profiler.start()
        ev0.record()
        for _ in range(args.steps):
            loss = epoch_step()
        ev1.record()
        fence()
        if args.profiler_range:
            torch.cuda.profiler.stop()
        prof = spmm_cpp.profile_end()
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    final_loss = float(loss.item())
    # ---- end-to-end leg: host features -> device, epoch, loss back to the host, every step ------------------------------
    # Every step's input is copied from pinned host memory inside the timed region (K copies for K steps) and its loss is
    # read back.  The copies go through two device buffers on a copy stream, as an input pipeline does: step i+1's
    # features cross PCIe while step i computes; only the first copy is exposed.
    fence()
    copy_stream = torch.cuda.Stream(device=env.device)
    bufs = [g.features, torch.empty_like(g.features)]
    arrived = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]

    def prefetch(i):
        b = i % 2
        with torch.cuda.stream(copy_stream):
            if i >= 2:
                copy_stream.wait_event(consumed[b])          # step i-2 (forward and backward) is done with this buffer
            bufs[b].copy_(feat_host, non_blocking=True)
            arrived[b].record(copy_stream)

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    copy_stream.wait_event(e0)
    prefetch(0)
    for i in range(args.steps):
        b = i % 2
        torch.cuda.current_stream().wait_event(arrived[b])
        g.features = bufs[b]
        if i + 1 < args.steps:
            prefetch(i + 1)
        loss_value = epoch_step().item()
        consumed[b].record()
    e1.record()
    fence()
    g.features = bufs[0]
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    # ---- per-stage-loop communication numbers (N > 1): one timed distributed SpMM per width ---------------------------
    comm_info = None
    if env.col_comm is not None:
        comm_info = measure_stage_loops(env, g, sorted(set(dims)), spmm_cpp)

    # per-rank product time: report the slowest rank's (it sets the epoch time)
    gathered = env.all_gather_object(prof) if world > 1 else [prof]
    slow = max(gathered, key=lambda p: p['spmm_ms'])
    launches = sum(int(p['kernel_launches']) + int(p.get('dense_launches', 0)) for p in gathered)   # SpMM + dense kernels of this library
    peaks = load_peaks()
    achieved = slow['alg_bytes'] / (slow['spmm_ms'] * 1e-3) / 1e9 if slow['spmm_ms'] > 0 else 0.0
    line = {
        'metric': METRIC, 'value': round(ms_total / args.steps, 4), 'unit': UNIT, 'n_gpus': world, 'steps': args.steps,
        'warmup': max(args.warmup, 3), 'ms_per_step': round(ms_total / args.steps, 4), 'higher_is_better': False,
        'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': describe(cfg, args, world), 'cache': 'inputs larger than L2 (adjacency + operands are GBs per rank); no flush',
                   'partition': '1d' if args.rep == 1 else f'1.5d(c={args.rep})', 'seed': args.seed,
                   'vertex_permutation': not args.no_permute, 'final_loss': round(final_loss, 6),
                   'stage_order': env.stage_order, 'stage_group': env.stage_group, 'dense': gcn_module.DENSE_MODE},
        'roofline': {'bound': 'hbm', 'achieved': round(achieved, 2), 'peak': peaks['hbm_gbs'], 'unit': 'GB/s',
                     'frac': round(achieved / peaks['hbm_gbs'], 4),
                     # ncu on the 1 M-node / degree-48 / F=256 product: 20.65 GB of DRAM traffic for 51.38 M entries x 256
                     # floats = 1.57 B per (entry x float); scaled here by this run's sum of nnz x F (= flops / 2), per step
                     'traffic': round(DRAM_BYTES_PER_ENTRY_FLOAT * slow['flops'] / 2 / args.steps),
                     'traffic_source': 'scaled from profiles/k_spmm_rows_v4_rmat1m_deg48_f256.md by nnz x F; per step, all products',
                     'peak_source': peaks['source'],
                     'kernel': 'k_spmm_rows_v4 + k_spmm_chunks_v4 (+ generic row kernels for odd widths), all local products of the slowest rank',
                     'products_per_step': slow['products'] // args.steps, 'spmm_ms_per_step': round(slow['spmm_ms'] / args.steps, 4),
                     'alg_bytes_per_step': slow['alg_bytes'] / args.steps,
                     'gather_gbs': round(slow['gather_bytes'] / (slow['spmm_ms'] * 1e-3) / 1e9, 2) if slow['spmm_ms'] > 0 else 0.0,
                     'gflops': round(slow['flops'] / (slow['spmm_ms'] * 1e-3) / 1e9, 2) if slow['spmm_ms'] > 0 else 0.0},
        'e2e': {'value': round(e2e_ms, 4), 'unit': UNIT, 'h2d_bytes_per_step': feat_host.numel() * 4, 'd2h_bytes_per_step': 4,
                'input_pipeline': 'two device buffers: the copy of step i+1 overlaps step i'},
        'gpu_launches': launches,
        'clocks': clocks.summary,
    }
    if comm_info is not None:
        line['comm'] = comm_info
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        line['cpu_baseline'] = cpu_baseline_from_device(cfg, args, g_single=g, steps=1)
    if rank == 0:
        print(json.dumps(line), flush=True)
    env.shutdown()


def measure_stage_loops(env, g, widths, spmm_cpp):
    """One timed distributed SpMM per width: broadcast bus GB/s, product time, and how much of the shorter of the two
    was hidden under the other:  overlap = (t_comm + t_spmm - t_loop) / min(t_comm, t_spmm)."""
    import torch.distributed as dist
    from models.gcn import group_plans, ordered_products
    stages = env.stages()
    group = min(env.stage_group, len(stages))
    roots = [st.root_in_group for st in stages]
    n = g.local_num_nodes
    out = {'stage_group': group, 'stage_order': env.stage_order}
    from models import gcn as gcn_module
    for true_width in widths:
        # the model pads operand rows to a multiple of 4 floats before the stage loop; measure what it runs
        width = true_width + (-true_width) % 4 if gcn_module.PAD_ODD_WIDTHS else true_width
        x = torch.randn(n, width, device=env.device)
        z = torch.empty_like(x)
        for timed in (False, True):
            gcn_module._stage_loop(env, g.adj_parts, x, z, stages, env.col_comm, timed=timed)     # the model's own dispatcher
            torch.cuda.synchronize()
        t = env.col_comm.last_times()
        vals = torch.tensor([t['comm_ms'], t['spmm_ms'], t['total_ms']], dtype=torch.float64, device=env.device)
        dist.all_reduce(vals, op=dist.ReduceOp.MAX, group=env.world_group)
        comm_ms, spmm_ms, total_ms = vals.tolist()
        received = sum(1 for st in stages if st.root_in_group != env.col_comm.rank) * n * width * 4
        moved = received if env.stage_order == 'peer_copy' else len(stages) * n * width * 4     # peer copies move remote blocks only
        if env.stage_order == 'peer_compact' and env.rep == 1:
            moved = received = sum(gcn_module.compact_exchange(env, g.adj_parts, stages)['stage_rows']) * width * 4
        out[f'F{true_width}'] = {
            'width_on_the_wire': width,
            'bcast_bus_gbs': round(moved / (comm_ms * 1e-3) / 1e9, 2) if comm_ms > 0 else None,
            'bcast_frac_of_900': round(moved / (comm_ms * 1e-3) / 1e9 / 900.0, 4) if comm_ms > 0 else None,
            'comm_ms': round(comm_ms, 4), 'spmm_ms': round(spmm_ms, 4), 'loop_ms': round(total_ms, 4),
            'overlap': round((comm_ms + spmm_ms - total_ms) / max(min(comm_ms, spmm_ms), 1e-9), 4),
            'received_bytes': received,
        }
    return out


def load_peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            return {'hbm_gbs': float(json.load(f)['hbm_gbs']), 'source': 'measured (MEASURED_PEAKS.json)'}
    return {'hbm_gbs': 6650.0, 'source': 'fallback (earlier measurement on this pool)'}


# ------------------------------------------------------------------------------------------------ CPU legs
def cpu_sample_inputs(cfg, args, device):
    """Row block 0 of a CPU_SAMPLE_PARTS-way 1D partition of the benchmark graph as CPU tensors, made on the GPU when
    there is one (seconds) and on the host otherwise (minutes)."""
    from coo_graph import COO_Graph, synthetic
    d = synthetic.make_dataset(seed=args.seed, permute=not args.no_permute, device=device, **cfg)
    full = COO_Graph.from_dict(args.config, d, device=device)
    part = full.part_dict(0, CPU_SAMPLE_PARTS)
    n = part['adj'].size(0)
    a = part['adj'].cpu().coalesce()
    # the partition pads the column count to CPU_SAMPLE_PARTS * n; the padding columns hold no entry, the features have N rows
    adj = torch.sparse_coo_tensor(a.indices(), a.values(), (n, full.features.size(0)), is_coalesced=True)
    return dict(adj=adj, x=full.features.cpu(), labels=full.labels[:n].cpu(), mask=full.train_mask[:n].cpu(), n=n)


def time_cpu_sample(inp, cfg, args, steps, warmup=0):
    from coo_graph import synthetic
    from oracle import ref_gcn
    threads = os.cpu_count() or 1
    dims = [cfg['feat_dim']] + [cfg['hidden']] * (cfg['layers'] - 1) + [cfg['num_classes']]
    weights = synthetic.glorot_weights(dims, args.seed)
    times = []
    for i in range(warmup + steps):
        sec, _ = ref_gcn.cpu_epoch_sample(inp['adj'], inp['x'], inp['labels'], inp['mask'], weights, threads)
        if i >= warmup:
            times.append(sec)
    return times, threads


def cpu_baseline_from_device(cfg, args, g_single, steps):
    """cpu_baseline leg of the N=1 run: the oracle's torch-CPU epoch on a bounded sample, scaled to a full epoch."""
    n = (cfg['num_nodes'] + CPU_SAMPLE_PARTS - 1) // CPU_SAMPLE_PARTS
    A = g_single.adj_parts[0]                          # P = 1: the whole normalised adjacency, on the device
    idx, val = A.indices(), A.values()
    hi = int(torch.searchsorted(idx[0].contiguous(), torch.tensor([n], device=idx.device)).item())
    adj = torch.sparse_coo_tensor(idx[:, :hi].cpu(), val[:hi].cpu(), (n, A.size(1)), is_coalesced=True)
    inp = dict(adj=adj, x=g_single.features.cpu(), labels=g_single.local_labels[:n].cpu(), mask=g_single.local_train_mask[:n].cpu(), n=n)
    times, threads = time_cpu_sample(inp, cfg, args, steps)
    ms = statistics.median(times) * 1e3 * CPU_SAMPLE_PARTS
    return {'value': round(ms, 1), 'unit': UNIT, 'cores': threads, 'kind': 'port', 'sample': cpu_sample_text(n, cfg, len(times))}


def cpu_sample_text(n, cfg, steps):
    return (f'oracle torch-CPU epoch (addmm_ sparse path + mm + CE + Adam) of rank 0 of a {CPU_SAMPLE_PARTS}-way 1D row partition '
            f"({n:,} of {cfg['num_nodes']:,} rows, all columns, no communication), median of {steps} run(s), ms x {CPU_SAMPLE_PARTS}")


def run_reference(args):
    """The reference's CPU path (its torch.sparse addmm_ stage products, dense mm, CE, Adam) on the host cores, through
    the oracle port: the reference's own files cannot travel to the GPU box."""
    rank = int(os.environ.get('RANK', 0))
    if rank != 0:
        return
    cfg = workload_config(args)
    device = 'cuda' if torch.cuda.is_available() else 'cpu'
    inp = cpu_sample_inputs(cfg, args, device)
    if device == 'cuda':
        torch.cuda.empty_cache()
    steps, warmup = min(args.steps, 3), min(args.warmup, 1)
    times, threads = time_cpu_sample(inp, cfg, args, steps, warmup)
    ms = sum(times) / len(times) * 1e3 * CPU_SAMPLE_PARTS
    world = int(os.environ.get('WORLD_SIZE', 1))
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': round(ms, 1), 'unit': UNIT, 'n_gpus': world, 'steps': steps, 'warmup': warmup,
        'ms_per_step': round(ms, 1), 'higher_is_better': False, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32',
        'data': 'synthetic', 'config': {'workload': describe(cfg, args, world), 'partition': '1d' if args.rep == 1 else f'1.5d(c={args.rep})',
                                        'seed': args.seed, 'vertex_permutation': not args.no_permute},
        'cpu_baseline': {'value': round(ms, 1), 'unit': UNIT, 'cores': threads, 'kind': 'port', 'sample': cpu_sample_text(inp['n'], cfg, steps)},
        'e2e': {'value': round(ms, 1), 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line), flush=True)


if __name__ == '__main__':
    a = parse()
    if a.impl == 'reference':
        run_reference(a)
    else:
        run_ours(a)
