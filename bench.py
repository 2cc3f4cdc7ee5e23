"""Benchmark of the broadcast-SpMM GCN epoch on the synthetic 2,449,029-node graph.

    python bench.py --gpus 1 --steps K --warmup W                 (one GPU)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...                          (the reference's CPU path, host cores)

A step is one training epoch as light_dist_gnn/dist_train.py:36-45 runs it: forward through the L DistGCNLayers
(2L distributed SpMMs per epoch counting backward), cross-entropy over the local train rows, backward, Adam.  The
graph, labels and split are regenerated from a seed on every rank (integer hash, identical everywhere); the same
total problem is split over N ranks, so scaling is "strong".  Rank 0 prints ONE JSON line.  Beside the contract's keys it
carries `parity` (the distributed product of the active schedule against a float64 evaluation of sampled rows; the run
exits non-zero above 1e-5), `reuse` (the same epochs with the constant first-layer product kept), `comm` (N > 1) and
`run` (schedule, median epoch).  A default 8-GPU run also carries `config3`: the same graph under the 1.5D partition (c = 2,
4 layers), measured afterwards by the same processes.  `--impl reference` runs the unmodified reference from baseline/_ref over gloo.
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
# DRAM traffic of the local products (dram__bytes_read + dram__bytes_write, ncu, one pass, --clock-control none):
#   the N = 1 default workload itself, one epoch of `bench.py --steps 1 --warmup 3 --no-cpu-baseline --profiler-range`:
#   128.18 GB for 147.87 G (stored entry x float) = 0.867 B each;
#   the 8 products of one distributed SpMM of rank 0 of 8 at F = 256 (spmm_sweep.py --block-of 8): 6.41 GB for 4.02 G = 1.594 B each.
MEASURED_TRAFFIC = {('sparse2m', 1, 3): 128.18e9}     # (config, ranks, layers) -> bytes per step, captured on that very workload
TRAFFIC_PER_ENTRY_FLOAT = {'whole_graph': 0.867, 'stage_blocks': 1.594}
CONFIG3_DEADLINE_S = 150      # the extra 1.5D measurement of an 8-GPU default run gives up after this long (it takes about 20 s)


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
    ap.add_argument('--stage-group', default=None, help='stages fused into one product: a number, or for peer_compact a size list such as 4,2,1 (default: that of DistEnv)')
    ap.add_argument('--stage-order', default=None, choices=['reference', 'local_first', 'feature_chunks', 'peer_copy', 'peer_compact', 'peer_gather'],
                    help='order of the products inside a distributed SpMM (default: that of DistEnv)')
    ap.add_argument('--chunk-width', type=int, default=0, help='column chunk width of the feature_chunks order (0 = default 64)')
    ap.add_argument('--dense', default=None, choices=['fp32', '3xtf32', 'tcgen05'],
                    help='dense transform: fp32 library GEMM, or three tensor-core TF32 passes with fp32 accumulation')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-config3', action='store_true', help='8 GPUs, default workload: do not also measure the 1.5D c = 2, 4-layer configuration')
    ap.add_argument('--then-rep', type=int, default=0, help='measure a second layout afterwards in the same processes: its replication factor')
    ap.add_argument('--then-layers', type=int, default=0, help='... and its number of layers (0 = as the first)')
    ap.add_argument('--cpu-sample-divisor', type=int, default=8,
                    help='the CPU legs run a graph with 1/D of the nodes and edges and scale by the stored entries (1 = the full graph)')
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
    del full                          # g.adj (the rank's whole row block) stays: the parity check reads sampled rows of it
    torch.cuda.empty_cache()
    return g


def run_ours(args):
    """The default workload (or the one the flags name); on 8 GPUs with no workload flags, the 1.5D c = 2, 4-layer
    configuration of the same graph is measured afterwards in the same processes and reported under `config3`
    (--then-rep / --then-layers ask for such a second measurement by hand; it is reported under `second`)."""
    import threading
    rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29555')
    os.environ.setdefault('DIST_GNN_LOG_ROOT', '/tmp/dist_gnn_bench_logs')
    if world != args.gpus:
        raise SystemExit(f'--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}')
    if not torch.cuda.is_available():
        raise SystemExit('bench.py (impl ours) needs CUDA devices; there is no CPU path')
    also_15d = (world == 8 and args.config == 'sparse2m' and args.rep == 1 and not args.layers and args.stage_order is None
                and args.stage_group is None and not args.profiler_range and not args.no_config3 and not args.then_rep)
    key, then_rep, then_layers = ('config3', 2, 4) if also_15d else ('second', args.then_rep, args.then_layers or args.layers)
    also_15d = also_15d or args.then_rep > 0
    line, ok = measure(args, rank, world, keep_process_group=also_15d)
    failed = None if ok else f"parity check failed: {line['parity']}"
    if also_15d:
        # Nothing below may cost the main line: a deadline prints it with an error note and leaves, an exception is recorded.
        claim = threading.Lock()

        def give_up():
            if claim.acquire(blocking=False):
                if rank == 0:
                    line[key] = {'error': f'no result within {CONFIG3_DEADLINE_S} s'}
                    print(json.dumps(line), flush=True)
                os._exit(0 if ok else 1)
        watchdog = threading.Timer(CONFIG3_DEADLINE_S, give_up)
        watchdog.daemon = True
        watchdog.start()
        clean = True
        try:
            sub = argparse.Namespace(**vars(args))
            sub.rep, sub.layers, sub.no_cpu_baseline = then_rep, then_layers, True
            import gc
            import models.gcn as gcn_module
            gcn_module.drop_cached_plans()
            gc.collect()
            torch.cuda.empty_cache()
            other, ok3 = measure(sub, rank, world, keep_process_group=False)
            line[key] = {k: other[k] for k in ('value', 'unit', 'steps', 'warmup', 'config', 'run', 'parity', 'e2e') if k in other}
            line[key]['roofline'] = {k: other['roofline'][k] for k in ('achieved', 'peak', 'unit', 'frac', 'spmm_ms_per_step', 'products_per_step')}
            if 'comm' in other:
                line[key]['comm'] = other['comm']
            if not ok3:
                failed = f"parity check failed ({key}): {other['parity']}"
        except Exception as e:      # noqa: BLE001 - recorded in the line; the ranks then leave without further collectives
            line[key] = {'error': repr(e)[:300]}
            clean = False
        if not claim.acquire(blocking=False):
            time.sleep(30)          # the deadline fired at this very moment: it prints and leaves
        watchdog.cancel()
        if rank == 0:
            print(json.dumps(line), flush=True)
        if not clean:
            os._exit(1 if failed else 0)
    elif rank == 0:
        print(json.dumps(line), flush=True)
    if failed:
        raise SystemExit(failed)


def measure(args, rank, world, keep_process_group=False):
    """One workload on the ranks of this job: returns (the JSON line as a dict, whether its parity check passed)."""
    import torch.distributed as dist
    import torch.nn as nn
    import spmm_cpp
    from coo_graph import synthetic
    from dist_train import local_loss
    from dist_utils import DistEnv
    from models import GCN

    env = DistEnv(rank, world, 'nccl', rep=args.rep, stage_group=args.stage_group, stage_order=args.stage_order)
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
        marks = [ev0]
        for _ in range(args.steps):
            loss = epoch_step()
            marks.append(torch.cuda.Event(enable_timing=True))
            marks[-1].record()
        ev1.record()
        fence()
        if args.profiler_range:
            torch.cuda.profiler.stop()
        prof = spmm_cpp.profile_end()
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    spmm_cpp.check_dense_status()                   # a dense kernel that gave up on a bounded wait voids the run
    step_ms = [a.elapsed_time(b) for a, b in zip(marks[:-1], marks[1:])]      # this rank's epochs, for the median
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
    # ---- the same epochs with the constant first-layer product reused (reported beside the like-for-like value, never as it)
    def timed_epochs(k):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        epoch_step()                                    # fills the cache / warms the changed path
        fence()
        t0.record()
        for _ in range(k):
            epoch_step()
        t1.record()
        fence()
        return max_over_ranks(t0.elapsed_time(t1)) / k

    model.cache_input_product = True
    cached_ms = timed_epochs(args.steps)
    model.input_gradient_shortcut = True
    shortcut_ms = timed_epochs(args.steps)
    model.transform_first = True
    all_ms = timed_epochs(args.steps)
    model.cache_input_product = model.input_gradient_shortcut = model.transform_first = False
    model._product = None
    # ---- per-stage-loop communication numbers (N > 1): one timed distributed SpMM per width ---------------------------
    comm_info = None
    if env.col_comm is not None:
        comm_info = measure_stage_loops(env, g, sorted(set(dims)), spmm_cpp)

    # ---- parity of the distributed product with a direct fp64 evaluation of sampled rows (outside every timed region) ----
    from dist_utils.selfcheck import sampled_rows_check
    parity = sampled_rows_check(env, g.adj, g.adj_parts, sorted({dims[1], dims[-1]}))

    # per-rank product time: report the slowest rank's (it sets the epoch time)
    gathered = env.all_gather_object(prof) if world > 1 else [prof]
    slow = max(gathered, key=lambda p: p['spmm_ms'])
    launches = sum(int(p['kernel_launches']) + int(p.get('dense_launches', 0)) for p in gathered)   # SpMM + dense kernels of this library
    peaks = load_peaks()
    traffic = MEASURED_TRAFFIC.get((args.config, world, cfg['layers'])) if args.rep == 1 else None
    achieved = slow['alg_bytes'] / (slow['spmm_ms'] * 1e-3) / 1e9 if slow['spmm_ms'] > 0 else 0.0
    line = {
        'metric': METRIC, 'value': round(ms_total / args.steps, 4), 'unit': UNIT, 'n_gpus': world, 'steps': args.steps,
        'warmup': max(args.warmup, 3), 'ms_per_step': round(ms_total / args.steps, 4), 'higher_is_better': False,
        'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': config_block(cfg, args, world),
        'run': {'final_loss': round(final_loss, 6), 'stage_order': env.stage_order, 'stage_group': env.stage_group,
                'dense': gcn_module.DENSE_MODE, 'ms_per_step_median': round(statistics.median(step_ms), 4),
                'value_is': 'mean over the K timed epochs (one event pair around all of them), max over ranks'},
        'roofline': {'bound': 'hbm', 'achieved': round(achieved, 2), 'peak': peaks['hbm_gbs'], 'unit': 'GB/s',
                     'frac': round(achieved / peaks['hbm_gbs'], 4),
                     # measured DRAM bytes of all products of one step where this very workload was captured under ncu, else
                     # null with an estimate beside it: captured bytes per (stored entry x float) x this run's nnz x F (= flops / 2)
                     'traffic': traffic,
                     'traffic_est': round(TRAFFIC_PER_ENTRY_FLOAT['whole_graph' if world == 1 else 'stage_blocks'] * slow['flops'] / 2 / args.steps),
                     'traffic_note': ('traffic: ncu dram__bytes of this workload\'s products, one epoch; ' if traffic else 'traffic: no capture of this workload; ')
                                     + 'traffic_est: captured bytes per (stored entry x float) of '
                                     + ('the whole-graph products' if world == 1 else 'the 8-rank stage-block products at F = 256') + ' x this run\'s nnz x F',
                     'peak_source': peaks['source'],
                     'kernel': 'k_spmm_v4 (+ generic row kernels for narrow widths on long rows) + k_spmm_heavy_finish, all local products of the slowest rank',
                     'products_per_step': slow['products'] // args.steps, 'spmm_ms_per_step': round(slow['spmm_ms'] / args.steps, 4),
                     'alg_bytes_per_step': slow['alg_bytes'] / args.steps,
                     'gather_gbs': round(slow['gather_bytes'] / (slow['spmm_ms'] * 1e-3) / 1e9, 2) if slow['spmm_ms'] > 0 else 0.0,
                     'gflops': round(slow['flops'] / (slow['spmm_ms'] * 1e-3) / 1e9, 2) if slow['spmm_ms'] > 0 else 0.0},
        'e2e': {'value': round(e2e_ms, 4), 'unit': UNIT, 'h2d_bytes_per_step': feat_host.numel() * 4, 'd2h_bytes_per_step': 4,
                'input_pipeline': 'two device buffers: the copy of step i+1 overlaps step i'},
        'gpu_launches': launches,
        'clocks': clocks.summary,
    }
    line['parity'] = parity
    line['reuse'] = {'cached_input_product_ms': round(cached_ms, 4), 'with_gradient_shortcut_ms': round(shortcut_ms, 4),
                     'with_transform_first_ms': round(all_ms, 4),
                     'note': 'same epochs with the first layer\'s A X kept between epochs (bit-identical losses); then with its weight '
                             'gradient also taken from that product (equal up to rounding for a symmetric adjacency); then with the last '
                             'layer computed as A (H W) too (47-wide stage loop, equal up to rounding); `value` uses none of them'}
    if comm_info is not None:
        line['comm'] = comm_info
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        ms_cpu, info = cpu_epoch(cfg, args, steps=1, warmup=1)
        line['cpu_baseline'] = dict(value=round(ms_cpu, 1), unit=UNIT, **info)
    env.shutdown(keep_process_group=keep_process_group)
    return line, bool(parity['ok'])


def measure_stage_loops(env, g, widths, spmm_cpp):
    """One timed distributed SpMM per width: broadcast bus GB/s, product time, and how much of the shorter of the two
    was hidden under the other:  overlap = (t_comm + t_spmm - t_loop) / min(t_comm, t_spmm)."""
    import torch.distributed as dist
    from models.gcn import group_plans, ordered_products
    stages = env.stages()
    group = env.stage_group
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
        if env.stage_order in ('peer_compact', 'peer_gather') and env.rep == 1:
            moved = received = sum(gcn_module.compact_exchange(env, g.adj_parts, stages, owner_packs=env.stage_order == 'peer_compact')['stage_rows']) * width * 4
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
REF_DIR = os.path.join(ROOT, 'baseline', '_ref', 'light_dist_gnn')     # unmodified copy made by __graft_entry__.build()


def sample_config(cfg, divisor):
    """The bounded CPU workload: the same generator, widths, classes, split and model, 1/divisor of the nodes and of the
    directed edges (so the average degree is kept).  The dense operands of the sample are that much smaller than the
    benchmark's and friendlier to the host's caches, which flatters the CPU side."""
    small = dict(cfg)
    small['num_nodes'] = cfg['num_nodes'] // divisor
    small['directed_edges'] = cfg['directed_edges'] // divisor // 2 * 2
    return small


def config_block(cfg, args, world):
    """The `config` object, the same in both arms."""
    return {'workload': describe(cfg, args, world), 'partition': '1d' if args.rep == 1 else f'1.5d(c={args.rep})', 'seed': args.seed,
            'vertex_permutation': not args.no_permute, 'cache': cache_note(cfg, args, world)}


def cache_note(cfg, args, world):
    """Whether one rank's share of the step's inputs exceeds the 126 MB L2 (no flush is made between timed steps)."""
    blocks = max(1, world // max(1, args.rep))
    stored = (cfg['directed_edges'] + cfg['num_nodes']) // blocks                      # entries of a rank's row block
    widest = max(cfg['feat_dim'], cfg['hidden'])
    per_rank = stored * 12 + 2 * (cfg['num_nodes'] // blocks) * widest * 4             # ids + values, an operand and a result
    if per_rank > 2 * 126e6:
        return f'inputs larger than L2 ({per_rank / 1e9:.2f} GB of adjacency + widest operand and result per rank against 126 MB); no flush'
    return f'inputs of {per_rank / 1e6:.0f} MB per rank fit in the 126 MB L2 and no flush is made: a plumbing workload, not a benchmark configuration'


def _reference_worker(rank, workdir, parts, name, warmup, steps, threads, port):
    """One gloo rank of the reference's own training flow on the host cores (child process).  Everything on the timed path
    is the reference's code: dist_utils.DistEnv, coo_graph.Parted_COO_Graph, dist_train.train -> models.GCN ->
    DistGCNLayer -> broadcast -> C.addmm_(A, B) (light_dist_gnn/main.py:9-21, dist_train.py:26-45, models/gcn.py:9-53).
    Outside its files: the rendezvous port, the thread count, and torch.cuda.synchronize made a no-op when the process
    sees no GPU (the reference's timer calls it unconditionally, dist_utils/timer.py:17-24)."""
    sys.path[:] = [workdir] + [p for p in sys.path if os.path.abspath(p or '.') not in (PKG, ROOT)]
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(parts))
    torch.set_num_threads(threads)
    if not torch.cuda.is_available():
        torch.cuda.synchronize = lambda *a, **k: None
    import dist_utils, dist_train                                   # the reference's modules (workdir is first on the path)
    from coo_graph import Parted_COO_Graph
    assert os.path.abspath(dist_train.__file__).startswith(os.path.abspath(workdir))
    env = dist_utils.DistEnv(rank, parts, 'gloo')
    g = Parted_COO_Graph(name, rank=rank, num_parts=parts, device=env.device)
    if warmup:
        dist_train.train(g, env, total_epoch=warmup)
    before = env.timer.duration_dict['epoch']
    dist_train.train(g, env, total_epoch=steps)
    keys = {k: float(v) for k, v in env.timer.duration_dict.items()}
    with open(os.path.join(workdir, f'result_{rank}.json'), 'w') as f:
        json.dump({'epoch_s': (env.timer.duration_dict['epoch'] - before) / steps, 'timer': keys, 'device': str(env.device),
                   'nnz': int(g.adj.values().numel())}, f)


def run_reference_files(cfg, args, steps, warmup):
    """Times the UNMODIFIED reference (baseline/_ref/light_dist_gnn) on the host cores over gloo on the sample workload and
    scales the epoch time to the benchmark graph by the ratio of stored entries.  Returns (ms per full epoch, info)."""
    import shutil
    import socket
    import tempfile
    import torch.multiprocessing as mp
    from coo_graph import COO_Graph, synthetic
    from coo_graph.parted_coo_graph import GraphCache
    cores = os.cpu_count() or 1
    parts = max(1, min(8, cores))
    if parts == 1:
        raise RuntimeError('the reference timer needs at least two ranks (statistics.stdev)')
    threads = max(1, cores // parts)
    small = sample_config(cfg, max(1, args.cpu_sample_divisor))
    work = tempfile.mkdtemp(prefix='dg_ref_arm_')
    try:
        pkg = os.path.join(work, 'light_dist_gnn')
        shutil.copytree(REF_DIR, pkg)                              # it writes data/ and logs_P/ beside itself
        device = 'cuda' if torch.cuda.is_available() else 'cpu'
        d = synthetic.make_dataset(seed=args.seed, permute=not args.no_permute, device=device, **small)
        full = COO_Graph.from_dict('bench_sample', d, device=device)
        nnz_sample = int(full.adj.values().numel())
        folder = os.path.join(pkg, 'data', f'bench_sample_GCN_{parts}_parts')
        os.makedirs(folder, exist_ok=True)
        for r in range(parts):                                     # the reference's part files (same keys, dtypes, layout)
            part = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in full.part_dict(r, parts).items()}
            GraphCache.save_dict(part, os.path.join(folder, f'part_{r}_of_{parts}.coo_graph'))
        del d, full
        with socket.socket() as sock:
            sock.bind(('127.0.0.1', 0))
            port = sock.getsockname()[1]
        saved = {k: os.environ.get(k) for k in ('CUDA_VISIBLE_DEVICES', 'TMPDIR')}
        os.environ['CUDA_VISIBLE_DEVICES'] = ''                    # host cores only, whatever the box has
        os.environ['TMPDIR'] = work                                # the reference's FileStore lives in the temp folder
        try:
            mp.spawn(_reference_worker, (pkg, parts, 'bench_sample', warmup, steps, threads, port), nprocs=parts, join=True)
        finally:
            for k, v in saved.items():
                if v is None:
                    os.environ.pop(k, None)
                else:
                    os.environ[k] = v
        results = [json.load(open(os.path.join(pkg, f'result_{r}.json'))) for r in range(parts)]
    finally:
        shutil.rmtree(work, ignore_errors=True)
    nnz_full = cfg['directed_edges'] + cfg['num_nodes']
    scale = nnz_full / nnz_sample
    slow = max(results, key=lambda r: r['epoch_s'])
    info = {'cores': cores, 'kind': 'reference',
            'sample': (f"unmodified light_dist_gnn (dist_train.train over gloo, {parts} ranks x {threads} thread(s), addmm_ sparse path) on a "
                       f"seeded R-MAT with 1/{max(1, args.cpu_sample_divisor)} of the nodes and edges ({small['num_nodes']:,} nodes, {nnz_sample:,} stored entries, "
                       f"same widths and model), mean of {steps} epoch(s) on the slowest rank = {slow['epoch_s'] * 1e3:.1f} ms, "
                       f"x {scale:.2f} (ratio of stored entries)"),
            'sample_epoch_ms': round(slow['epoch_s'] * 1e3, 2), 'scale': round(scale, 3),
            'reference_timer_s': {k: round(v, 3) for k, v in slow['timer'].items()}}
    return slow['epoch_s'] * 1e3 * scale, info


def run_port_sample(cfg, args, steps, warmup):
    """Fallback when the reference's files are not in baseline/_ref: the oracle's torch-CPU epoch (the calls the reference
    issues on its CPU path) of one rank's share of the sample workload, one process, all host threads."""
    from coo_graph import COO_Graph, synthetic
    from oracle import ref_gcn
    threads = os.cpu_count() or 1
    small = sample_config(cfg, max(1, args.cpu_sample_divisor))
    device = 'cuda' if torch.cuda.is_available() else 'cpu'
    d = synthetic.make_dataset(seed=args.seed, permute=not args.no_permute, device=device, **small)
    full = COO_Graph.from_dict('bench_sample', d, device=device)
    adj = full.adj.cpu().coalesce()
    dims = [cfg['feat_dim']] + [cfg['hidden']] * (cfg['layers'] - 1) + [cfg['num_classes']]
    weights = synthetic.glorot_weights(dims, args.seed)
    times = []
    for i in range(warmup + steps):
        sec, _ = ref_gcn.cpu_epoch_sample(adj, full.features.cpu(), full.labels.cpu(), full.train_mask.cpu(), weights, threads)
        if i >= warmup:
            times.append(sec)
    scale = (cfg['directed_edges'] + cfg['num_nodes']) / adj.values().numel()
    ms = sum(times) / len(times) * 1e3
    info = {'cores': threads, 'kind': 'port',
            'sample': (f"oracle torch-CPU epoch (addmm_ sparse path + mm + CE + Adam, one process, no communication) on a seeded R-MAT with "
                       f"1/{max(1, args.cpu_sample_divisor)} of the nodes and edges, mean of {steps} epoch(s) = {ms:.1f} ms, x {scale:.2f}"),
            'sample_epoch_ms': round(ms, 2), 'scale': round(scale, 3)}
    return ms * scale, info


def cpu_epoch(cfg, args, steps, warmup):
    if os.path.isdir(REF_DIR):
        return run_reference_files(cfg, args, steps, warmup)
    return run_port_sample(cfg, args, steps, warmup)


def run_reference(args):
    """The reference's CPU implementation of the path on the host cores (rank 0 only under torchrun)."""
    if int(os.environ.get('RANK', 0)) != 0:
        return
    cfg = workload_config(args)
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    ms, info = cpu_epoch(cfg, args, steps, warmup)
    world = int(os.environ.get('WORLD_SIZE', 1))
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': round(ms, 1), 'unit': UNIT, 'n_gpus': world, 'steps': steps, 'warmup': warmup,
        'ms_per_step': round(ms, 1), 'higher_is_better': False, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32',
        'data': 'synthetic', 'config': config_block(cfg, args, world),
        'cpu_baseline': dict(value=round(ms, 1), unit=UNIT, **info),
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
