"""Host-side logic of the N>1 path on CPU ranks over gloo: DistEnv groups, the stage schedules, the partition files
and loaders.  The sparse product inside the loop is done by the oracle here, from the test only - the product has no
CPU engine, which one of the tests checks."""
import os
import sys
import tempfile

import numpy as np
import pytest
import torch

from conftest import GOLDEN, PKG, ROOT, assert_close


def _dataset(z):
    n, e, c = (int(v) for v in z['in/meta'])
    m = torch.from_numpy(z['in/masks'])
    return dict(edge_index=torch.from_numpy(z['in/edge_index']), features=torch.from_numpy(z['in/features']),
                labels=torch.from_numpy(z['in/labels']), train_mask=m[0], val_mask=m[1], test_mask=m[2],
                num_nodes=n, num_edges=e, num_classes=c)


def _worker(rank, world, rep, port, data_root, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), DIST_GNN_DATA_ROOT=data_root, DIST_GNN_LOG_ROOT=out_dir)
    for p in (ROOT, PKG):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    from coo_graph import Parted_COO_Graph
    from dist_utils import DistEnv
    from models.gcn import broadcast
    from oracle import ref_gcn, ref_graph
    torch.set_num_threads(1)
    env = DistEnv(rank, world, 'gloo', rep=rep)
    try:
        assert env.device.type == 'cpu' and env.comm is None
        g = Parted_COO_Graph('gsmall', rank // rep, world // rep, device=env.device)
        rec = {}
        try:
            broadcast(g.adj_parts, g.features, 'x')
            rec['cpu_refused'] = False
        except RuntimeError as e:
            rec['cpu_refused'] = 'no CPU path' in str(e)
        # the stage loop, executed by the test: gloo broadcasts in the schedule's group + oracle products
        group = env.col_groups[env.rank_col] if rep > 1 else env.world_group
        x = g.features.clone()
        z = np.zeros(tuple(x.shape), dtype=np.float32)
        for st in env.stages():
            buf = x.clone() if st.root_global == rank else torch.zeros_like(x)
            dist.broadcast(buf, src=st.root_global, group=group)
            a = g.adj_parts[st.part]
            idx = a.indices().numpy()
            ref_gcn.spmm_coo(ref_graph.Coo(idx[0], idx[1], a.values().numpy(), tuple(a.shape)), buf.numpy(), z, 1.0, 1.0)
        zt = torch.from_numpy(z)
        if rep > 1:
            dist.all_reduce(zt, group=env.row_groups[env.rank_grp])
        rec['z'] = zt.numpy()
        w = torch.full((3, 2), float(rank + 1))
        env.all_reduce_sum(w)                                   # dW reduction group: world (1D) or column group (1.5D)
        rec['w'] = w.numpy()
        rec['gathered'] = env.all_gather_then_cat(torch.full((2, 1), float(rank // rep))).numpy()
        with env.timer.timing('epoch'):
            pass
        summary = env.timer.summary_all()
        rec['summary_ok'] = 'epoch' in summary
        env.logger.log('hello from', rank)
        rec['log_ok'] = os.path.exists(os.path.join(out_dir, f'logs_{world}', f'all_log_{rank}.txt'))
        np.savez(os.path.join(out_dir, f'rank{rank}.npz'), **rec)
    finally:
        env.shutdown()


def _run(world, rep, port):
    import torch.multiprocessing as mp
    from coo_graph import COO_Graph, datasets
    z = np.load(os.path.join(GOLDEN, 'graph_small.npz'))
    data_root, out_dir = tempfile.mkdtemp(prefix='dg_gloo_data_'), tempfile.mkdtemp(prefix='dg_gloo_out_')
    old = datasets.data_root
    datasets.data_root = data_root
    try:
        datasets.save_dataset(name='gsmall', **_dataset(z))
        COO_Graph('gsmall').partition(world // rep)
    finally:
        datasets.data_root = old
    mp.spawn(_worker, (world, rep, port, data_root, out_dir), nprocs=world, join=True)
    return z, [np.load(os.path.join(out_dir, f'rank{r}.npz')) for r in range(world)]



def _two_layouts_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), DIST_GNN_LOG_ROOT=out_dir)
    for p in (ROOT, PKG):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    from dist_utils import DistEnv
    torch.set_num_threads(1)
    first = DistEnv(rank, world, 'gloo')
    w = torch.full((2,), float(rank + 1))
    first.all_reduce_sum(w)
    stages_1d = len(first.stages())
    first.shutdown(keep_process_group=True)
    assert dist.is_initialized() and DistEnv.env is None
    second = DistEnv(rank, world, 'gloo', rep=2)            # another layout on the same process group
    v = torch.full((2,), float(rank + 1))
    second.all_reduce_sum(v)                                # column group: the ranks with the same replica index
    second.barrier_all()
    rec = dict(w=w.numpy(), v=v.numpy(), stages=np.array([stages_1d, len(second.stages())]))
    second.shutdown()
    assert not dist.is_initialized()
    np.savez(os.path.join(out_dir, f'rank{rank}.npz'), **rec)


def test_a_second_layout_follows_in_the_same_processes():
    """bench.py measures the 1.5D configuration after the 1D one without a new rendezvous."""
    import torch.multiprocessing as mp
    out_dir = tempfile.mkdtemp(prefix='dg_gloo_two_')
    mp.spawn(_two_layouts_worker, (4, 29631, out_dir), nprocs=4, join=True)
    recs = [np.load(os.path.join(out_dir, f'rank{r}.npz')) for r in range(4)]
    for r, rec in enumerate(recs):
        assert rec['w'].tolist() == [10.0, 10.0]                                   # 1 + 2 + 3 + 4 over the world
        assert rec['v'].tolist() == ([4.0, 4.0] if r % 2 == 0 else [6.0, 6.0])      # ranks {0, 2} and {1, 3}
        assert rec['stages'].tolist() == [4, 1]                                       # R = 2 blocks, each replica takes one


def _oracle_parts(z, R):
    from oracle import ref_graph
    n = int(z['in/meta'][0])
    A = ref_graph.Coo(z['full/adj_idx'][0], z['full/adj_idx'][1], z['full/adj_val'], (n, n))
    return [ref_graph.parted_graph(p) for p in ref_graph.partition(A, z['full/features'], z['in/labels'].astype(np.int64), z['in/masks'], R)]


def test_1d_schedule_over_two_gloo_ranks_matches_reference(golden):
    z, res = _run(2, 1, 29811)
    t = golden('gcn_small')
    for r in range(2):
        assert bool(res[r]['cpu_refused'])
        assert_close(res[r]['z'], t[f'r{r}/bcast_0'], 1e-5, f'rank {r} vs the reference over gloo')
        assert np.array_equal(res[r]['w'], np.full((3, 2), 3.0))
        assert np.array_equal(res[r]['gathered'].ravel(), [0, 0, 1, 1])
        assert bool(res[r]['summary_ok']) and bool(res[r]['log_ok'])


def test_15d_schedule_over_four_gloo_ranks_matches_oracle_and_1d(golden):
    from oracle import ref_gcn
    z, res = _run(4, 2, 29813)
    parts = _oracle_parts(z, 2)
    want = ref_gcn.broadcast_15d([p['adj_parts'] for p in parts], [p['features'] for p in parts], 4, 2)
    one_d = ref_gcn.broadcast_1d([p['adj_parts'] for p in parts], [p['features'] for p in parts])
    for r in range(4):
        assert_close(res[r]['z'], want[r], 1e-5, f'rank {r} vs 1.5D oracle')
        assert_close(res[r]['z'], one_d[r // 2], 1e-5, f'rank {r} vs 1D over the same 2 row blocks')
        # dW is summed over the column group {r%2, r%2+2}: ranks (1,3) -> 1+3... with values rank+1
        assert np.array_equal(res[r]['w'], np.full((3, 2), float((r % 2 + 1) + (r % 2 + 3))))
        assert np.array_equal(res[r]['gathered'].ravel(), [0, 0, 1, 1])


def test_schedule_shapes():
    from dist_utils import schedule
    assert [tuple(s) for s in schedule.stages_1d(3)] == [(0, 0, 0), (1, 1, 1), (2, 2, 2)]
    # 8 ranks, c = 2: 4 row blocks, 2 stages each; replica 0 takes column blocks 0,1 and replica 1 takes 2,3
    assert [s.part for s in schedule.stages_15d(0, 8, 2)] == [0, 1] and [s.root_global for s in schedule.stages_15d(0, 8, 2)] == [0, 2]
    assert [s.part for s in schedule.stages_15d(7, 8, 2)] == [2, 3] and [s.root_global for s in schedule.stages_15d(7, 8, 2)] == [5, 7]
    assert schedule.row_groups(8, 2) == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert schedule.col_groups(8, 2) == [[0, 2, 4, 6], [1, 3, 5, 7]]
    # the last replica takes the remainder: 12 ranks, c = 3 -> 4 row blocks, P // c^2 = 1 stage each, last replica 2 stages
    assert [len(schedule.stages_15d(r, 12, 3)) for r in range(3)] == [1, 1, 2]
    covered = sorted(s.part for r in range(3) for s in schedule.stages_15d(r, 12, 3))
    assert covered == [0, 1, 2, 3]
    for P, c in ((4, 2), (8, 2), (9, 3), (12, 3), (16, 4)):
        for rank in range(P):
            for s in schedule.stages_15d(rank, P, c):
                assert s.root_global % c == rank % c and s.root_global // c == s.part
                assert schedule.col_groups(P, c)[rank % c][s.root_in_group] == s.root_global
    with pytest.raises(ValueError):
        schedule.check_layout(6, 4)
    with pytest.raises(ValueError):
        schedule.check_layout(2, 2)


def test_pull_order_of_the_peer_copy_loop():
    """1D: every rank handles its own block first and then reads from rank+1, rank+2, ...: at every step the P readers
    read from P different owners.  1.5D: own stages first, every stage exactly once."""
    from dist_utils import schedule
    for P in (2, 3, 8):
        orders = []
        for me in range(P):
            st = schedule.stages(me, P, 1)
            own, remote = schedule.pull_order(st, me, P)
            assert [st[i].root_in_group for i in own] == [me]
            assert [st[i].root_in_group for i in remote] == [(me + j) % P for j in range(1, P)]
            orders.append([st[i].root_in_group for i in remote])
        for step in range(P - 1):
            assert sorted(o[step] for o in orders) == list(range(P))
    for P, c in ((8, 2), (12, 3), (4, 2)):
        for rank in range(P):
            st = schedule.stages(rank, P, c)
            me = schedule.col_groups(P, c)[rank % c].index(rank)
            own, remote = schedule.pull_order(st, me, P // c)
            assert sorted(own + remote) == list(range(len(st)))
            assert all(st[i].root_in_group == me for i in own) and all(st[i].root_in_group != me for i in remote)


def test_pack_layout_of_the_compact_peer_loop():
    """Readers' row lists lie one after the other in the owner's send buffer, in reader order, the owner itself taking
    no room; every rank derives the same layout from the gathered sizes."""
    from dist_utils import schedule
    sizes = [[0, 5, 2], [7, 0, 0], [3, 4, 0]]          # sizes[q][s]: rows of block s that reader q needs
    assert schedule.pack_layout(sizes, 0) == ([0, 0, 7], 10)
    assert schedule.pack_layout(sizes, 1) == ([0, 5, 5], 9)
    assert schedule.pack_layout(sizes, 2) == ([0, 2, 2], 2)


@pytest.mark.parametrize('P', [2, 3, 4, 8])
def test_compact_peer_loop_bookkeeping_simulated_on_the_host(P):
    """The index bookkeeping of the 'peer_compact' stage order (lists of touched rows, pack layout inside the owners' send
    buffers, pull offsets, re-numbered blocks), run for all P ranks at once in NumPy: every rank's result equals the plain
    sum over the stages A[r, s] @ X_s, and no reader ever pulls a row it did not ask for."""
    from dist_utils import schedule
    rng = np.random.default_rng(P)
    n, F = 37, 5
    A = [[(rng.random((n, n)) < 0.06) * rng.standard_normal((n, n)) for _ in range(P)] for _ in range(P)]   # A[r][s]
    A[1][0][:] = 0.0                                                                      # an empty block
    X = [rng.standard_normal((n, F)) for _ in range(P)]
    per_rank = []
    for me in range(P):
        stages = schedule.stages(me, P, 1)
        own, remote = schedule.pull_order(stages, me, P)
        wanted, kept, blocks = {}, [], []
        for i in remote:
            root = stages[i].root_in_group
            touched = np.flatnonzero(np.abs(A[me][stages[i].part]).sum(axis=0))
            if touched.size == 0:
                continue
            wanted[root] = touched.astype(np.int32)
            kept.append(i)
            blocks.append(A[me][stages[i].part][:, touched])                              # columns re-numbered to list positions
        per_rank.append(dict(stages=stages, own=own, kept=kept, wanted=wanted, blocks=blocks))
    gathered = [r['wanted'] for r in per_rank]
    lays = [schedule.compact_layout(gathered, me, [per_rank[me]['stages'][i].root_in_group for i in per_rank[me]['kept']]) for me in range(P)]
    assert len({lay['send_rows'] for lay in lays}) == 1                                   # every rank allocates the same size
    send = []
    for s in range(P):                                                                    # owners pack
        buf = np.full((lays[s]['send_rows'], F), np.nan)
        for q, offset in lays[s]['packs']:
            rows = gathered[q][s]
            buf[offset:offset + len(rows)] = X[s][rows]
        send.append(buf)
    for me in range(P):                                                                   # readers pull and multiply
        r, lay = per_rank[me], lays[me]
        z = sum(A[me][r['stages'][i].part] @ X[me] for i in r['own'])
        area = np.full((max(lay['area_rows'], 1), F), np.nan)
        for j, i in enumerate(r['kept']):
            root = r['stages'][i].root_in_group
            pulled = send[root][lay['stage_offsets'][j]:lay['stage_offsets'][j] + lay['stage_rows'][j]]
            assert np.array_equal(pulled, X[root][gathered[me][root]])
            area[lay['area_offsets'][j]:lay['area_offsets'][j] + lay['stage_rows'][j]] = pulled
            z = z + r['blocks'][j] @ area[lay['area_offsets'][j]:lay['area_offsets'][j] + lay['stage_rows'][j]]
        want = sum(A[me][s] @ X[s] for s in range(P))
        assert np.allclose(z, want, rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize('P,spec', [(4, 3), (8, (4, 2, 1)), (8, 7), (5, (2, 1))])
def test_joined_arrivals_of_the_compact_loop_on_the_host(P, spec):
    """Arrivals joined into fewer products (stage_group as a size list): the joined block, multiplied by the group's slice
    of the landing area, adds exactly what the member blocks add one by one, and its entries are in row-major,
    (arrival, column) order."""
    from dist_utils import schedule
    from models.gcn import group_sizes
    rng = np.random.default_rng(100 + P)
    n, F, me = 29, 4, 1
    stages = schedule.stages(me, P, 1)
    _, remote = schedule.pull_order(stages, me, P)
    blocks, dense, rows_of = [], [], []
    for i in remote:
        a = (rng.random((n, n)) < 0.08) * rng.standard_normal((n, n))
        touched = np.flatnonzero(np.abs(a).sum(axis=0))
        if touched.size == 0:
            continue
        r, c = np.nonzero(a[:, touched])
        blocks.append((torch.from_numpy(r), torch.from_numpy(c), torch.from_numpy(a[:, touched][r, c]), int(touched.size)))
        dense.append(a[:, touched])
        rows_of.append(int(touched.size))
    offsets = [sum(rows_of[:j]) for j in range(len(rows_of))]
    area = rng.standard_normal((sum(rows_of), F))
    want = sum(d @ area[o:o + k] for d, o, k in zip(dense, offsets, rows_of))
    got, first = np.zeros((n, F)), 0
    for count in group_sizes(len(blocks), spec):
        row, col, val, total = schedule.join_packed_blocks(blocks, offsets, first, count)
        assert total == sum(rows_of[first:first + count])
        keys = (row * total + col).numpy()
        assert np.all(np.diff(keys) > 0)                                   # sorted, no duplicates
        joined = np.zeros((n, total))
        joined[row.numpy(), col.numpy()] = val.numpy()
        got += joined @ area[offsets[first]:offsets[first] + total]
        first += count
    assert first == len(blocks) and np.allclose(got, want, rtol=1e-12, atol=1e-12)


def test_default_stage_groups():
    from dist_utils import schedule
    from models.gcn import group_sizes
    assert schedule.default_stage_group('reference', 1, 8) == 4 and schedule.default_stage_group('reference', 2, 2) == 1
    assert schedule.default_stage_group('peer_compact', 1, 2) == 1 and schedule.default_stage_group('peer_compact', 1, 4) == 1
    assert schedule.default_stage_group('peer_compact', 1, 8) == (1, 1, 1, 1, 1, 2)
    assert group_sizes(7, schedule.default_stage_group('peer_compact', 1, 8)) == [1, 1, 1, 1, 1, 2]
    assert group_sizes(15, schedule.default_stage_group('peer_gather', 1, 16)) == [1] * 13 + [2]
    assert schedule.default_stage_group('peer_copy', 1, 8) == 1 and schedule.default_stage_group('peer_compact', 2, 8) == 1


def test_group_sizes_of_the_compact_loop():
    from models.gcn import group_sizes
    assert group_sizes(7, 1) == [1] * 7 and group_sizes(7, 3) == [3, 3, 1] and group_sizes(7, (4, 2, 1)) == [4, 2, 1]
    assert group_sizes(7, (3, 1)) == [3, 1, 1, 1, 1] and group_sizes(0, 2) == [] and group_sizes(2, (5,)) == [2]


def _tiny_bench_args():
    import argparse
    return argparse.Namespace(seed=0, no_permute=False, config='ragged', rep=1, cpu_sample_divisor=4)


TINY = dict(num_nodes=4012, directed_edges=32000, feat_dim=12, num_classes=5, split=(0.6, 0.2, 0.2), hidden=8, layers=3)


def test_cpu_leg_port_runs_on_a_sample_and_scales_by_stored_entries():
    """The fallback CPU leg of bench.py (the oracle's torch-CPU epoch) on a quarter-size sample of a small ragged config."""
    sys.path.insert(0, ROOT)
    import bench
    small = bench.sample_config(TINY, 4)
    assert small['num_nodes'] == 1003 and small['directed_edges'] == 8000
    ms, info = bench.run_port_sample(TINY, _tiny_bench_args(), steps=1, warmup=0)
    assert ms > 0 and info['kind'] == 'port' and 3.0 < info['scale'] < 5.0


@pytest.mark.skipif(not os.path.isdir(os.path.join(ROOT, 'baseline', '_ref', 'light_dist_gnn')), reason='no copy of the reference in baseline/_ref')
def test_cpu_leg_runs_the_unmodified_reference_over_gloo():
    """bench.py's reference arm: the reference's own files (copied by __graft_entry__.build) train over gloo on part files
    this package wrote, and report the reference timer's keys."""
    sys.path.insert(0, ROOT)
    import bench
    ms, info = bench.run_reference_files(TINY, _tiny_bench_args(), steps=2, warmup=1)
    assert ms > 0 and info['kind'] == 'reference' and info['cores'] >= 2
    assert {'broadcast', 'spmm', 'mm', 'all_reduce', 'epoch'} <= set(info['reference_timer_s'])
