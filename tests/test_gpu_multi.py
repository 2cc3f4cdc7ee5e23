"""The stage loops on real ranks: one process per GPU.  Skipped unless the box has at least 2 (4, 8) GPUs.

2 GPUs: the product's whole training path at P=2 against the values the reference itself produced on 2 gloo ranks.
4 GPUs: the 1.5D schedule (P=4, c=2) against the oracle.
8 GPUs: every 1D schedule at P=8, 1.5D at P=8 / c=2, and 3 epochs of training at P=8, against the oracle.
NVLS is switched off in the workers so that a failing worker cannot leave a multicast binding behind on the shared box.
"""
import os
import sys
import tempfile

import numpy as np
import pytest
import torch

from conftest import GOLDEN, PKG, ROOT, assert_close

pytestmark = pytest.mark.gpu


def _worker(rank, world, rep, port, out_dir, mode):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0',
                      DIST_GNN_LOG_ROOT=out_dir, LOCAL_RANK=str(rank))
    for p in (ROOT, PKG):
        if p not in sys.path:
            sys.path.insert(0, p)
    import dist_train
    from coo_graph import COO_Graph, Parted_COO_Graph
    from dist_utils import DistEnv
    from models.gcn import broadcast
    z = np.load(os.path.join(GOLDEN, 'graph_small.npz'))
    n, e, c = (int(v) for v in z['in/meta'])
    m = torch.from_numpy(z['in/masks'])
    d = dict(edge_index=torch.from_numpy(z['in/edge_index']), features=torch.from_numpy(z['in/features']),
             labels=torch.from_numpy(z['in/labels']), train_mask=m[0], val_mask=m[1], test_mask=m[2],
             num_nodes=n, num_edges=e, num_classes=c)
    env = DistEnv(rank, world, 'nccl', rep=rep)
    try:
        full = COO_Graph.from_dict('gsmall', d, device=env.device)
        g = Parted_COO_Graph.from_full(full, rank // rep, world // rep)
        rec = {}
        if mode == 'train':
            z1 = broadcast(g.adj_parts, g.features, 'probe')
            rec['z1'] = z1.cpu().numpy()
            model, losses = dist_train.train(g, env, total_epoch=3, hidden_dim=16, num_layers=3)
            rec['losses'] = np.array(losses)
            for l, w in enumerate(model.weights()):
                rec[f'w{l}'] = w.detach().cpu().numpy()
        else:   # repeated stage loops of several widths, back to back, to exercise buffer reuse across calls
            gen = torch.Generator().manual_seed(100 + rank // rep)
            for i, width in enumerate((32, 7, 64, 32)):
                x = torch.randn(g.local_num_nodes, width, generator=gen).to(env.device)
                rec[f'x{i}'] = x.cpu().numpy()
                rec[f'z{i}'] = broadcast(g.adj_parts, x, f'w{width}').cpu().numpy()
                env.stage_group = 2          # the same loop with two stages fused into one product
                rec[f'zg{i}'] = broadcast(g.adj_parts, x, f'w{width}').cpu().numpy()
                env.stage_group = 1
                env.stage_order = 'local_first'   # own block first, every broadcast queued up front
                rec[f'zl{i}'] = broadcast(g.adj_parts, x, f'w{width}').cpu().numpy()
                env.stage_group = 2
                rec[f'zlg{i}'] = broadcast(g.adj_parts, x, f'w{width}').cpu().numpy()
                env.stage_group, env.stage_order, env.chunk_width = 1, 'feature_chunks', 16     # 1D only; 1.5D falls through
                rec[f'zf{i}'] = broadcast(g.adj_parts, x, f'w{width}').cpu().numpy()
                env.stage_order, env.chunk_width = 'peer_copy', 64      # remote blocks pulled from the owners' send buffers
                rec[f'zp{i}'] = broadcast(g.adj_parts, x, f'w{width}').cpu().numpy()
                env.stage_group = 2
                rec[f'zpg{i}'] = broadcast(g.adj_parts, x, f'w{width}').cpu().numpy()
                env.stage_group, env.stage_order = 1, 'peer_compact'    # only the rows each reader's block touches travel (1D)
                rec[f'zc{i}'] = broadcast(g.adj_parts, x, f'w{width}').cpu().numpy()
                env.stage_group = (3, 2, 1)                             # the same with arrivals joined into fewer products
                rec[f'zcg{i}'] = broadcast(g.adj_parts, x, f'w{width}').cpu().numpy()
                env.stage_group, env.stage_order = 1, 'peer_gather'     # the reader gathers its rows out of the owner's whole block
                rec[f'zq{i}'] = broadcast(g.adj_parts, x, f'w{width}').cpu().numpy()
                env.stage_group = (2, 1)
                rec[f'zqg{i}'] = broadcast(g.adj_parts, x, f'w{width}').cpu().numpy()
                env.stage_group, env.stage_order = 1, 'reference'
        torch.cuda.synchronize()
        np.savez(os.path.join(out_dir, f'rank{rank}.npz'), **rec)
    finally:
        env.shutdown()


def _run(world, rep, mode, port):
    import torch.multiprocessing as mp
    out_dir = tempfile.mkdtemp(prefix='dg_multi_')
    mp.spawn(_worker, (world, rep, port, out_dir, mode), nprocs=world, join=True)
    return [np.load(os.path.join(out_dir, f'rank{r}.npz')) for r in range(world)]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs 2 GPUs')
def test_training_at_two_ranks_matches_the_reference_over_gloo(golden):
    t = golden('gcn_small')
    res = _run(2, 1, 'train', 29741)
    for r in range(2):
        assert_close(res[r]['z1'], t[f'r{r}/bcast_0'], 1e-5, f'first stage loop, rank {r}')
        for epoch in range(3):
            want = t[f'r{r}/losses'][epoch]
            assert abs(res[r]['losses'][epoch] - want) <= 2e-5 * max(1.0, abs(want)), (r, epoch)
        for l in range(3):
            assert_close(res[r][f'w{l}'], t[f'r{r}/wfinal_{l}'], 1e-4, f'weights after 3 steps, rank {r} layer {l}')


def _oracle_blocks(golden, R):
    from oracle import ref_graph
    z = golden('graph_small')
    n = int(z['in/meta'][0])
    A = ref_graph.Coo(z['full/adj_idx'][0], z['full/adj_idx'][1], z['full/adj_val'], (n, n))
    return [ref_graph.parted_graph(p) for p in ref_graph.partition(A, z['full/features'], z['in/labels'].astype(np.int64), z['in/masks'], R)]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs 2 GPUs')
def test_back_to_back_stage_loops_at_two_ranks(golden):
    from oracle import ref_gcn
    res = _run(2, 1, 'loops', 29743)
    parts = _oracle_blocks(golden, 2)
    for i in range(4):
        want = ref_gcn.broadcast_1d([p['adj_parts'] for p in parts], [res[r][f'x{i}'] for r in range(2)])
        for r in range(2):
            assert_close(res[r][f'z{i}'], want[r], 1e-5, f'loop {i} rank {r}')
            for key in ('zg', 'zl', 'zlg', 'zf', 'zp', 'zpg', 'zc', 'zcg', 'zq', 'zqg'):
                assert_close(res[r][f'{key}{i}'], want[r], 1e-5, f'{key} loop {i} rank {r}')


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason='needs 4 GPUs')
def test_15d_stage_loop_at_four_ranks(golden):
    from oracle import ref_gcn
    res = _run(4, 2, 'loops', 29745)
    parts = _oracle_blocks(golden, 2)
    for i in range(4):
        want = ref_gcn.broadcast_15d([p['adj_parts'] for p in parts], [res[b * 2][f'x{i}'] for b in range(2)], 4, 2)
        for r in range(4):
            assert_close(res[r][f'z{i}'], want[r], 1e-5, f'loop {i} rank {r}')
            for key in ('zg', 'zl', 'zlg', 'zf', 'zp', 'zpg', 'zc', 'zcg', 'zq', 'zqg'):
                assert_close(res[r][f'{key}{i}'], want[r], 1e-5, f'{key} loop {i} rank {r}')


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason='needs 8 GPUs')
def test_every_1d_schedule_at_eight_ranks(golden):
    from oracle import ref_gcn
    res = _run(8, 1, 'loops', 29747)
    parts = _oracle_blocks(golden, 8)
    for i in range(4):
        want = ref_gcn.broadcast_1d([p['adj_parts'] for p in parts], [res[r][f'x{i}'] for r in range(8)])
        for r in range(8):
            for key in ('z', 'zg', 'zl', 'zlg', 'zf', 'zp', 'zpg', 'zc', 'zcg', 'zq', 'zqg'):
                assert_close(res[r][f'{key}{i}'], want[r], 1e-5, f'{key} loop {i} rank {r}')


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason='needs 8 GPUs')
def test_15d_stage_loop_at_eight_ranks(golden):
    from oracle import ref_gcn
    res = _run(8, 2, 'loops', 29749)
    parts = _oracle_blocks(golden, 4)
    for i in range(4):
        want = ref_gcn.broadcast_15d([p['adj_parts'] for p in parts], [res[b * 2][f'x{i}'] for b in range(4)], 8, 2)
        for r in range(8):
            for key in ('z', 'zg', 'zl', 'zlg', 'zf', 'zp', 'zpg', 'zc', 'zcg', 'zq', 'zqg'):
                assert_close(res[r][f'{key}{i}'], want[r], 1e-5, f'{key} loop {i} rank {r}')


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason='needs 8 GPUs')
def test_training_at_eight_ranks_matches_the_oracle(golden):
    """3 epochs of dist_train.train at P=8 with the default schedule (reference initialiser) against the oracle's 8-rank
    model: the first stage loop, each rank's losses, the weights after 3 Adam steps."""
    from oracle import ref_gcn
    res = _run(8, 1, 'train', 29751)
    parts = _oracle_blocks(golden, 8)
    torch.manual_seed(0)
    w0 = [torch.rand(32, 16).numpy(), torch.rand(16, 16).numpy(), torch.rand(16, 7).numpy()]
    oracle = ref_gcn.gcn_1d(parts, w0)
    want_z = ref_gcn.broadcast_1d([p['adj_parts'] for p in parts], [p['features'] for p in parts])
    for r in range(8):
        assert_close(res[r]['z1'], want_z[r], 1e-5, f'first stage loop, rank {r}')
    for epoch in range(3):
        losses, *_ = oracle.epoch([p['features'] for p in parts], [p['local_labels'] for p in parts], [p['local_train_mask'] for p in parts])
        for r in range(8):
            assert abs(res[r]['losses'][epoch] - losses[r]) <= 2e-5 * max(1.0, abs(losses[r])), (r, epoch)
    for l in range(3):
        assert_close(res[0][f'w{l}'], oracle.weights[l], 1e-4, f'weights after 3 steps, layer {l}')
