"""The product's training path (DistEnv -> Parted_COO_Graph -> GCN/DistGCNLayer -> stage loop) on one GPU, and
size-independent properties of the SpMM at the full benchmark size.  Needs a GPU."""
import os

import numpy as np
import pytest
import torch

from conftest import assert_close
from oracle import ref_gcn, ref_graph

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(scope='module')
def env1():
    """A one-rank NCCL environment (no collective is issued with one rank)."""
    import torch.distributed as dist
    from dist_utils import DistEnv
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29731')
    os.environ.setdefault('DIST_GNN_LOG_ROOT', '/tmp/dist_gnn_test_logs')
    env = DistEnv(0, 1, 'nccl')
    yield env
    env.shutdown()
    assert not dist.is_initialized()


def _fixture_dataset(z):
    n, e, c = (int(v) for v in z['in/meta'])
    m = torch.from_numpy(z['in/masks'])
    return dict(edge_index=torch.from_numpy(z['in/edge_index']), features=torch.from_numpy(z['in/features']),
                labels=torch.from_numpy(z['in/labels']), train_mask=m[0], val_mask=m[1], test_mask=m[2],
                num_nodes=n, num_edges=e, num_classes=c)


def test_training_on_one_rank_matches_oracle(golden, env1):
    """3 epochs of dist_train.train (3 layers, reference initialiser) against the oracle at P=1: losses, outputs path
    through autograd, Adam.  Inputs are the reference-normalised fixture graph."""
    import dist_train
    from coo_graph import COO_Graph, Parted_COO_Graph
    z = golden('graph_small')
    full = COO_Graph.from_dict('gsmall', _fixture_dataset(z), device='cuda')
    g = Parted_COO_Graph.from_full(full, 0, 1)
    assert g.features.is_cuda and all(p.is_cuda for p in g.adj_parts)
    model, losses = dist_train.train(g, env1, total_epoch=3, hidden_dim=16, num_layers=3)

    n = int(z['in/meta'][0])
    A = ref_graph.Coo(z['full/adj_idx'][0], z['full/adj_idx'][1], z['full/adj_val'], (n, n))
    parted = [ref_graph.parted_graph(p) for p in ref_graph.partition(A, z['full/features'], z['in/labels'].astype(np.int64), z['in/masks'], 1)]
    torch.manual_seed(0)
    w0 = [torch.rand(32, 16).numpy(), torch.rand(16, 16).numpy(), torch.rand(16, 7).numpy()]
    oracle = ref_gcn.gcn_1d(parted, w0)
    for epoch in range(3):
        want, *_ = oracle.epoch([parted[0]['features']], [parted[0]['local_labels']], [parted[0]['local_train_mask']])
        assert abs(losses[epoch] - want[0]) <= 2e-5 * max(1.0, abs(want[0])), (epoch, losses[epoch], want[0])
    for l, w in enumerate(model.weights()):
        assert_close(w.detach().cpu().numpy(), oracle.weights[l], 1e-4, f'weights after 3 steps, layer {l}')


def test_layer_activations_and_gradients_match_oracle(golden, env1):
    """One DistGCNLayer forward/backward on the GPU: z@W, dX and dW against the oracle, per tensor."""
    from coo_graph import COO_Graph, Parted_COO_Graph
    from models.gcn import DistGCNLayer, broadcast
    z = golden('graph_small')
    g = Parted_COO_Graph.from_full(COO_Graph.from_dict('gsmall', _fixture_dataset(z), device='cuda'), 0, 1)
    rng = np.random.Generator(np.random.PCG64(21))
    W = rng.standard_normal((32, 24), dtype=np.float32)
    G = rng.standard_normal((1000, 24), dtype=np.float32)
    x = g.features.clone().requires_grad_(True)
    w = torch.from_numpy(W).cuda().requires_grad_(True)
    out = DistGCNLayer.apply(x, w, g.adj_parts, 'L1')
    out.backward(torch.from_numpy(G).cuda())
    n = 1000
    A = ref_graph.Coo(z['full/adj_idx'][0], z['full/adj_idx'][1], z['full/adj_val'], (n, n))
    X = g.features.cpu().numpy()
    zz = ref_gcn.spmm_coo(A, X, np.zeros_like(X), 1.0, 0.0)
    ag = ref_gcn.spmm_coo(A, G, np.zeros_like(G), 1.0, 0.0)
    assert_close(broadcast(g.adj_parts, g.features, 't').cpu().numpy(), zz, TOL, 'z')
    assert_close(out.detach().cpu().numpy(), zz @ W, TOL, 'z @ W')
    assert_close(x.grad.cpu().numpy(), ag @ W.T, TOL, 'dX')
    assert_close(w.grad.cpu().numpy(), X.T @ ag, TOL, 'dW')


def test_cpu_tensors_are_refused(golden, env1):
    from coo_graph import COO_Graph, Parted_COO_Graph
    from models.gcn import broadcast
    z = golden('graph_small')
    g = Parted_COO_Graph.from_full(COO_Graph.from_dict('gsmall', _fixture_dataset(z)), 0, 1)
    with pytest.raises(RuntimeError, match='no CPU path'):
        broadcast(g.adj_parts, g.features, 't')


def test_three_pass_tf32_dense_transform_stays_inside_the_parity_bound(golden, env1, monkeypatch):
    """The tensor-core dense transform (three TF32 GEMMs per product, fp32 accumulation) against float64 and, through a
    whole layer forward/backward, against the fp32 path: 1e-5 relative per tensor like every other parity check."""
    import models.gcn as gcn
    g = torch.Generator(device='cuda').manual_seed(3)
    a = torch.randn(20000, 256, device='cuda', generator=g)
    b = torch.randn(256, 256, device='cuda', generator=g)
    c = torch.randn(20000, 47, device='cuda', generator=g)
    monkeypatch.setattr(gcn, 'DENSE_MODE', '3xtf32')
    for got, want in ((gcn.dense_mm(a, b), a.double() @ b.double()),
                      (gcn.dense_mm(a, b, tb=True), a.double() @ b.double().t()),
                      (gcn.dense_mm(a, c, ta=True), a.double().t() @ c.double())):
        assert_close(got.cpu().numpy(), want.cpu().numpy(), TOL, 'dense transform vs float64')
    # one-pass TF32 would not pass: make sure the bound is meaningful
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        one_pass = torch.mm(a, b)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = False
    err = (one_pass.double() - a.double() @ b.double()).abs().max().item() / (a.double() @ b.double()).abs().max().item()
    assert err > TOL
    # and a short training run keeps matching the fp32 path
    import dist_train
    from coo_graph import COO_Graph, Parted_COO_Graph
    z = golden('graph_small')
    graph = Parted_COO_Graph.from_full(COO_Graph.from_dict('gsmall', _fixture_dataset(z), device='cuda'), 0, 1)
    _, losses_tc = dist_train.train(graph, env1, total_epoch=3, hidden_dim=16, num_layers=3)
    monkeypatch.setattr(gcn, 'DENSE_MODE', 'fp32')
    _, losses_fp32 = dist_train.train(graph, env1, total_epoch=3, hidden_dim=16, num_layers=3)
    for x, y in zip(losses_tc, losses_fp32):
        assert abs(x - y) <= 2e-5 * max(1.0, abs(y))


@pytest.fixture(scope='module')
def big_graph():
    """The 2,449,029-node / 123.7 M-edge benchmark graph, generated and normalised on the GPU."""
    from coo_graph import graph_utils, synthetic
    cfg = synthetic.CONFIGS['sparse2m']
    ei = synthetic.rmat_edge_index(cfg['num_nodes'], cfg['directed_edges'], seed=0, device='cuda')
    assert ei.shape == (2, cfg['directed_edges'])
    A = graph_utils.sym_normalization(ei, cfg['num_nodes'])
    del ei
    return A


def test_full_size_graph_and_spmm_properties(big_graph):
    """Checks that do not need a CPU pass over 126 M entries: structure of the normalised graph, linearity,
    symmetry (x'Ay == y'Ax), row sums, the 4-way column-block stage sum against the one-block product, and 64 sampled
    rows recomputed by the CPU oracle."""
    import spmm_cpp
    A = big_graph
    N = A.size(0)
    idx, val = A.indices(), A.values()
    assert A._nnz() == 123_718_280 + N
    key = idx[0] * N + idx[1]
    assert bool((key[1:] > key[:-1]).all())                                  # sorted, no duplicates
    sym = torch.sort(idx[1] * N + idx[0]).values
    assert torch.equal(sym, key)                                             # structurally symmetric
    del key, sym
    plan = spmm_cpp.SpmmPlan.from_coo(A)
    st = plan.stats()
    assert st['nnz'] == A._nnz() and st['touched_columns'] == N
    rp = plan.rowptr()
    assert rp[0] == 0 and rp[-1] == A._nnz() and bool((rp[1:] >= rp[:-1]).all())
    assert torch.equal((rp[1:] - rp[:-1]).cuda(), torch.bincount(idx[0], minlength=N))

    F = 64
    g = torch.Generator(device='cuda').manual_seed(5)
    X = torch.randn(N, F, device='cuda', generator=g)
    Y = torch.randn(N, F, device='cuda', generator=g)
    AX, AY, AXY = (torch.empty(N, F, device='cuda') for _ in range(3))
    plan.spmm(X, AX, 1.0, 0.0)
    plan.spmm(Y, AY, 1.0, 0.0)
    plan.spmm(2.0 * X - 0.5 * Y, AXY, 1.0, 0.0)
    scale = AX.abs().max().item()
    assert (AXY - (2.0 * AX - 0.5 * AY)).abs().max().item() <= 1e-5 * 3 * scale     # linearity
    lhs, rhs = (Y.double() * AX.double()).sum().item(), (X.double() * AY.double()).sum().item()
    assert abs(lhs - rhs) <= 1e-6 * max(abs(lhs), abs(rhs), 1.0) * 10                # symmetry of A
    ones = torch.ones(N, 4, device='cuda')
    rs = torch.empty(N, 4, device='cuda')
    plan.spmm(ones, rs, 1.0, 0.0)
    want_rs = torch.zeros(N, dtype=torch.float64, device='cuda').index_add_(0, idx[0], val.double())
    assert (rs[:, 0].double() - want_rs).abs().max().item() <= 1e-5 * want_rs.abs().max().item()

    # accumulate mode: C = 0.5*A*X + 2*C
    C = AY.clone()
    plan.spmm(X, C, 0.5, 2.0)
    assert (C - (0.5 * AX + 2.0 * AY)).abs().max().item() <= 1e-5 * 3 * scale

    # sampled rows against the CPU oracle
    rows = torch.randint(0, N, (64,), generator=torch.Generator().manual_seed(9)).unique()
    rows = torch.cat((rows, (rp[1:] - rp[:-1]).argmax().view(1)))         # and the heaviest row
    for i in rows.tolist():
        e0, e1 = int(rp[i]), int(rp[i + 1])
        cols = idx[1, e0:e1]
        sub = ref_graph.Coo(np.zeros(e1 - e0, np.int64), np.arange(e1 - e0, dtype=np.int64), val[e0:e1].cpu().numpy(), (1, e1 - e0))
        want = ref_gcn.spmm_coo(sub, np.ascontiguousarray(X[cols].cpu().numpy()), np.zeros((1, F), np.float32), 1.0, 0.0)
        assert np.abs(AX[i].cpu().numpy() - want[0]).max() <= 1e-5 * scale, i      # per-tensor scale, as everywhere

    # the stage structure: 4 column blocks accumulated in order == one block
    from coo_graph import graph_utils
    n4 = (N + 3) // 4
    parts = graph_utils.sparse_2d_split(A, n4, split_dim=1)
    Xpad = torch.cat((X, torch.zeros(n4 * 4 - N, F, device='cuda')))
    Z = torch.empty(N, F, device='cuda')
    for s, part in enumerate(parts):
        block = Xpad[s * n4:(s + 1) * n4]
        if part.size(1) < n4:
            block = block[:part.size(1)]
        spmm_cpp.SpmmPlan.from_coo(part).spmm(block, Z, 1.0, 0.0 if s == 0 else 1.0)
    assert (Z - AX).abs().max().item() <= 1e-5 * scale


def test_fused_relu_equals_separate_relu(golden, env1):
    """The ReLU between two layers, run inside the dense kernels' epilogues (forward: max(x, 0); backward: the gradient
    zeroed where the activation is zero), gives bit-identical logits and weight gradients to F.relu between the layers."""
    from coo_graph import COO_Graph, Parted_COO_Graph
    from models import gcn as gcn_module
    from models import GCN
    z = golden('graph_small')
    full = COO_Graph.from_dict('gsmall', _fixture_dataset(z), device='cuda')
    g = Parted_COO_Graph.from_full(full, 0, 1)
    gen = torch.Generator().manual_seed(3)
    weights = [torch.randn(32, 64, generator=gen) * 0.3, torch.randn(64, 64, generator=gen) * 0.3, torch.randn(64, 7, generator=gen) * 0.3]
    results = {}
    saved = gcn_module.FUSE_RELU
    try:
        for fused in (True, False):
            gcn_module.FUSE_RELU = fused
            model = GCN(g, env1, hidden_dim=64, num_layers=3, weights=weights)
            out = model(g.features)
            (out * torch.linspace(-1, 1, out.numel(), device=out.device).view_as(out)).sum().backward()
            results[fused] = (out.detach().clone(), [w.grad.detach().clone() for w in model.weights()])
    finally:
        gcn_module.FUSE_RELU = saved
    assert torch.equal(results[True][0], results[False][0])
    assert (results[True][0] != 0).any()
    for a, b in zip(results[True][1], results[False][1]):
        assert torch.equal(a, b)


@pytest.mark.parametrize('dense', ['host', 'cuda'])
def test_plumbing_config_on_emulated_ranks_matches_the_reference_run(golden, dense, monkeypatch):
    """BASELINE config 0 (10,000-node R-MAT, 128 -> 64 -> 10, Glorot weights, 2 ranks) with this package's loaders and
    CUDA kernels, against what the unmodified reference produced for it on 2 gloo ranks (tests/golden/plumbing.npz):
    every stage-loop result of epoch 0 (sampled rows, column sums, norms), dW after the all-reduce, 3 losses.  The two
    ranks are emulated on one GPU: rank r adds plan(A[r, s]) @ X_s for s = 0, 1 in stage order.
    dense='host': only the sparse products run on the GPU; dense='cuda': the dense transforms too (dg_dense_nt / _tn)."""
    import spmm_cpp
    from coo_graph import COO_Graph, Parted_COO_Graph, synthetic
    from models.gcn import dense_mm
    t = golden('plumbing')
    cfg = synthetic.CONFIGS['plumbing']
    full = COO_Graph.from_dict('plumbing', synthetic.make_dataset(seed=0, device='cuda', **cfg), device='cuda')
    assert full.adj.values().numel() == int(t['full/adj_nnz'])
    ranks = [Parted_COO_Graph.from_full(full, r, 2) for r in range(2)]
    plans = [[spmm_cpp.plan_for(a) for a in g.adj_parts] for g in ranks]

    def bcast(blocks):
        xs = [torch.from_numpy(np.ascontiguousarray(b)).cuda() for b in blocks]
        out = []
        for r in range(2):
            z = torch.empty_like(xs[r])
            for s in range(2):
                plans[r][s].spmm(xs[s], z, 1.0, 0.0 if s == 0 else 1.0)
            out.append(z.cpu().numpy())
        return out

    if dense == 'cuda':
        def mm(a, b):
            if not a.flags['C_CONTIGUOUS'] and a.T.flags['C_CONTIGUOUS']:      # x^T @ ag: the weight-gradient kernel
                return dense_mm(torch.from_numpy(a.T).cuda(), torch.from_numpy(np.ascontiguousarray(b)).cuda(), ta=True).cpu().numpy()
            return dense_mm(torch.from_numpy(np.ascontiguousarray(a)).cuda(), torch.from_numpy(np.ascontiguousarray(b)).cuda()).cpu().numpy()
        monkeypatch.setattr(ref_gcn, '_mm', mm)
    dims = [cfg['feat_dim'], cfg['hidden'], cfg['num_classes']]
    weights = [w.numpy() for w in synthetic.glorot_weights(dims, seed=0)]
    model = ref_gcn.GcnOracle(bcast, weights, [[0, 1]])
    feats = [g.features.cpu().numpy() for g in ranks]
    labels = [g.local_labels.cpu().numpy() for g in ranks]
    masks = [g.local_train_mask.cpu().numpy() for g in ranks]
    rows = t['sample_rows']
    for epoch in range(3):
        losses, outputs, trace, btrace = model.epoch(feats, labels, masks)
        for r in range(2):
            want = t[f'r{r}/losses'][epoch]
            assert abs(losses[r] - want) <= 2e-5 * max(1.0, abs(want)), (epoch, r, losses[r], want)
        if epoch == 0:
            for r in range(2):
                got = [trace[0]['z'][r], trace[1]['z'][r], btrace[1]['ag'][r], btrace[0]['ag'][r]]
                for i, g in enumerate(got):
                    scale = float(t[f'r{r}/bcast_{i}/absmax'])
                    assert np.abs(g[rows] - t[f'r{r}/bcast_{i}/rows']).max() <= TOL * scale, (r, i)
                    assert np.abs(g.astype(np.float64).sum(0) - t[f'r{r}/bcast_{i}/colsum']).max() <= 1e-4 * scale * np.sqrt(g.shape[0])
                    fro = float(t[f'r{r}/bcast_{i}/fro'])
                    assert abs(np.sqrt((g.astype(np.float64) ** 2).sum()) - fro) <= TOL * fro
                for l in range(2):
                    assert_close(btrace[l]['dw'][r], t[f'r{r}/dw_{l}'], TOL, f'dW{l} rank {r}')
    if dense == 'cuda':
        assert spmm_cpp.dense_status() == 0


def test_cached_input_product_gives_bit_identical_training(golden, env1):
    """GCN(cache_input_product=True) keeps the first layer's A X between epochs: same losses and weights bit for bit;
    the cache follows the features tensor (a new tensor or an in-place change recomputes it)."""
    import dist_train
    from coo_graph import COO_Graph, Parted_COO_Graph
    from models.gcn import broadcast
    z = golden('graph_small')
    g = Parted_COO_Graph.from_full(COO_Graph.from_dict('gsmall', _fixture_dataset(z), device='cuda'), 0, 1)
    plain_model, plain = dist_train.train(g, env1, total_epoch=4, hidden_dim=16, num_layers=3)
    cached_model, cached = dist_train.train(g, env1, total_epoch=4, hidden_dim=16, num_layers=3, cache_input_product=True)
    assert plain == cached
    for a, b in zip(plain_model.weights(), cached_model.weights()):
        assert torch.equal(a.detach(), b.detach())
    first = cached_model.input_product(g.features)
    assert first is cached_model.input_product(g.features)                    # a hit
    assert torch.equal(first, broadcast(g.adj_parts, g.features, 'check'))
    other = (g.features * 2).contiguous()
    assert torch.equal(cached_model.input_product(other), broadcast(g.adj_parts, other, 'check'))      # another tensor
    other.mul_(0.5)
    assert torch.equal(cached_model.input_product(other), first)              # changed in place: recomputed
    assert plain_model.input_product(g.features) is None                      # caching is off by default


def test_input_gradient_shortcut_matches_within_rounding(golden, env1):
    """GCN(input_gradient_shortcut=True): dW1 = (A X)^T G instead of X^T (A G).  Equal for the symmetric normalised
    adjacency up to rounding: losses within 2e-5, weights after 4 steps within 1e-4, and no stage loop runs for layer 1."""
    import dist_train
    import spmm_cpp
    from coo_graph import COO_Graph, Parted_COO_Graph
    z = golden('graph_small')
    g = Parted_COO_Graph.from_full(COO_Graph.from_dict('gsmall', _fixture_dataset(z), device='cuda'), 0, 1)
    plain_model, plain = dist_train.train(g, env1, total_epoch=4, hidden_dim=16, num_layers=3)
    spmm_cpp.profile_begin()
    short_model, short = dist_train.train(g, env1, total_epoch=4, hidden_dim=16, num_layers=3, input_gradient_shortcut=True)
    prof = spmm_cpp.profile_end()
    assert prof['products'] == 1 + 4 * 4            # the cached product once, then 2 forward + 2 backward loops per epoch
    for a, b in zip(plain, short):
        assert abs(a - b) <= 2e-5 * max(1.0, abs(a))
    for a, b in zip(plain_model.weights(), short_model.weights()):
        assert_close(b.detach().cpu().numpy(), a.detach().cpu().numpy(), 1e-4, 'weights with the gradient shortcut')


def test_transform_first_matches_within_rounding(golden, env1):
    """GCN(transform_first=True): the last layer computes A (H W) instead of (A H) W, so its stage loop runs at the class
    count instead of the hidden width.  Same losses within 2e-5, same weights after 4 steps within 1e-4; the backward pass
    is the same computation."""
    import dist_train
    from coo_graph import COO_Graph, Parted_COO_Graph
    z = golden('graph_small')
    g = Parted_COO_Graph.from_full(COO_Graph.from_dict('gsmall', _fixture_dataset(z), device='cuda'), 0, 1)
    plain_model, plain = dist_train.train(g, env1, total_epoch=4, hidden_dim=16, num_layers=3)
    first_model, first = dist_train.train(g, env1, total_epoch=4, hidden_dim=16, num_layers=3, transform_first=True)
    for a, b in zip(plain, first):
        assert abs(a - b) <= 2e-5 * max(1.0, abs(a))
    for a, b in zip(plain_model.weights(), first_model.weights()):
        assert_close(b.detach().cpu().numpy(), a.detach().cpu().numpy(), 1e-4, 'weights with transform_first')
    with torch.no_grad():
        assert_close(first_model(g.features).cpu().numpy(), plain_model(g.features).cpu().numpy(), 1e-4, 'outputs')
