"""Parity of the CUDA SpMM (through the C ABI) with the reference's outputs and with the CPU oracle.  Needs a GPU."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import assert_close
from oracle import ref_gcn, ref_graph

pytestmark = pytest.mark.gpu
TOL = 1e-5   # fp32 parity tolerance of the path (max-abs and Frobenius relative error); the sum order differs


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return t.to('cuda', dtype=dtype) if dtype else t.cuda()


def make_plan(A, **kw):
    import spmm_cpp
    return spmm_cpp.SpmmPlan(dev(A.row, torch.int32), dev(A.col, torch.int32), dev(A.val), A.shape[0], A.shape[1], **kw)


def random_coo(rng, m, k, nnz, heavy=None):
    flat = rng.choice(m * k, size=min(nnz, m * k), replace=False)
    row, col = flat // k, flat % k
    if heavy:   # (row id, entries) pairs forced to be dense-ish rows
        for r, cnt in heavy:
            keep = row != r
            row, col = row[keep], col[keep]
            row = np.concatenate((row, np.full(cnt, r)))
            col = np.concatenate((col, rng.choice(k, cnt, replace=False)))
    val = rng.standard_normal(row.size, dtype=np.float32)
    return ref_graph.fast_coalesce_sorted(row.astype(np.int64), col.astype(np.int64), val, (m, k))


def test_library_exports_and_version():
    import spmm_cpp
    assert spmm_cpp.lib().dg_version() >= 100


def test_golden_cases_through_the_drop_in_signature(golden):
    """spmm_cusparse(row, col, val, A_row, A_col, B, C, alpha, beta) against the reference's C.addmm_(A, B)."""
    import spmm_cpp
    z = golden('spmm_cases')
    for name in z['names']:
        g = lambda key: z[f'{name}/{key}']
        m, k, F = (int(v) for v in g('dims'))
        alpha, beta = (float(v) for v in g('ab'))
        C = dev(g('C0'))
        spmm_cpp.spmm_cusparse(dev(g('row')), dev(g('col')), dev(g('val')), m, k, dev(g('B')), C, alpha, beta)
        assert_close(C.cpu().numpy(), g('C'), TOL, name)


def test_drop_in_route_keeps_plans_only_for_the_same_matrix():
    """spmm_cusparse recognises a block by the address of its values and re-checks the ids it is given: the same block
    again reuses the plan (fresh int32 copies of the ids, as the reference's binding passes them), other ids at the same
    values address build a new one, and the transient-plan route (cache off) gives the same numbers."""
    import spmm_cpp
    rng = np.random.Generator(np.random.PCG64(91))
    A = random_coo(rng, 200, 150, 3000, heavy=[(9, 140)])
    B = rng.standard_normal((150, 36), dtype=np.float32)
    C0 = rng.standard_normal((200, 36), dtype=np.float32)
    want = ref_gcn.spmm_coo(A, B, C0.copy(), 1.0, 1.0)
    row, col, val = dev(A.row, torch.int32), dev(A.col, torch.int32), dev(A.val)
    spmm_cpp._dropin_plans.clear()
    for _ in range(3):
        C = dev(C0)
        spmm_cpp.spmm_cusparse(row.clone(), col.clone(), val, 200, 150, dev(B), C, 1, 1)
        assert_close(C.cpu().numpy(), want, TOL, 'drop-in, cached plan')
    assert len(spmm_cpp._dropin_plans) == 1
    first_plan = next(iter(spmm_cpp._dropin_plans.values()))[0]
    # another matrix whose values live at the same address: same nnz and shape, rows reversed
    A2 = ref_graph.fast_coalesce_sorted((199 - A.row).astype(np.int64), A.col.astype(np.int64), A.val, (200, 150))
    val.copy_(dev(A2.val))
    C = dev(C0)
    spmm_cpp.spmm_cusparse(dev(A2.row, torch.int32), dev(A2.col, torch.int32), val, 200, 150, dev(B), C, 1, 1)
    assert_close(C.cpu().numpy(), ref_gcn.spmm_coo(A2, B, C0.copy(), 1.0, 1.0), TOL, 'drop-in after the matrix changed')
    assert len(spmm_cpp._dropin_plans) == 1 and next(iter(spmm_cpp._dropin_plans.values()))[0] is not first_plan
    keep = spmm_cpp.DROPIN_PLAN_CACHE
    try:
        spmm_cpp.DROPIN_PLAN_CACHE = 0
        C = dev(C0)
        spmm_cpp.spmm_cusparse(dev(A2.row, torch.int32), dev(A2.col, torch.int32), val, 200, 150, dev(B), C, 1, 1)
        assert_close(C.cpu().numpy(), ref_gcn.spmm_coo(A2, B, C0.copy(), 1.0, 1.0), TOL, 'drop-in, transient plan')
    finally:
        spmm_cpp.DROPIN_PLAN_CACHE = keep
        spmm_cpp._dropin_plans.clear()


@pytest.mark.parametrize('F', [1, 2, 3, 4, 6, 8, 10, 16, 20, 32, 41, 47, 64, 100, 128, 130, 256, 300, 512, 602, 1024])
def test_widths_against_oracle(F):
    rng = np.random.Generator(np.random.PCG64(F))
    A = random_coo(rng, 257, 193, 4000, heavy=[(5, 150), (256, 193)])
    B = rng.standard_normal((193, F), dtype=np.float32)
    C0 = rng.standard_normal((257, F), dtype=np.float32)
    want = ref_gcn.spmm_coo(A, B, C0.copy(), 0.75, -1.25)
    for kw in ({}, {'heavy_threshold': 16, 'chunk': 7}):     # default bins, and bins that force the split-row path
        plan = make_plan(A, **kw)
        C = dev(C0)
        plan.spmm(dev(B), C, 0.75, -1.25)
        assert_close(C.cpu().numpy(), want, TOL, f'F={F} {kw}')


def test_beta_zero_ignores_garbage_in_c():
    rng = np.random.Generator(np.random.PCG64(11))
    A = random_coo(rng, 100, 80, 900, heavy=[(7, 60)])
    B = rng.standard_normal((80, 48), dtype=np.float32)
    want = ref_gcn.spmm_coo(A, B, np.zeros((100, 48), dtype=np.float32), 2.0, 0.0)
    for kw in ({}, {'heavy_threshold': 8, 'chunk': 8}):
        C = torch.full((100, 48), float('nan'), device='cuda')
        make_plan(A, **kw).spmm(dev(B), C, 2.0, 0.0)
        assert_close(C.cpu().numpy(), want, TOL, 'beta=0')


def test_empty_shapes():
    import spmm_cpp
    empty = ref_graph.Coo(np.zeros(0, np.int64), np.zeros(0, np.int64), np.zeros(0, np.float32), (6, 5))
    plan = make_plan(empty)
    C = torch.ones(6, 4, device='cuda')
    plan.spmm(torch.ones(5, 4, device='cuda'), C, 1.0, 1.0)
    assert torch.equal(C.cpu(), torch.ones(6, 4))
    plan.spmm(torch.ones(5, 4, device='cuda'), C, 1.0, 0.0)
    assert torch.equal(C.cpu(), torch.zeros(6, 4))
    assert plan.rowptr().tolist() == [0] * 7
    zero_rows = ref_graph.Coo(np.zeros(0, np.int64), np.zeros(0, np.int64), np.zeros(0, np.float32), (0, 5))
    make_plan(zero_rows).spmm(torch.ones(5, 4, device='cuda'), torch.ones(0, 4, device='cuda'))
    spmm_cpp.spmm_cusparse(torch.zeros(0, dtype=torch.int32, device='cuda'), torch.zeros(0, dtype=torch.int32, device='cuda'),
                           torch.zeros(0, device='cuda'), 3, 2, torch.ones(2, 0, device='cuda'), torch.ones(3, 0, device='cuda'), 1, 1)


def test_row_strided_operands_and_unaligned_views():
    rng = np.random.Generator(np.random.PCG64(12))
    A = random_coo(rng, 90, 70, 1200)
    for F, ld, off in ((32, 40, 0), (32, 35, 1), (6, 9, 3)):     # aligned stride, odd stride, odd offset
        Bbig = rng.standard_normal((70, ld + off), dtype=np.float32)
        Cbig = rng.standard_normal((90, ld + off), dtype=np.float32)
        want = ref_gcn.spmm_coo(A, np.ascontiguousarray(Bbig[:, off:off + F]), np.ascontiguousarray(Cbig[:, off:off + F]), 1.0, 1.0)
        Bd, Cd = dev(Bbig), dev(Cbig)
        make_plan(A).spmm(Bd[:, off:off + F], Cd[:, off:off + F])
        got = Cd.cpu().numpy()
        assert_close(got[:, off:off + F], want, TOL, f'F={F} ld={ld + off}')
        untouched = np.ones(Cbig.shape, dtype=bool)
        untouched[:, off:off + F] = False
        assert np.array_equal(got[untouched], Cbig[untouched])


@pytest.mark.parametrize('F', [20, 47, 256])
def test_fused_epilogue(F):
    rng = np.random.Generator(np.random.PCG64(13))
    A = random_coo(rng, 120, 110, 2500, heavy=[(3, 100)])
    B = rng.standard_normal((110, F), dtype=np.float32)
    C0 = rng.standard_normal((120, F), dtype=np.float32)
    scale = rng.uniform(0.1, 2.0, 120).astype(np.float32)
    bias = rng.standard_normal(F, dtype=np.float32)
    want = ref_gcn.spmm_epilogue(A, B, C0, 1.0, 0.5, row_scale=scale, bias=bias, relu=True)
    for kw in ({}, {'heavy_threshold': 8, 'chunk': 16}):
        C = dev(C0)
        make_plan(A, **kw).spmm(dev(B), C, 1.0, 0.5, row_scale=dev(scale), bias=dev(bias), relu=True)
        assert_close(C.cpu().numpy(), want, TOL, f'epilogue F={F}')
        assert (C >= 0).all()


def test_results_are_bit_reproducible():
    rng = np.random.Generator(np.random.PCG64(14))
    A = random_coo(rng, 500, 400, 30000, heavy=[(0, 400), (499, 333)])
    B = dev(rng.standard_normal((400, 100), dtype=np.float32))
    plan = make_plan(A, heavy_threshold=64, chunk=50)
    outs = []
    for _ in range(3):
        C = torch.zeros(500, 100, device='cuda')
        plan.spmm(B, C, 1.0, 0.0)
        outs.append(C.cpu())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_csr_indexing_is_bit_exact_on_the_reference_partition(golden):
    """Row offsets of every adj_parts block of the reference's own partition (P=2,3), and the plan census."""
    z = golden('graph_small')
    for P in (2, 3):
        for r in range(P):
            pre = f'P{P}/r{r}/'
            nnz, idx, val, shapes = z[pre + 'parts_nnz'], z[pre + 'parts_idx'], z[pre + 'parts_val'], z[pre + 'parts_shape']
            start = 0
            for s in range(P):
                sl = slice(start, start + int(nnz[s]))
                A = ref_graph.Coo(idx[0, sl], idx[1, sl], val[sl], tuple(int(v) for v in shapes[s]))
                start += int(nnz[s])
                plan = make_plan(A)
                assert np.array_equal(plan.rowptr().numpy(), ref_graph.rowptr_of(A))
                st = plan.stats()
                assert st['nnz'] == A.nnz and (st['m'], st['k']) == A.shape
                assert st['touched_columns'] == np.unique(A.col).size
                assert st['max_row_nnz'] == np.bincount(A.row, minlength=A.shape[0]).max()
                assert torch.equal(plan.col.cpu(), torch.from_numpy(A.col.astype(np.int32)))


def test_plan_census_of_heavy_rows():
    rng = np.random.Generator(np.random.PCG64(15))
    A = random_coo(rng, 60, 500, 800, heavy=[(4, 300), (40, 101)])
    st = make_plan(A, heavy_threshold=100, chunk=64).stats()
    deg = np.bincount(A.row, minlength=60)
    assert st['heavy_rows'] == int((deg > 100).sum()) == 2
    assert st['heavy_chunks'] == sum(-(-int(d) // 64) for d in deg if d > 100)
    assert st['heavy_nnz'] == int(deg[deg > 100].sum())


def test_bad_input_is_rejected_before_any_product():
    import spmm_cpp
    row = torch.tensor([0, 2, 1], dtype=torch.int32, device='cuda')      # not ascending
    col = torch.tensor([0, 1, 1], dtype=torch.int32, device='cuda')
    val = torch.ones(3, device='cuda')
    with pytest.raises(RuntimeError, match='row-sorted'):
        spmm_cpp.SpmmPlan(row, col, val, 3, 2)
    with pytest.raises(RuntimeError, match='row-sorted'):                 # column id outside the matrix
        spmm_cpp.SpmmPlan(torch.tensor([0, 1, 2], dtype=torch.int32, device='cuda'), torch.tensor([0, 5, 1], dtype=torch.int32, device='cuda'), val, 3, 2)
    with pytest.raises(RuntimeError, match='CUDA tensor'):
        spmm_cpp.spmm_cusparse(row.cpu(), col.cpu(), val.cpu(), 3, 2, torch.ones(2, 4), torch.ones(3, 4), 1, 1)
    plan = spmm_cpp.SpmmPlan(torch.tensor([0, 1, 2], dtype=torch.int32, device='cuda'), col, val, 3, 2)
    with pytest.raises(RuntimeError):
        plan.spmm(torch.ones(3, 4, device='cuda'), torch.ones(3, 4, device='cuda'))     # B has the wrong row count
    L = spmm_cpp.lib()
    assert L.dg_spmm_csr(None, None, None, 4, None, 4, 4, 1.0, 1.0, 0, None, None, None) == -1
    assert L.dg_spmm_csr(plan.handle, val.data_ptr(), val.data_ptr(), 2, val.data_ptr(), 4, 4, 1.0, 1.0, 0, None, None, None) == -2
    assert L.dg_spmm_csr(plan.handle, val.data_ptr(), val.data_ptr(), 4, val.data_ptr(), 4, 4, 1.0, 1.0, 64, None, None, None) == -4
    assert b'NULL' in L.dg_strerror(-1)
    # after all those refusals the context still computes
    C = torch.zeros(3, 1, device='cuda')
    plan.spmm(torch.ones(2, 1, device='cuda'), C, 1.0, 0.0)
    assert C.cpu().flatten().tolist() == [1.0, 1.0, 1.0]


def _emulated_bcast(parted):
    """One distributed SpMM for P ranks emulated on one GPU: rank r adds plan(A[r][s]) @ X_s for s = 0..P-1 in order."""
    plans = [[make_plan(a) for a in p['adj_parts']] for p in parted]

    def bcast(blocks):
        xs = [dev(np.ascontiguousarray(b)) for b in blocks]
        out = []
        for r in range(len(parted)):
            z = torch.empty_like(xs[r])
            for s, x in enumerate(xs):
                plans[r][s].spmm(x, z, 1.0, 0.0 if s == 0 else 1.0)
            out.append(z.cpu().numpy())
        return out
    return bcast


def test_stage_loop_values_match_reference_run_over_gloo(golden):
    """Every broadcast-SpMM result of the reference's epoch 0 at P=2 (3 forward, 3 backward), with the CUDA kernels
    doing the sparse products and the oracle doing the dense algebra around them; then losses over 3 epochs."""
    from test_oracle_golden import _parted_from_fixture
    z, t = golden('graph_small'), golden('gcn_small')
    parted = _parted_from_fixture(z, 2)
    model = ref_gcn.GcnOracle(_emulated_bcast(parted), [t[f'r0/w0_{i}'] for i in range(3)], [[0, 1]])
    feats = [p['features'] for p in parted]
    for epoch in range(3):
        losses, outputs, trace, btrace = model.epoch(feats, [p['local_labels'] for p in parted], [p['local_train_mask'] for p in parted])
        for r in range(2):
            assert abs(losses[r] - t[f'r{r}/losses'][epoch]) <= 2e-5 * max(1.0, abs(t[f'r{r}/losses'][epoch]))
        if epoch == 0:
            for r in range(2):
                got = [trace[l]['z'][r] for l in range(3)] + [btrace[l]['ag'][r] for l in (2, 1, 0)]
                for i, g in enumerate(got):
                    assert_close(g, t[f'r{r}/bcast_{i}'], TOL, f'rank {r} bcast {i}')
                for l in range(3):
                    assert_close(btrace[l]['dw'][r], t[f'r{r}/dw_{l}'], TOL, f'dW{l}')


@pytest.mark.parametrize('P,c', [(4, 2), (8, 2), (9, 3)])
def test_15d_schedule_with_cuda_products_equals_1d_and_full_product(golden, P, c):
    """1.5D(P, c) == 1D(P/c) == single full product, the identity that pins the 1.5D schedule."""
    from dist_utils import schedule
    z = golden('graph_small')
    n_nodes = int(z['in/meta'][0])
    A = ref_graph.Coo(z['full/adj_idx'][0], z['full/adj_idx'][1], z['full/adj_val'], (n_nodes, n_nodes))
    R = P // c
    parts = [ref_graph.parted_graph(p) for p in ref_graph.partition(A, z['full/features'], z['in/labels'].astype(np.int64), z['in/masks'], R)]
    plans = [[make_plan(a) for a in p['adj_parts']] for p in parts]
    X = [dev(p['features']) for p in parts]
    rows_grp = schedule.row_groups(P, c)
    partial = []
    for rank in range(P):
        b = rank // c
        zr = torch.zeros_like(X[b])
        for st in schedule.stages_15d(rank, P, c):
            assert st.root_global // c == st.part and schedule.col_groups(P, c)[rank % c][st.root_in_group] == st.root_global
            plans[b][st.part].spmm(X[st.part], zr, 1.0, 1.0)
        partial.append(zr)
    full = ref_gcn.spmm_coo(A, np.ascontiguousarray(z['full/features']), np.zeros_like(z['full/features']), 1.0, 0.0)
    pad = parts[0]['adj'].shape[0] * R - n_nodes
    full = np.concatenate((full, np.zeros((pad, full.shape[1]), dtype=np.float32)))
    oracle_15d = ref_gcn.broadcast_15d([p['adj_parts'] for p in parts], [p['features'] for p in parts], P, c)
    n = parts[0]['adj'].shape[0]
    for grp in rows_grp:
        total = partial[grp[0]].clone()
        for r in grp[1:]:
            total += partial[r]
        b = grp[0] // c
        assert_close(total.cpu().numpy(), full[b * n:(b + 1) * n], TOL, f'block {b} vs full product')
        assert_close(total.cpu().numpy(), oracle_15d[grp[0]], TOL, f'block {b} vs 1.5D oracle')


@pytest.mark.parametrize('F', [64, 100, 128, 256, 300, 512, 1024])
@pytest.mark.parametrize('task', [5, 32, 100, 0])
def test_streaming_kernel_against_oracle(F, task):
    """Widths whose rows are 16-byte aligned take the bulk-copy streaming kernel; small task sizes cut rows at many task
    boundaries (carry rows + fix-up), 0 keeps the default.  Includes empty leading/trailing rows and a row spanning
    dozens of tasks."""
    rng = np.random.Generator(np.random.PCG64(1000 + F + task))
    A = random_coo(rng, 261, 190, 3500, heavy=[(7, 150), (200, 190)])
    keep = (A.row >= 3) & (A.row < 255) & (A.row != 100) & (A.row != 101)       # rows 0-2, 100-101, 255-260 are empty
    A = ref_graph.Coo(A.row[keep], A.col[keep], A.val[keep], A.shape)
    B = rng.standard_normal((190, F), dtype=np.float32)
    C0 = rng.standard_normal((261, F), dtype=np.float32)
    import spmm_cpp
    plan = make_plan(A).set_task_size(task)
    spmm_cpp.select_kernel('stream')
    try:
        for alpha, beta in ((1.0, 0.0), (0.75, -1.25)):
            want = ref_gcn.spmm_coo(A, B, C0.copy(), alpha, beta)
            C = dev(C0) if beta != 0 else torch.full((261, F), float('nan'), device='cuda')
            plan.spmm(dev(B), C, alpha, beta)
            assert_close(C.cpu().numpy(), want, TOL, f'F={F} task={task} beta={beta}')
    finally:
        spmm_cpp.select_kernel('auto')
    assert plan.device_status() == 0


def test_streaming_kernel_epilogue_and_reproducibility():
    rng = np.random.Generator(np.random.PCG64(77))
    A = random_coo(rng, 400, 300, 20000, heavy=[(0, 300), (399, 250)])
    B = rng.standard_normal((300, 256), dtype=np.float32)
    C0 = rng.standard_normal((400, 256), dtype=np.float32)
    scale = rng.uniform(0.1, 2.0, 400).astype(np.float32)
    bias = rng.standard_normal(256, dtype=np.float32)
    want = ref_gcn.spmm_epilogue(A, B, C0, 1.0, 0.5, row_scale=scale, bias=bias, relu=True)
    import spmm_cpp
    plan = make_plan(A).set_task_size(64)
    outs = []
    spmm_cpp.select_kernel('stream')
    try:
        for _ in range(3):
            C = dev(C0)
            plan.spmm(dev(B), C, 1.0, 0.5, row_scale=dev(scale), bias=dev(bias), relu=True)
            outs.append(C.cpu())
    finally:
        spmm_cpp.select_kernel('auto')
    assert_close(outs[0].numpy(), want, TOL, 'streaming epilogue')
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert plan.device_status() == 0
