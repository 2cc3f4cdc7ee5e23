"""dg_spmm_csr_static, the product variant for hosts that cannot let the library allocate device memory (their pool
owns all of it, or an allocation's device-wide synchronisation is not acceptable in their loop).  It must give what
dg_spmm_csr gives, call after call, while keeping its split-row partial sums in a fixed array inside the library.

Collected last on purpose: a failure here never hides another test's result in a run that stops at the first failure.
"""
import ctypes

import numpy as np
import pytest
import torch

from conftest import assert_close
from oracle import ref_gcn, ref_graph

pytestmark = pytest.mark.gpu
TOL = 1e-5


def _case(seed, m, k, nnz, heavy_rows):
    rng = np.random.Generator(np.random.PCG64(seed))
    flat = rng.choice(m * k, size=nnz, replace=False)
    row, col = flat // k, flat % k
    for r, cnt in heavy_rows:
        keep = row != r
        row, col = np.concatenate((row[keep], np.full(cnt, r))), np.concatenate((col[keep], rng.choice(k, cnt, replace=False)))
    val = rng.standard_normal(row.size, dtype=np.float32)
    return ref_graph.fast_coalesce_sorted(row.astype(np.int64), col.astype(np.int64), val, (m, k)), rng


def _call(fn, plan, B, C, alpha, beta, flags=0, row_scale=None, bias=None):
    F = B.size(1)
    return fn(plan.handle, plan.values.data_ptr(), B.data_ptr(), F, C.data_ptr(), F, F, alpha, beta, flags,
              row_scale.data_ptr() if row_scale is not None else None, bias.data_ptr() if bias is not None else None,
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_static_scratch_entry_matches_the_allocating_entry_twice_in_a_row():
    import spmm_cpp
    L = spmm_cpp.lib()
    A, rng = _case(31, 300, 400, 9000, [(2, 390), (150, 257), (299, 400)])
    dev = lambda a, dt=None: torch.from_numpy(np.ascontiguousarray(a)).to('cuda', dtype=dt)
    plan = spmm_cpp.SpmmPlan(dev(A.row, torch.int32), dev(A.col, torch.int32), dev(A.val), 300, 400, heavy_threshold=32, chunk=24)
    assert plan.stats()['heavy_chunks'] > 0                       # the scratch path is what this test is about
    assert L.dg_static_scratch_prepare() == 0                     # the one step that may touch the module loader
    for width, alpha, beta, flags in ((64, 1.0, 1.0, 0), (47, 0.5, 0.0, 4), (256, 1.25, -0.5, 0)):
        B_host = rng.standard_normal((400, width), dtype=np.float32)
        C_host = rng.standard_normal((300, width), dtype=np.float32)
        B, C0 = dev(B_host), dev(C_host)
        oracle = ref_gcn.spmm_epilogue(A, B_host, C_host, alpha, beta, relu=bool(flags & 4))     # the CPU restatement
        want = C0.clone()
        assert _call(L.dg_spmm_csr, plan, B, want, alpha, beta, flags) == 0
        for attempt in range(2):                                  # the array keeps the previous call's contents
            got = C0.clone()
            assert _call(L.dg_spmm_csr_static, plan, B, got, alpha, beta, flags) == 0
            torch.cuda.synchronize()
            assert_close(got.cpu().numpy(), oracle, TOL, f'F={width} call {attempt + 1} vs the oracle')
            assert_close(got.cpu().numpy(), want.cpu().numpy(), TOL, f'F={width} call {attempt + 1} vs dg_spmm_csr')
        # a different product in between must not leak into the next one
        other = torch.zeros(300, 8, device='cuda')
        assert _call(L.dg_spmm_csr_static, plan, torch.ones(400, 8, device='cuda'), other, 1.0, 0.0) == 0
    torch.cuda.synchronize()


def test_static_scratch_entry_refuses_requests_beyond_its_capacity():
    import spmm_cpp
    L = spmm_cpp.lib()
    cap = L.dg_static_scratch_capacity()
    assert cap == 4 * 1024 * 1024
    # 8192 split rows of 2 entries each with chunk = 1 -> 16384 chunks; F = 512 needs 8 Mi floats > capacity
    m = 8192
    row = torch.arange(m, dtype=torch.int32, device='cuda').repeat_interleave(2)
    col = torch.tensor([0, 1], dtype=torch.int32, device='cuda').repeat(m)
    plan = spmm_cpp.SpmmPlan(row, col, torch.ones(2 * m, device='cuda'), m, 2, heavy_threshold=1, chunk=1)
    assert plan.stats()['heavy_chunks'] == 2 * m
    B, C = torch.ones(2, 512, device='cuda'), torch.zeros(m, 512, device='cuda')
    assert _call(L.dg_spmm_csr_static, plan, B, C, 1.0, 0.0) == -6
    assert b'scratch' in L.dg_strerror(-6)
    assert float(C.abs().max()) == 0.0                            # nothing was launched
    B, C = torch.ones(2, 256, device='cuda'), torch.zeros(m, 256, device='cuda')       # exactly at the limit: accepted
    assert _call(L.dg_spmm_csr_static, plan, B, C, 1.0, 0.0) == 0
    assert torch.equal(C.cpu(), torch.full((m, 256), 2.0))
