"""The tcgen05 dense transform (three TF32 passes, fp32 accumulation in tensor memory) against float64.  Needs a GPU."""
import numpy as np
import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.mark.parametrize('M,K,N', [(128, 32, 16), (128, 256, 256), (1000, 256, 256), (300, 100, 256), (129, 256, 47),
                                   (5000, 32, 16), (77, 8, 8), (4096, 256, 128), (513, 100, 47)])
def test_dense_nt_matches_float64(M, K, N):
    import spmm_cpp
    g = torch.Generator(device='cuda').manual_seed(M + K + N)
    a = torch.randn(M, K, device='cuda', generator=g)
    bt = torch.randn(N, K, device='cuda', generator=g)
    c = spmm_cpp.dense_nt(a, bt)
    assert c is not None and c.shape == (M, N)
    want = a.double() @ bt.double().t()
    assert_close(c.cpu().numpy(), want.cpu().numpy(), TOL, f'{M}x{K}x{N}')
    r = spmm_cpp.dense_nt(a, bt, relu=True)
    assert_close(r.cpu().numpy(), want.clamp(min=0).cpu().numpy(), TOL, f'relu {M}x{K}x{N}')
    assert spmm_cpp.dense_status() == 0


def test_dense_split_is_exact_and_unsupported_shapes_fall_back():
    import spmm_cpp
    w = torch.randn(64, 48, device='cuda')
    head, tail = spmm_cpp.dense_split(w)
    assert torch.equal(head + tail, w)
    assert torch.equal(head.view(torch.int32) & 8191, torch.zeros_like(head, dtype=torch.int32))
    assert spmm_cpp.dense_nt(torch.randn(100, 47, device='cuda'), torch.randn(16, 47, device='cuda')) is None     # 188-byte rows
    assert spmm_cpp.dense_nt(torch.randn(100, 64, device='cuda'), torch.randn(300, 64, device='cuda')) is None     # N > 256


@pytest.mark.parametrize('n,Km,Nn', [(16, 32, 16), (1000, 256, 256), (5000, 100, 256), (300, 128, 48), (70000, 256, 256),
                                     (33, 8, 8), (4099, 100, 64), (250000, 256, 128)])
def test_dense_tn_matches_float64(n, Km, Nn):
    import spmm_cpp
    g = torch.Generator(device='cuda').manual_seed(n + Km + Nn)
    x = torch.randn(n, Km, device='cuda', generator=g)
    y = torch.randn(n, Nn, device='cuda', generator=g)
    d = spmm_cpp.dense_tn(x, y)
    assert d is not None and d.shape == (Km, Nn)
    want = x.double().t() @ y.double()
    assert_close(d.cpu().numpy(), want.cpu().numpy(), TOL, f'{n}x{Km}x{Nn}')
    assert torch.equal(d, spmm_cpp.dense_tn(x, y))                 # partials are added in a fixed order
    assert spmm_cpp.dense_status() == 0


def test_dense_tn_error_does_not_grow_with_the_row_count():
    """All-positive operands over the full benchmark row count: the worst case for the truncating tensor-core accumulator,
    whose error without the periodic flush is 3e-4 here (and linear in the number of rows)."""
    import spmm_cpp
    n = 2449029
    g = torch.Generator(device='cuda').manual_seed(5)
    x = torch.rand(n, 256, device='cuda', generator=g)
    y = torch.rand(n, 256, device='cuda', generator=g)
    want = torch.zeros(256, 256, device='cuda', dtype=torch.float64)
    for s in range(0, n, 200000):
        want += x[s:s + 200000].double().t() @ y[s:s + 200000].double()
    d = spmm_cpp.dense_tn(x, y)
    assert_close(d.cpu().numpy(), want.cpu().numpy(), TOL, 'full-size weight gradient')
    assert spmm_cpp.dense_status() == 0


@pytest.mark.parametrize('M,N,K', [(1000, 256, 256), (777, 100, 48), (130, 47, 256)])
def test_dense_nt_mask_zeroes_where_the_activation_is_zero(M, N, K):
    import spmm_cpp
    g = torch.Generator(device='cuda').manual_seed(M + N)
    a = torch.randn(M, K, device='cuda', generator=g)
    bt = torch.randn(N, K, device='cuda', generator=g)
    act = torch.relu(torch.randn(M, N, device='cuda', generator=g))       # about half zeros, like a ReLU output
    out = spmm_cpp.dense_nt(a, bt, mask=act)
    plain = spmm_cpp.dense_nt(a, bt)
    assert out is not None and plain is not None
    assert torch.equal(out, plain * (act > 0))
    want = (a.double() @ bt.double().t()) * (act > 0)
    assert_close(out.cpu().numpy(), want.cpu().numpy(), TOL, f'masked {M}x{N}x{K}')
    with pytest.raises(RuntimeError):
        spmm_cpp.dense_nt(a, bt, mask=act[:, :-1])


def test_dense_kernels_take_column_slices_of_padded_buffers():
    """47 columns held in rows of 48 floats (what the stage loop returns for an odd class count): both products read the
    slice in place and ignore the padding column."""
    import spmm_cpp
    n = 20000
    g = torch.Generator(device='cuda').manual_seed(47)
    wide = torch.randn(n, 48, device='cuda', generator=g)
    ag = wide[:, :47]
    w = torch.randn(256, 47, device='cuda', generator=g)          # layer weight [in x out]: dX = AG * W^T
    h = torch.randn(n, 256, device='cuda', generator=g)
    dx = spmm_cpp.dense_nt(ag, w)
    assert dx is not None and dx.shape == (n, 256)
    assert_close(dx.cpu().numpy(), (ag.double() @ w.double().t()).cpu().numpy(), TOL, 'dX from a 47-of-48 slice')
    dw = spmm_cpp.dense_tn(h, ag)
    assert dw is not None and dw.shape == (256, 47)
    assert_close(dw.cpu().numpy(), (h.double().t() @ ag.double()).cpu().numpy(), TOL, 'dW from a 47-of-48 slice')
    with pytest.raises(RuntimeError):
        spmm_cpp.dense_tn(h, wide.t()[:47].t()[:, ::2])           # not row-major
    assert spmm_cpp.dense_status() == 0


def test_dense_tn_unsupported_shapes_fall_back():
    import spmm_cpp
    assert spmm_cpp.dense_tn(torch.randn(100, 47, device='cuda'), torch.randn(100, 16, device='cuda')) is None
    assert spmm_cpp.dense_tn(torch.randn(100, 64, device='cuda'), torch.randn(100, 300, device='cuda')) is None
