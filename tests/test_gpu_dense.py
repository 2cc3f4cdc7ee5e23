"""The tcgen05 dense transform (three TF32 passes, fp32 accumulation in tensor memory) against float64.  Needs a GPU."""
import numpy as np
import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.mark.parametrize('M,K,N', [(128, 32, 16), (128, 256, 256), (1000, 256, 256), (300, 100, 256), (129, 256, 47),
                                   (5000, 32, 16), (77, 8, 8), (4096, 256, 128), (513, 100, 47), (400000, 256, 256)])
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


@pytest.mark.parametrize('M,K,N', [(29121, 602, 256), (1000, 64, 300), (3000, 256, 602), (515, 604, 41)])
def test_dense_nt_on_the_reddit_shaped_widths(M, K, N):
    """Config 1's layer shapes (602 -> 256 -> 41 on 29,121-row blocks): an inner dimension of 602 read from rows padded to
    604 floats, and results wider than one 256-column accumulator computed in panels."""
    import spmm_cpp
    g = torch.Generator(device='cuda').manual_seed(M + K + N)
    wide = torch.randn(M, K + (-K) % 4, device='cuda', generator=g)
    a = wide[:, :K]                                                # what the stage loop hands over for K = 602
    w = torch.randn(K, N, device='cuda', generator=g)              # layer weight [in x out]
    c = spmm_cpp.dense_nt(a, w, transposed=True, relu=True)
    assert c is not None and c.shape == (M, N)
    want = (a.double() @ w.double()).clamp(min=0)
    assert_close(c.cpu().numpy(), want.cpu().numpy(), TOL, f'{M}x{K}x{N}')
    # the split copy of a weight is kept until the weight changes in place
    p = torch.nn.Parameter(w.clone())
    first = spmm_cpp.dense_nt(a, p, transposed=True, cache_key=p)
    assert torch.equal(first, spmm_cpp.dense_nt(a, p, transposed=True, cache_key=p))
    with torch.no_grad():
        p.mul_(2.0)
    assert_close(spmm_cpp.dense_nt(a, p, transposed=True, cache_key=p).cpu().numpy(), (2 * (a.double() @ w.double())).cpu().numpy(), TOL, 'after an in-place update')
    assert spmm_cpp.dense_status() == 0


@pytest.mark.parametrize('n,Km,Nn', [(29121, 602, 256), (2000, 300, 300), (777, 256, 602), (4100, 604, 44)])
def test_dense_tn_in_panels(n, Km, Nn):
    """Weight gradients wider than two accumulators (config 1: X^T * AG with 602 input features) as 256 x 256 panels."""
    import spmm_cpp
    g = torch.Generator(device='cuda').manual_seed(n + Km + Nn)
    x = torch.randn(n, Km + (-Km) % 4, device='cuda', generator=g)[:, :Km]
    y = torch.randn(n, Nn + (-Nn) % 4, device='cuda', generator=g)[:, :Nn]
    d = spmm_cpp.dense_tn(x, y)
    assert d is not None and d.shape == (Km, Nn)
    assert_close(d.cpu().numpy(), (x.double().t() @ y.double()).cpu().numpy(), TOL, f'{n}x{Km}x{Nn}')
    assert torch.equal(d, spmm_cpp.dense_tn(x, y))
    assert spmm_cpp.dense_status() == 0


def test_dense_mm_pads_odd_row_strides_instead_of_leaving_the_tensor_cores():
    """models.gcn.dense_mm on operands whose rows are not 16-byte multiples (602 input features, 41 classes, contiguous):
    they are copied once into padded rows and still run on the hand-written kernels (the launch counter moves)."""
    import spmm_cpp
    from models.gcn import dense_mm
    g = torch.Generator(device='cuda').manual_seed(602)
    x = torch.randn(5000, 602, device='cuda', generator=g)
    ag = torch.randn(5000, 41, device='cuda', generator=g)
    w = torch.randn(602, 41, device='cuda', generator=g)
    before = spmm_cpp.dense_launches
    dw = dense_mm(x, ag, ta=True, constant_a=True)
    out = dense_mm(x, w)
    dx = dense_mm(ag, w, tb=True)
    assert spmm_cpp.dense_launches > before + 3
    assert_close(dw.cpu().numpy(), (x.double().t() @ ag.double()).cpu().numpy(), TOL, 'dW 602 x 41')
    assert_close(out.cpu().numpy(), (x.double() @ w.double()).cpu().numpy(), TOL, 'X W')
    assert_close(dx.cpu().numpy(), (ag.double() @ w.double().t()).cpu().numpy(), TOL, 'AG W^T, 602 wide')
    assert spmm_cpp.dense_status() == 0


def test_bounded_wait_gives_up_and_leaves_the_context_usable():
    """The dense kernels bound every mbarrier wait.  dg_dense_wait_selftest runs that path on purpose - a wait on a barrier
    nothing arrives at, with a short limit - and must report that the wait ran out, free its tensor memory and return;
    the real kernels then run as before and their status word is untouched."""
    import spmm_cpp
    assert spmm_cpp.dense_wait_selftest() is True
    a = torch.randn(300, 64, device='cuda')
    w = torch.randn(64, 32, device='cuda')
    c = spmm_cpp.dense_nt(a, w, transposed=True)                   # needs the tensor memory the self-test held
    assert_close(c.cpu().numpy(), (a.double() @ w.double()).cpu().numpy(), TOL, 'product after the self-test')
    assert spmm_cpp.dense_status() == 0
    spmm_cpp.check_dense_status()


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
    assert spmm_cpp.dense_tn(torch.randn(100, 47, device='cuda'), torch.randn(100, 16, device='cuda')) is None      # 188-byte rows
