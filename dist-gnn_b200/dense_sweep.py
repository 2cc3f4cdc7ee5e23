"""Standalone sweep of the dense transforms around the SpMM (torch.mm at models/gcn.py:41 and :49-50 of the reference).

    python dist-gnn_b200/dense_sweep.py --rows 2449029 --shapes 256x256,100x256,256x47 --iters 10
    python dist-gnn_b200/dense_sweep.py --rows 400000 --shapes 256x256 --iters 2 --warmup 1        (profiler-sized)

For every K x N shape it prints two JSON lines, one for  C[rows x N] = A[rows x K] * W[K x N]  (dg_dense_nt) and one
for the weight gradient  D[K x N] = A[rows x K]^T * G[rows x N]  (dg_dense_tn): device time per call (CUDA events),
algorithmic GB/s (every operand read once, the result written once) against the measured HBM peak, effective TFLOP/s,
the library fp32 GEMM's time for the same product, and the error of both against a float64 product
(max |x - y| / max |y|).  Shapes the kernels do not take (row strides that are not multiples of 4 floats) print
"unsupported"; the model then uses the library GEMM for them.
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
if HERE not in sys.path:
    sys.path.insert(0, HERE)

import torch  # noqa: E402


def hbm_peak_gbs():
    path = os.path.join(os.path.dirname(HERE), 'MEASURED_PEAKS.json')
    try:
        with open(path) as f:
            return float(json.load(f)['hbm_gbs']), 'measured'
    except Exception:
        return 6650.0, 'fallback'


def timed(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def rel_err(x, want):
    return ((x.double() - want).abs().max() / want.abs().max()).item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--rows', type=int, default=2449029)
    ap.add_argument('--shapes', default='256x256,100x256,256x47')
    ap.add_argument('--iters', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--seed', type=int, default=0)
    ap.add_argument('--no-library', action='store_true', help='skip the library GEMM and the float64 check')
    args = ap.parse_args()

    import spmm_cpp
    if not torch.cuda.is_available():
        raise SystemExit('dense_sweep needs a CUDA device: the dense transforms have no CPU implementation')
    peak, peak_source = hbm_peak_gbs()
    g = torch.Generator(device='cuda').manual_seed(args.seed)
    n = args.rows
    for shape in args.shapes.split(','):
        K, N = (int(v) for v in shape.split('x'))
        a = torch.randn(n, K, device='cuda', generator=g)
        w = torch.randn(K, N, device='cuda', generator=g)
        gr = torch.randn(n, N, device='cuda', generator=g)
        wt = w.t().contiguous()
        for kind in ('nt', 'tn'):
            if kind == 'nt':
                ours, lib = (lambda: spmm_cpp.dense_nt(a, wt)), (lambda: torch.mm(a, w))
                alg_bytes = 4.0 * (n * K + K * N + n * N)
            else:
                ours, lib = (lambda: spmm_cpp.dense_tn(a, gr)), (lambda: torch.mm(a.t(), gr))
                alg_bytes = 4.0 * (n * K + n * N + K * N)
            line = {'product': f'{kind} rows={n} K={K} N={N}'}
            out = ours()
            if out is None:
                line['kernel'] = 'unsupported'
                print(json.dumps(line), flush=True)
                continue
            ms = timed(ours, args.iters, args.warmup)
            line.update(ms=round(ms, 4), alg_gbs=round(alg_bytes / ms / 1e6, 1), hbm_frac=round(alg_bytes / ms / 1e6 / peak, 3),
                        peak_gbs=peak, peak_source=peak_source, eff_tflops=round(2.0 * n * K * N / ms / 1e9, 1))
            if not args.no_library:
                line['library_fp32_ms'] = round(timed(lib, args.iters, args.warmup), 4)
                want = torch.zeros(out.shape, dtype=torch.float64, device='cuda')
                step = 200000
                for s in range(0, n, step):
                    if kind == 'nt':
                        want[s:s + step] = a[s:s + step].double() @ w.double()
                    else:
                        want += a[s:s + step].double().t() @ gr[s:s + step].double()
                line['rel_err'] = float(f'{rel_err(out, want):.3e}')
                line['library_rel_err'] = float(f'{rel_err(lib(), want):.3e}')
            line['status'] = spmm_cpp.dense_status()
            print(json.dumps(line), flush=True)
        del a, w, gr, wt


if __name__ == '__main__':
    main()
