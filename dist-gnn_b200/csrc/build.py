"""Builds libdist_gnn_b200.so (sm_100a only) in place with nvcc.  Usage: python dist-gnn_b200/csrc/build.py [-v]

The library links the NCCL that PyTorch bundles (headers and libnccl.so.2 from the `nvidia.nccl` wheel) so the
stage loop and torch.distributed share one NCCL in the process.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
SOURCES = ['dg_plan.cu', 'dg_spmm.cu', 'dg_spmm_stream.cu', 'dg_spmm_static.cu', 'dg_dense.cu', 'dg_pipeline.cu', 'dg_peer.cu']
OUTPUT = os.path.join(HERE, 'libdist_gnn_b200.so')


def nccl_paths():
    import importlib.util
    spec = importlib.util.find_spec('nvidia')
    for base in (spec.submodule_search_locations if spec else []):
        inc, lib = os.path.join(base, 'nccl', 'include'), os.path.join(base, 'nccl', 'lib')
        if os.path.exists(os.path.join(inc, 'nccl.h')) and os.path.exists(os.path.join(lib, 'libnccl.so.2')):
            return inc, lib
    return '/usr/include', '/usr/lib/x86_64-linux-gnu'


def command(verbose=False):
    inc, lib = nccl_paths()
    srcs = [os.path.join(HERE, s) for s in SOURCES if os.path.exists(os.path.join(HERE, s))]
    cmd = ['nvcc', '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
           '-Xcompiler', '-fPIC,-Wall', '-shared', '-I', os.path.join(ROOT, 'include'), '-I', inc,
           '-L', lib, '-l:libnccl.so.2', '-Xlinker', f'-rpath={lib}', '-o', OUTPUT] + srcs
    if verbose:
        cmd.insert(1, '-Xptxas=-v')
    return cmd, srcs


def up_to_date(srcs):
    if not os.path.exists(OUTPUT):
        return False
    deps = srcs + [os.path.join(HERE, 'dg_internal.h'), os.path.join(HERE, 'dg_comm.h'), os.path.join(ROOT, 'include', 'dist_gnn_b200.h'), __file__]
    return all(os.path.getmtime(d) <= os.path.getmtime(OUTPUT) for d in deps)


def build(verbose=False, force=False):
    cmd, srcs = command(verbose)
    if not force and not verbose and up_to_date(srcs):
        return OUTPUT
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode:
        raise RuntimeError('nvcc failed: ' + ' '.join(cmd))
    return OUTPUT


if __name__ == '__main__':
    print(build(verbose='-v' in sys.argv, force=True))
