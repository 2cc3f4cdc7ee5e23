import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, 'dist-gnn_b200')
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)
GOLDEN = os.path.join(ROOT, 'tests', 'golden')


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run on the B200 box)')
    os.environ.setdefault('DIST_GNN_DATA_ROOT', os.path.join('/tmp', f'dist_gnn_test_data_{os.getpid()}'))
    so = os.path.join(ROOT, 'oracle', '_build', 'liboracle_spmm.so')
    if not os.path.exists(so):
        subprocess.check_call(['make', '-C', os.path.join(ROOT, 'oracle')])


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason='no CUDA device')
    for item in items:
        if 'gpu' in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope='session')
def golden():
    cache = {}

    def load(name):
        if name not in cache:
            cache[name] = np.load(os.path.join(GOLDEN, name + '.npz'))
        return cache[name]
    return load


def rel_err(x, y):
    """max|x-y| / max|y| and Frobenius ratio, the two parity measures (both must be <= 1e-5)."""
    x, y = np.asarray(x, dtype=np.float64), np.asarray(y, dtype=np.float64)
    denom_max = max(np.abs(y).max() if y.size else 0.0, 1e-30)
    denom_fro = max(np.sqrt((y ** 2).sum()), 1e-30)
    return (np.abs(x - y).max() if y.size else 0.0) / denom_max, np.sqrt(((x - y) ** 2).sum()) / denom_fro


def assert_close(x, y, tol=1e-5, what=''):
    assert np.shape(x) == np.shape(y), f'{what}: shape {np.shape(x)} vs {np.shape(y)}'
    e_max, e_fro = rel_err(x, y)
    assert e_max <= tol and e_fro <= tol, f'{what}: rel max err {e_max:.3e}, rel fro err {e_fro:.3e} (tol {tol})'
