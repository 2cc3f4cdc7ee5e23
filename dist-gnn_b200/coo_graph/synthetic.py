"""Seeded synthetic datasets that stand in for the public graphs the reference trains on.

The reference downloads Reddit / ogbn-products style datasets
(light_dist_gnn/coo_graph/datasets.py:86-108) and stores them through
``save_dataset`` (datasets.py:15-31).  Those datasets are not available offline,
so this module draws R-MAT graphs with the same shapes and writes them through
the same ``save_dataset`` call, which makes every loader downstream behave as it
does on a real dataset.

Everything integer (edges, permutation, labels, split) comes from a counter
based 32-bit hash evaluated with plain integer tensor arithmetic, so the CPU and
the GPU produce bit-identical graphs and any rank can regenerate the data from
the seed alone.  Features and weights are floating point and come from a seeded
NumPy ``Generator`` on the host (moved to the device afterwards), or from a
seeded device generator for sweeps too large for host memory.

Generator rules (these are the contract the CPU oracle restates):

* scale = ceil(log2 N); draw ``e`` picks one quadrant per level, most
  significant bit first, from ``hash32(e, key(seed, STREAM_RMAT, level))``
  compared with the cumulative thresholds floor(a*2^32), floor((a+b)*2^32),
  floor((a+b+c)*2^32); quadrant b sets the column bit, c the row bit, d both.
* a draw is kept if both endpoints are < N and differ; it stands for the
  undirected edge {min, max}.
* the graph is the first ``target_directed // 2`` DISTINCT undirected edges in
  draw order (so the result does not depend on how many draws a batch made).
* vertex ids are then relabelled by ``perm = argsort(hash32(i, key(seed,
  STREAM_PERM, 0)))`` (stable) unless ``permute=False``.
* the directed edge list is all (u, v) followed by all (v, u).
"""
import math

import numpy as np
import torch

M32 = 0xFFFFFFFF
M64 = 0xFFFFFFFFFFFFFFFF
STREAM_RMAT, STREAM_PERM, STREAM_LABEL, STREAM_SPLIT = 0, 1, 2, 3
RMAT_ABCD = (0.57, 0.19, 0.19, 0.05)


def stream_key(seed, stream, level):
    """Two 32-bit constants for one (seed, stream, level), from a splitmix64 finaliser on Python ints."""
    z = (seed * 0x9E3779B97F4A7C15 + stream * 0xBF58476D1CE4E5B9 + level * 0x94D049BB133111EB + 0x1234567) & M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
    z ^= z >> 31
    return z & M32, z >> 32


def _fmix32(x):
    # x: int64 tensor whose values lie in [0, 2^32).  The products may wrap past 2^63; the
    # mask keeps the low 32 bits, which two's complement leaves exact.
    x = x ^ (x >> 16)
    x = (x * 0x85EBCA6B) & M32
    x = x ^ (x >> 13)
    x = (x * 0xC2B2AE35) & M32
    return x ^ (x >> 16)


def hash32(idx, key):
    """Counter-based hash: idx is an int64 tensor of counters < 2^32, key a pair from stream_key."""
    k1, k2 = key
    return _fmix32(_fmix32((idx + k1) & M32) ^ k2)


def _rmat_draws(first, count, num_nodes, seed, abcd, device):
    """Endpoints of draws [first, first+count): two int64 tensors (may be >= num_nodes)."""
    a, b, c, _ = abcd
    ta, tab, tabc = int(a * 2**32), int((a + b) * 2**32), int((a + b + c) * 2**32)
    scale = max(1, math.ceil(math.log2(num_nodes)))
    e = torch.arange(first, first + count, dtype=torch.int64, device=device)
    r = torch.zeros_like(e)
    col = torch.zeros_like(e)
    for level in range(scale):
        u = hash32(e, stream_key(seed, STREAM_RMAT, level))
        rbit = (u >= tab).to(torch.int64)
        cbit = (((u >= ta) & (u < tab)) | (u >= tabc)).to(torch.int64)
        r = (r << 1) | rbit
        col = (col << 1) | cbit
    return r, col


def rmat_undirected(num_nodes, target_directed, seed, abcd=RMAT_ABCD, device='cpu', max_rounds=12):
    """The first target_directed//2 distinct undirected edges in draw order, as (lo, hi) int64 tensors."""
    need = target_directed // 2
    if need > num_nodes * (num_nodes - 1) // 2:
        raise ValueError('more undirected edges requested than the graph can hold')
    if num_nodes * num_nodes >= 2**62:
        raise ValueError('graph too large for the 62-bit edge key')
    draws = int(need * 1.12) + 4096
    for _ in range(max_rounds):
        if draws >= 2**32:
            raise ValueError('graph needs more draws than the 32-bit draw counter holds')
        r, c = _rmat_draws(0, draws, num_nodes, seed, abcd, device)
        valid = (r < num_nodes) & (c < num_nodes) & (r != c)
        e = torch.nonzero(valid).squeeze(1)
        key = torch.minimum(r[e], c[e]) * num_nodes + torch.maximum(r[e], c[e])
        del r, c, valid
        key, order = torch.sort(key, stable=True)
        e = e[order]
        del order
        first = torch.ones_like(key, dtype=torch.bool)
        first[1:] = key[1:] != key[:-1]
        key, e = key[first], e[first]          # distinct keys with the index of their first draw
        if key.numel() >= need:
            keep = torch.sort(e).indices[:need]  # the `need` earliest first-draws
            key = torch.sort(key[keep]).values
            return key // num_nodes, key % num_nodes
        draws = int(draws * 1.6) + 4096
    raise RuntimeError('R-MAT oversampling did not reach the requested number of distinct edges')


def vertex_permutation(num_nodes, seed, device='cpu'):
    i = torch.arange(num_nodes, dtype=torch.int64, device=device)
    return torch.sort(hash32(i, stream_key(seed, STREAM_PERM, 0)), stable=True).indices


def rmat_edge_index(num_nodes, target_directed, seed, abcd=RMAT_ABCD, permute=True, device='cpu'):
    """Symmetrised, deduplicated, loop-free directed edge list [2, E] (int64), E = 2*(target//2)."""
    lo, hi = rmat_undirected(num_nodes, target_directed, seed, abcd, device)
    if permute:
        perm = vertex_permutation(num_nodes, seed, device)
        lo, hi = perm[lo], perm[hi]
    return torch.stack((torch.cat((lo, hi)), torch.cat((hi, lo))))


def uniform_labels(num_nodes, num_classes, seed, device='cpu'):
    i = torch.arange(num_nodes, dtype=torch.int64, device=device)
    return hash32(i, stream_key(seed, STREAM_LABEL, 0)) % num_classes


def random_split(num_nodes, fractions, seed, device='cpu'):
    """Three disjoint boolean masks; the first two sized floor(frac*N), the third takes the rest."""
    i = torch.arange(num_nodes, dtype=torch.int64, device=device)
    order = torch.sort(hash32(i, stream_key(seed, STREAM_SPLIT, 0)), stable=True).indices
    n_train, n_val = int(fractions[0] * num_nodes), int(fractions[1] * num_nodes)
    masks = [torch.zeros(num_nodes, dtype=torch.bool, device=device) for _ in range(3)]
    masks[0][order[:n_train]] = True
    masks[1][order[n_train:n_train + n_val]] = True
    masks[2][order[n_train + n_val:]] = True
    return masks


def normal_features(num_nodes, dim, seed, device='cpu', on_device=False):
    """fp32 N(0,1) features.  Host NumPy stream by default (identical on every box); on_device=True
    draws on the device for sweeps whose operand would not fit host memory."""
    if on_device:
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        return torch.randn((num_nodes, dim), generator=g, device=device, dtype=torch.float32)
    rng = np.random.Generator(np.random.PCG64(seed))
    x = rng.standard_normal((num_nodes, dim), dtype=np.float32)
    return torch.from_numpy(x).to(device)


def glorot_weights(dims, seed):
    """Glorot-uniform weights [d_i, d_{i+1}] on the host from a NumPy stream (moved by the caller)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    out = []
    for fan_in, fan_out in zip(dims[:-1], dims[1:]):
        bound = math.sqrt(6.0 / (fan_in + fan_out))
        out.append(torch.from_numpy(rng.uniform(-bound, bound, (fan_in, fan_out)).astype(np.float32)))
    return out


# Shapes of the benchmark configurations (graph, features, labels, split, model).
CONFIGS = {
    'plumbing': dict(num_nodes=10_000, directed_edges=200_000, feat_dim=128, num_classes=10,
                     split=(0.6, 0.2, 0.2), hidden=64, layers=2),
    'dense233k': dict(num_nodes=232_965, directed_edges=114_615_892, feat_dim=602, num_classes=41,
                      split=(0.66, 0.10, 0.24), hidden=256, layers=2),
    'sparse2m': dict(num_nodes=2_449_029, directed_edges=123_718_280, feat_dim=100, num_classes=47,
                     split=(0.08, 0.02, 0.90), hidden=256, layers=3),
}


def make_dataset(num_nodes, directed_edges, feat_dim, num_classes, split, seed=0, permute=True,
                 device='cpu', features_on_device=False, **_unused):
    """A dataset dict with the keys and dtypes ``save_dataset`` stores (datasets.py:29-31)."""
    edge_index = rmat_edge_index(num_nodes, directed_edges, seed, permute=permute, device=device)
    train, val, test = random_split(num_nodes, split, seed, device)
    return {
        'edge_index': edge_index.int(),
        'features': normal_features(num_nodes, feat_dim, seed, device, on_device=features_on_device),
        'labels': uniform_labels(num_nodes, num_classes, seed, device).char(),
        'train_mask': train, 'val_mask': val, 'test_mask': test,
        'num_nodes': num_nodes, 'num_edges': edge_index.size(1), 'num_classes': num_classes,
    }
