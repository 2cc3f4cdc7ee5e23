"""TEST INFRASTRUCTURE: NumPy restatement of the reference's graph preparation, and of the synthetic
generator rules, written as literally as possible (mask per block, sort + merge for coalesce) so it
shares no code and no shortcuts with the product's tensor implementation.

Follows, by reference file:line (light_dist_gnn/):
  add_self_loops      coo_graph/graph_utils.py:18-21
  sym_normalization   coo_graph/graph_utils.py:24-40
  sparse_2d_split     coo_graph/graph_utils.py:43-55
  preprocess          coo_graph/graph_utils.py:5-15
  partition           coo_graph/parted_coo_graph.py:63-93
  parted_graph        coo_graph/parted_coo_graph.py:97-111

Parity status: pinned against outputs of the reference code itself (tests/golden/, produced by
tests/golden/make_golden.py which imports the reference in the build container).
"""
import math

import numpy as np

M32 = np.uint64(0xFFFFFFFF)
_M64 = 0xFFFFFFFFFFFFFFFF


# ---------------------------------------------------------------- synthetic generator (restated rules)
def stream_key(seed, stream, level):
    z = (seed * 0x9E3779B97F4A7C15 + stream * 0xBF58476D1CE4E5B9 + level * 0x94D049BB133111EB + 0x1234567) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    z ^= z >> 31
    return z & 0xFFFFFFFF, z >> 32


def _fmix32(x):
    x = x ^ (x >> np.uint64(16))
    x = (x * np.uint64(0x85EBCA6B)) & M32
    x = x ^ (x >> np.uint64(13))
    x = (x * np.uint64(0xC2B2AE35)) & M32
    return x ^ (x >> np.uint64(16))


def hash32(idx, key):
    k1, k2 = key
    idx = idx.astype(np.uint64)
    return _fmix32(_fmix32((idx + np.uint64(k1)) & M32) ^ np.uint64(k2))


def rmat_edge_index(num_nodes, target_directed, seed, abcd=(0.57, 0.19, 0.19, 0.05), permute=True):
    """Walk the draws one batch at a time, keeping a Python set of the undirected edges seen so far,
    until target_directed//2 distinct ones exist (draw order decides which ones)."""
    a, b, c, _ = abcd
    ta, tab, tabc = int(a * 2**32), int((a + b) * 2**32), int((a + b + c) * 2**32)
    scale = max(1, math.ceil(math.log2(num_nodes)))
    need = target_directed // 2
    seen, lo_list, hi_list = set(), [], []
    first, batch = 0, max(1024, need // 4)
    while len(lo_list) < need:
        e = np.arange(first, first + batch, dtype=np.uint64)
        r = np.zeros(batch, dtype=np.int64)
        col = np.zeros(batch, dtype=np.int64)
        for level in range(scale):
            u = hash32(e, stream_key(seed, 0, level))
            rbit = u >= tab
            cbit = ((u >= ta) & (u < tab)) | (u >= tabc)
            r = r * 2 + rbit
            col = col * 2 + cbit
        for x, y in zip(r.tolist(), col.tolist()):
            if x >= num_nodes or y >= num_nodes or x == y:
                continue
            k = (min(x, y), max(x, y))
            if k in seen:
                continue
            seen.add(k)
            lo_list.append(k[0])
            hi_list.append(k[1])
            if len(lo_list) == need:
                break
        first += batch
    order = sorted(range(need), key=lambda i: (lo_list[i], hi_list[i]))
    lo = np.array([lo_list[i] for i in order], dtype=np.int64)
    hi = np.array([hi_list[i] for i in order], dtype=np.int64)
    if permute:
        perm = np.argsort(hash32(np.arange(num_nodes), stream_key(seed, 1, 0)), kind='stable')
        lo, hi = perm[lo], perm[hi]
    return np.stack((np.concatenate((lo, hi)), np.concatenate((hi, lo))))


def uniform_labels(num_nodes, num_classes, seed):
    return (hash32(np.arange(num_nodes), stream_key(seed, 2, 0)) % np.uint64(num_classes)).astype(np.int64)


def random_split(num_nodes, fractions, seed):
    order = np.argsort(hash32(np.arange(num_nodes), stream_key(seed, 3, 0)), kind='stable')
    n_train, n_val = int(fractions[0] * num_nodes), int(fractions[1] * num_nodes)
    masks = np.zeros((3, num_nodes), dtype=bool)
    masks[0, order[:n_train]] = True
    masks[1, order[n_train:n_train + n_val]] = True
    masks[2, order[n_train + n_val:]] = True
    return masks


# ---------------------------------------------------------------- COO helpers
class Coo:
    """A coalesced COO matrix: row/col int64 sorted row-major, val fp32, shape (m, k)."""

    def __init__(self, row, col, val, shape):
        self.row, self.col, self.val, self.shape = row, col, val, shape

    @property
    def nnz(self):
        return self.row.shape[0]

    def dense(self):
        d = np.zeros(self.shape, dtype=np.float64)
        np.add.at(d, (self.row, self.col), self.val.astype(np.float64))
        return d


def coalesce(row, col, val, shape):
    """Sort row-major and add duplicates in fp32, in their original order (what torch's CPU coalesce does)."""
    order = np.lexsort((col, row))  # stable: primary row, secondary col
    row, col, val = row[order], col[order], val[order]
    if row.size == 0:
        return Coo(row, col, val, shape)
    new = np.ones(row.size, dtype=bool)
    new[1:] = (row[1:] != row[:-1]) | (col[1:] != col[:-1])
    starts = np.flatnonzero(new)
    out = np.zeros(starts.size, dtype=np.float32)
    seg = np.cumsum(new) - 1
    for i in range(row.size):        # literal sequential fp32 accumulation; oracle sizes are small
        out[seg[i]] = np.float32(out[seg[i]] + val[i])
    return Coo(row[starts], col[starts], out, shape)


def add_self_loops(edge_index, num_nodes):
    mask = edge_index[0] != edge_index[1]
    loops = np.arange(num_nodes, dtype=edge_index.dtype)
    return np.concatenate((edge_index[:, mask], np.stack((loops, loops))), axis=1)


def sym_normalization(edge_index, num_nodes):
    ei = add_self_loops(edge_index.astype(np.int64), num_nodes)
    A = coalesce(ei[0], ei[1], np.ones(ei.shape[1], dtype=np.float32), (num_nodes, num_nodes))
    degree = np.zeros(num_nodes, dtype=np.float32)
    for c, v in zip(A.col.tolist(), A.val.tolist()):   # column sums, fp32, entry order
        degree[c] = np.float32(degree[c] + np.float32(v))
    d_rsqrt = np.power(degree, np.float32(-0.5), dtype=np.float32)
    da = (d_rsqrt[A.row] * A.val).astype(np.float32)            # D^-1/2 * A
    dad = (da * d_rsqrt[A.col]).astype(np.float32)              # (D^-1/2 A) * D^-1/2
    return Coo(A.row, A.col, dad, A.shape)


def sparse_2d_split(st, split_size, split_dim=0):
    size = st.shape[split_dim]
    seps = list(range(0, size, split_size)) + [size]
    split_idx = st.row if split_dim == 0 else st.col
    other_idx = st.col if split_dim == 0 else st.row
    parts = []
    for lower, upper in zip(seps[:-1], seps[1:]):
        mask = (split_idx < upper) & (split_idx >= lower)
        if split_dim == 0:
            parts.append(coalesce(split_idx[mask] - lower, other_idx[mask], st.val[mask], (upper - lower, st.shape[1])))
        else:
            parts.append(coalesce(other_idx[mask], split_idx[mask] - lower, st.val[mask], (st.shape[0], upper - lower)))
    return parts


def fast_coalesce_sorted(row, col, val, shape):
    """coalesce() for inputs known to hold no duplicates (vectorised; used for the larger oracle cases)."""
    order = np.lexsort((col, row))
    return Coo(row[order], col[order], val[order], shape)


def preprocess_features(features):
    s = features.sum(axis=1, keepdims=True, dtype=np.float32)
    return (features / np.maximum(s, np.float32(1))).astype(np.float32)


def partition(adj, features, labels, masks, num_parts):
    """Per-rank dicts as COO_Graph.partition stores them (padding=True)."""
    num_nodes = adj.shape[0]
    n = (num_nodes + num_parts - 1) // num_parts
    pad = n * num_parts - num_nodes
    adj_list = sparse_2d_split(adj, n)
    feat_list = [features[i:i + n] for i in range(0, num_nodes, n)]
    if pad > 0:
        feat_list[-1] = np.concatenate((feat_list[-1], np.zeros((pad, features.shape[1]), dtype=features.dtype)))
        labels = np.concatenate((labels, np.zeros((pad,) + labels.shape[1:], dtype=labels.dtype)))
        masks = np.concatenate((masks, np.zeros((3, pad), dtype=bool)), axis=1)
        adj_list = [Coo(a.row, a.col, a.val, (n, n * num_parts)) for a in adj_list]
    return [dict(adj=adj_list[r], features=feat_list[r], labels=labels, masks=masks, n=n, rank=r, num_parts=num_parts)
            for r in range(num_parts)]


def parted_graph(part):
    """What Parted_COO_Graph.__init__ derives from a stored part."""
    n, r = part['adj'].shape[0], part['rank']
    out = dict(part)
    out['local_labels'] = part['labels'][n * r:n * (r + 1)]
    out['local_train_mask'] = part['masks'][0][n * r:n * (r + 1)]
    out['adj_parts'] = sparse_2d_split(part['adj'], n, split_dim=1)
    return out


def rowptr_of(coo):
    """CSR row pointer (int64, m+1) of a coalesced COO."""
    return np.concatenate(([0], np.cumsum(np.bincount(coo.row, minlength=coo.shape[0])))).astype(np.int64)
