"""TEST INFRASTRUCTURE: CPU oracle of the distributed SpMM stage loops and the GCN epoch built on them.

All P ranks are simulated inside one process: a "broadcast" is a plain read of the root rank's block,
an "all-reduce" is a sum over the participating ranks in ascending rank order.  The local sparse
product is the C restatement in spmm_ref.c (via ctypes) or, for the timed CPU baseline, torch's own
sparse addmm_ - the call the reference makes on CPU (light_dist_gnn/models/gcn.py:13).

Follows, by reference file:line:
  broadcast_1d        light_dist_gnn/models/gcn.py:16-30        (1D stage loop, stages in ascending root order)
  layer_forward       light_dist_gnn/models/gcn.py:35-42
  layer_backward      light_dist_gnn/models/gcn.py:45-53        (row block of A reused un-transposed; dW summed over ranks)
  gcn_forward         light_dist_gnn/models/gcn.py:68-72        (ReLU between layers, none after the last)
  epoch               light_dist_gnn/dist_train.py:36-46        (CE mean over LOCAL train rows, Adam lr 0.01)
  groups_15d          1D_CAGNET/utils.py:21-24, :36-49          (row groups = consecutive c ranks, column groups = stride c)
  stages_15d          1D_CAGNET/dist_15d.py:64-76               (stage count, column block and root per stage)
  broadcast_15d       1D_CAGNET/dist_15d.py:61-106              (column-group broadcast, row-group all-reduce of the partial z)
  dW all-reduce 1.5D  1D_CAGNET/dist_15d.py:29                  (over the column group only)

Parity status: the 1D functions are pinned against the reference run over gloo (tests/golden/); the
1.5D script of the reference cannot run (undefined attributes, removed native dependencies), so the
1.5D functions are pinned only through the identity  1.5D(P, c) == 1D(P/c) == single-process product.
"""
import ctypes
import os

import numpy as np

from . import ref_graph

_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), '_build', 'liboracle_spmm.so')
        if not os.path.exists(path):
            raise FileNotFoundError(f'{path} missing: run `make -C oracle`')
        _LIB = ctypes.CDLL(path)
        p = ctypes.c_void_p
        _LIB.oracle_spmm_csr.argtypes = [p, p, p, ctypes.c_int32, p, ctypes.c_int64, p, ctypes.c_int64,
                                         ctypes.c_int32, ctypes.c_float, ctypes.c_float, ctypes.c_int]
        _LIB.oracle_spmm_csr.restype = None
        _LIB.oracle_spmm_coo.argtypes = [p, p, p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, p, p,
                                         ctypes.c_int32, ctypes.c_float, ctypes.c_float, p, ctypes.c_int]
        _LIB.oracle_spmm_coo.restype = None
    return _LIB


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def spmm_coo(A, B, C, alpha=1.0, beta=1.0, threads=1):
    """C <- alpha*A*B + beta*C in place; A is a ref_graph.Coo, B and C contiguous fp32 arrays."""
    assert B.dtype == np.float32 and C.dtype == np.float32 and B.flags.c_contiguous and C.flags.c_contiguous
    assert B.shape[0] == A.shape[1] and C.shape == (A.shape[0], B.shape[1])
    row, col = A.row.astype(np.int32), A.col.astype(np.int32)
    val = np.ascontiguousarray(A.val, dtype=np.float32)
    scratch = np.empty(A.shape[0] + 1, dtype=np.int64)
    lib().oracle_spmm_coo(_ptr(row), _ptr(col), _ptr(val), A.nnz, A.shape[0], A.shape[1], _ptr(B), _ptr(C),
                          B.shape[1], alpha, beta, _ptr(scratch), threads)
    return C


def spmm_epilogue(A, B, C, alpha, beta, row_scale=None, bias=None, relu=False):
    """out = act(row_scale[i] * (alpha*A*B + beta*C)[i,:] + bias): the fused epilogue the CUDA kernel offers."""
    out = spmm_coo(A, B, C.copy(), alpha, beta)
    if row_scale is not None:
        out = (out * row_scale[:, None].astype(np.float32)).astype(np.float32)
    if bias is not None:
        out = (out + bias[None, :].astype(np.float32)).astype(np.float32)
    if relu:
        out = np.maximum(out, np.float32(0))
    return out


# ---------------------------------------------------------------- 1D
def broadcast_1d(adj_parts_by_rank, blocks):
    """z_r = sum_s A[r,s] * X_s for every rank r, stage s ascending (gcn.py:16-30)."""
    P = len(blocks)
    out = []
    for r in range(P):
        z = np.zeros_like(blocks[r])
        for src in range(P):
            spmm_coo(adj_parts_by_rank[r][src], np.ascontiguousarray(blocks[src]), z, 1.0, 1.0)
        out.append(z)
    return out


# ---------------------------------------------------------------- 1.5D
def groups_15d(P, c):
    rows = [list(range(i, i + c)) for i in range(0, P, c)]
    cols = [list(range(j, P, c)) for j in range(c)]
    return rows, cols


def stages_15d(rank, P, c):
    """[(column block id, root rank)] for one rank (dist_15d.py:64-76)."""
    rank_col = rank % c
    basic = P // (c * c)
    stages = basic if rank_col != c - 1 else P // c - (c - 1) * basic
    out = []
    for i in range(stages):
        part = rank_col * basic + i
        out.append((part, part * c + rank_col))
    return out


def broadcast_15d(adj_parts_by_block, blocks, P, c):
    """adj_parts_by_block[b][s], blocks[b] for the R = P/c row blocks; rank -> block rank//c.
    Returns z per RANK (all replicas of a row group hold the same reduced z)."""
    rows, _ = groups_15d(P, c)
    partial = []
    for rank in range(P):
        b = rank // c
        z = np.zeros_like(blocks[b])
        for part, root in stages_15d(rank, P, c):
            spmm_coo(adj_parts_by_block[b][part], np.ascontiguousarray(blocks[root // c]), z, 1.0, 1.0)
        partial.append(z)
    out = [None] * P
    for grp in rows:
        total = partial[grp[0]].copy()
        for r in grp[1:]:
            total = (total + partial[r]).astype(np.float32)
        for r in grp:
            out[r] = total
    return out


# ---------------------------------------------------------------- GCN on top of a stage loop
def _mm(a, b):
    return (a.astype(np.float32) @ b.astype(np.float32)).astype(np.float32)


class GcnOracle:
    """L-layer GCN over P simulated ranks.  `bcast(blocks)` is one distributed SpMM (list in, list out);
    `weight_groups` lists the rank groups whose dW are summed together (1D: one group of all ranks;
    1.5D: the column groups)."""

    def __init__(self, bcast, weights, weight_groups, block_of_rank=None):
        self.bcast, self.weight_groups = bcast, weight_groups
        self.weights = [w.astype(np.float32).copy() for w in weights]
        self.block_of_rank = block_of_rank
        self.adam = None

    def forward(self, feats):
        """feats: per-rank input blocks.  Returns outputs per rank and a trace of every intermediate."""
        trace, h = [], feats
        L = len(self.weights)
        for l, w in enumerate(self.weights):
            z = self.bcast(h)
            y = [_mm(zr, w) for zr in z]
            a = [np.maximum(yr, np.float32(0)) for yr in y] if l < L - 1 else y
            trace.append(dict(x=h, z=z, y=y, a=a))
            h = a
        return h, trace

    def backward(self, trace, grad_out):
        """grad_out: per-rank dLoss/dOutputs.  Returns dW per layer (after the all-reduce) and a trace."""
        L = len(self.weights)
        g, dws, btrace = grad_out, [None] * L, [None] * L
        for l in range(L - 1, -1, -1):
            if l < L - 1:   # ReLU backward
                g = [np.where(trace[l]['y'][r] > 0, g[r], np.float32(0)).astype(np.float32) for r in range(len(g))]
            ag = self.bcast(g)
            dx = [_mm(ag[r], self.weights[l].T) for r in range(len(g))]
            dw_local = [_mm(trace[l]['x'][r].T, ag[r]) for r in range(len(g))]
            dw = [None] * len(g)
            for grp in self.weight_groups:
                total = dw_local[grp[0]].copy()
                for r in grp[1:]:
                    total = (total + dw_local[r]).astype(np.float32)
                for r in grp:
                    dw[r] = total
            dws[l] = dw
            btrace[l] = dict(g=g, ag=ag, dx=dx, dw=dw)
            g = dx
        return dws, btrace

    @staticmethod
    def ce_loss_and_grad(outputs, labels, mask):
        """CrossEntropyLoss(mean) over the masked rows of one rank (dist_train.py:39-43); float64 inside."""
        grad = np.zeros_like(outputs)
        idx = np.flatnonzero(mask)
        if idx.size == 0:
            return 0.0, grad
        o = outputs[idx].astype(np.float64)
        o = o - o.max(axis=1, keepdims=True)
        logp = o - np.log(np.exp(o).sum(axis=1, keepdims=True))
        loss = -logp[np.arange(idx.size), labels[idx]].mean()
        p = np.exp(logp)
        p[np.arange(idx.size), labels[idx]] -= 1.0
        grad[idx] = (p / idx.size).astype(np.float32)
        return float(loss), grad

    def adam_step(self, dws_rank0, lr=0.01, b1=0.9, b2=0.999, eps=1e-8):
        """torch.optim.Adam defaults (dist_train.py:30); every rank holds the same dW so one copy is stepped."""
        if self.adam is None:
            self.adam = dict(t=0, m=[np.zeros_like(w) for w in self.weights], v=[np.zeros_like(w) for w in self.weights])
        st = self.adam
        st['t'] += 1
        for i, (w, g) in enumerate(zip(self.weights, dws_rank0)):
            st['m'][i] = (b1 * st['m'][i] + (1 - b1) * g).astype(np.float32)
            st['v'][i] = (b2 * st['v'][i] + (1 - b2) * g * g).astype(np.float32)
            step = lr / (1 - b1 ** st['t'])
            denom = np.sqrt(st['v'][i]) / np.float32(np.sqrt(1 - b2 ** st['t'])) + np.float32(eps)
            self.weights[i] = (w - np.float32(step) * st['m'][i] / denom).astype(np.float32)

    def epoch(self, feats, labels_local, masks_local):
        outputs, trace = self.forward(feats)
        losses, grads = zip(*[self.ce_loss_and_grad(outputs[r], labels_local[r], masks_local[r]) for r in range(len(feats))])
        dws, btrace = self.backward(trace, list(grads))
        self.adam_step([dws[l][0] for l in range(len(self.weights))])
        return list(losses), outputs, trace, btrace


def gcn_1d(parted, weights):
    """parted: list over ranks of ref_graph.parted_graph() dicts."""
    P = len(parted)
    adj = [p['adj_parts'] for p in parted]
    return GcnOracle(lambda blocks: broadcast_1d(adj, blocks), weights, [list(range(P))])


def gcn_15d(parted_blocks, weights, P, c):
    """parted_blocks: list over the R = P/c row blocks; rank r works on block r//c."""
    adj = [p['adj_parts'] for p in parted_blocks]
    _, cols = groups_15d(P, c)

    def bcast(per_rank):
        blocks = [per_rank[b * c] for b in range(P // c)]      # replicas of a row group hold equal blocks
        return broadcast_15d(adj, blocks, P, c)
    return GcnOracle(bcast, weights, cols)


# ---------------------------------------------------------------- timed CPU baseline (torch sparse path)
def cpu_epoch_sample(adj_block, x_full, labels, train_mask, weights, threads, stand_in_seed=0):
    """One GCN epoch of ONE rank's share, on the CPU, with the calls the reference makes on its CPU/gloo path:
    z.addmm_(A, B) for the sparse product (light_dist_gnn/models/gcn.py:13), torch.mm for the dense ones
    (gcn.py:41, :49-50), CrossEntropyLoss over the local train rows and Adam (dist_train.py:30-45).

    adj_block   torch sparse COO [n x N], the rank's row block of the normalised adjacency (all column blocks joined:
                the reference multiplies them one broadcast stage at a time, the work is the same)
    x_full      [N x d0] features of every rank (what the stage-loop broadcasts deliver for layer 1)
    For the deeper layers and for backward, the blocks other ranks would broadcast are stood in for by a fixed
    random [N x width] matrix whose rows [0, n) are overwritten with this rank's own activations / gradients; the
    arithmetic volume is exactly that of a rank in a 1D partition, with no communication time.
    Returns (seconds, loss)."""
    import time
    import torch
    torch.set_num_threads(threads)
    n, N = adj_block.shape
    gen = torch.Generator().manual_seed(stand_in_seed)
    widths = sorted({w.shape[1] for w in weights})
    stand_in = {w: torch.randn(N, w, generator=gen) * 0.01 for w in widths}
    ws = [w.clone() for w in weights]
    L = len(ws)
    t0 = time.perf_counter()
    # forward
    xs, zs, ys = [], [], []
    b_full = x_full
    for l, w in enumerate(ws):
        z = torch.zeros(n, b_full.shape[1])
        z.addmm_(adj_block, b_full)
        y = torch.mm(z, w)
        xs.append(b_full[:n])
        zs.append(z)
        ys.append(y)
        if l < L - 1:
            b_full = stand_in[y.shape[1]]
            b_full[:n] = torch.relu(y)
    out = ys[-1].requires_grad_(True)
    idx = train_mask.nonzero().squeeze(1)
    loss = torch.nn.functional.cross_entropy(out[idx], labels[idx]) if idx.numel() else (out * 0).sum()
    g = torch.autograd.grad(loss, out)[0]
    # backward
    grads = [None] * L
    for l in range(L - 1, -1, -1):
        if l < L - 1:
            g = g * (ys[l] > 0)
        g_full = stand_in[g.shape[1]]
        g_full[:n] = g
        ag = torch.zeros(n, g.shape[1])
        ag.addmm_(adj_block, g_full)
        grads[l] = torch.mm(xs[l].t(), ag)
        g = torch.mm(ag, ws[l].t())
    # Adam, first step (m = (1-b1) g, v = (1-b2) g^2)
    for l in range(L):
        m, v = 0.1 * grads[l], 0.001 * grads[l] * grads[l]
        ws[l] = ws[l] - 0.01 * (m / 0.1) / ((v / 0.001).sqrt() + 1e-8)
    return time.perf_counter() - t0, float(loss.detach())
