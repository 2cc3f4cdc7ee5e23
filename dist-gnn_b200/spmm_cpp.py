"""Python face of libdist_gnn_b200.so, under the module name the reference imports (``spmm_cpp``).

``spmm_cusparse(row, col, val, A_row, A_col, B, C, alpha, beta)`` keeps the nine-argument signature of the
reference's pybind module (light_dist_gnn/spmm_cpp/spmm.cpp:17, :35-37) and updates C in place, so
``from spmm_cpp import spmm_cusparse`` in light_dist_gnn/models/gcn.py:10 binds to the hand-written sm_100a kernels.
Everything goes through the C ABI of include/dist_gnn_b200.h with raw device pointers (ctypes); torch only owns
the memory and the streams.  There is no CPU implementation behind any of these calls: without the library or
without CUDA tensors they raise.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, 'csrc', 'libdist_gnn_b200.so')
_lib = None

EPI_ROW_SCALE, EPI_BIAS, EPI_RELU = 1, 2, 4


class PlanStats(ctypes.Structure):
    _fields_ = [('nnz', ctypes.c_int64), ('m', ctypes.c_int32), ('k', ctypes.c_int32),
                ('heavy_threshold', ctypes.c_int32), ('chunk', ctypes.c_int32),
                ('heavy_rows', ctypes.c_int32), ('heavy_chunks', ctypes.c_int32),
                ('heavy_nnz', ctypes.c_int64), ('max_row_nnz', ctypes.c_int64), ('touched_columns', ctypes.c_int64)]


class StageTimes(ctypes.Structure):
    _fields_ = [('comm_ms', ctypes.c_float), ('spmm_ms', ctypes.c_float), ('total_ms', ctypes.c_float),
                ('stages', ctypes.c_int32)]


class Profile(ctypes.Structure):
    _fields_ = [('spmm_ms', ctypes.c_double), ('alg_bytes', ctypes.c_double), ('gather_bytes', ctypes.c_double),
                ('flops', ctypes.c_double), ('products', ctypes.c_int64), ('kernel_launches', ctypes.c_int64)]


def lib():
    """The loaded C library; raises if it has not been built (python dist-gnn_b200/csrc/build.py)."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(f'{_LIB_PATH} is missing: build it with `python dist-gnn_b200/csrc/build.py`; '
                               'there is no fallback implementation')
        L = ctypes.CDLL(_LIB_PATH)
        vp, i32, i64, f32, u32 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_float, ctypes.c_uint32
        pp = ctypes.POINTER(ctypes.c_void_p)
        sig = {
            'dg_strerror': ([ctypes.c_int], ctypes.c_char_p),
            'dg_version': ([], ctypes.c_int),
            'dg_plan_create': ([vp, vp, i64, i32, i32, vp, pp], ctypes.c_int),
            'dg_plan_create_ex': ([vp, vp, i64, i32, i32, i32, i32, vp, pp], ctypes.c_int),
            'dg_plan_destroy': ([vp], ctypes.c_int),
            'dg_plan_get_stats': ([vp, ctypes.POINTER(PlanStats)], ctypes.c_int),
            'dg_plan_copy_rowptr': ([vp, vp, vp], ctypes.c_int),
            'dg_plan_set_task_size': ([vp, i32, vp], ctypes.c_int),
            'dg_plan_device_status': ([vp, ctypes.POINTER(ctypes.c_int), vp], ctypes.c_int),
            'dg_spmm_csr': ([vp, vp, vp, i64, vp, i64, i32, f32, f32, u32, vp, vp, vp], ctypes.c_int),
            'dg_spmm_csr_static': ([vp, vp, vp, i64, vp, i64, i32, f32, f32, u32, vp, vp, vp], ctypes.c_int),
            'dg_static_scratch_capacity': ([], ctypes.c_int64),
            'dg_static_scratch_prepare': ([], ctypes.c_int),
            'dg_spmm_coo': ([vp, vp, vp, i64, i32, i32, vp, vp, i32, f32, f32, vp], ctypes.c_int),
            'dg_comm_unique_id': ([ctypes.c_char_p], ctypes.c_int),
            'dg_comm_create': ([ctypes.c_char_p, ctypes.c_int, ctypes.c_int, pp], ctypes.c_int),
            'dg_comm_split': ([vp, ctypes.c_int, ctypes.c_int, pp], ctypes.c_int),
            'dg_comm_destroy': ([vp], ctypes.c_int),
            'dg_comm_rank': ([vp, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)], ctypes.c_int),
            'dg_comm_allreduce_sum': ([vp, vp, i64, vp], ctypes.c_int),
            'dg_comm_broadcast': ([vp, vp, i64, ctypes.c_int, vp], ctypes.c_int),
            'dg_bcast_spmm_1d': ([vp, i32, vp, i32, vp, vp, vp, i32, i32, vp, i32, vp, ctypes.c_int, vp], ctypes.c_int),
            'dg_bcast_spmm_15d': ([vp, vp, i32, vp, i32, vp, vp, vp, i32, i32, vp, i32, vp, ctypes.c_int, vp], ctypes.c_int),
            'dg_bcast_spmm_ordered': ([vp, vp, i32, vp, i32, vp, i32, vp, vp, vp, vp, vp, i32, i32, vp, ctypes.c_int, vp], ctypes.c_int),
            'dg_allgather_spmm': ([vp, vp, vp, vp, i32, i32, i32, vp, vp, vp, vp, ctypes.c_int, vp], ctypes.c_int),
            'dg_comm_last_times': ([vp, ctypes.POINTER(StageTimes)], ctypes.c_int),
            'dg_select_kernel': ([ctypes.c_int], ctypes.c_int),
            'dg_comm_peer_alloc': ([vp, i64, ctypes.c_char_p], ctypes.c_int),
            'dg_comm_peer_open': ([vp, ctypes.c_char_p], ctypes.c_int),
            'dg_comm_peer_close': ([vp], ctypes.c_int),
            'dg_comm_peer_capacity': ([vp], ctypes.c_int64),
            'dg_peer_spmm_packed': ([vp, vp, i32, vp, vp, vp, i32, vp, vp, vp, vp, i32, vp, vp, vp, vp, vp, i32, i32, vp, ctypes.c_int, vp], ctypes.c_int),
            'dg_peer_spmm': ([vp, vp, i32, vp, vp, i32, vp, vp, vp, vp, vp, i32, i32, vp, ctypes.c_int, vp], ctypes.c_int),
            'dg_peer_spmm_gather': ([vp, vp, i32, vp, vp, vp, vp, i32, vp, vp, vp, vp, vp, i32, i32, vp, ctypes.c_int, vp], ctypes.c_int),
            'dg_dense_split': ([vp, vp, vp, i64, vp], ctypes.c_int),
            'dg_dense_supported': ([i64, i32, i32, i64, i64, vp, vp, vp], ctypes.c_int),
            'dg_dense_nt': ([vp, i64, vp, vp, i64, vp, i64, i64, i32, i32, i32, vp], ctypes.c_int),
            'dg_dense_nt_masked': ([vp, i64, vp, vp, i64, vp, i64, i64, i32, i32, i32, vp, i64, vp], ctypes.c_int),
            'dg_dense_tn_supported': ([i64, i32, i32, i64, i64, vp, vp], ctypes.c_int),
            'dg_dense_tn': ([vp, i64, vp, i64, vp, i64, i64, i32, i32, vp, i64, i32, vp], ctypes.c_int),
            'dg_dense_status': ([ctypes.POINTER(ctypes.c_int), vp], ctypes.c_int),
            'dg_dense_status_reset': ([vp], ctypes.c_int),
            'dg_dense_wait_selftest': ([ctypes.POINTER(ctypes.c_int), vp], ctypes.c_int),
            'dg_profile_begin': ([], ctypes.c_int),
            'dg_profile_end': ([ctypes.POINTER(Profile)], ctypes.c_int),
        }
        for name, (argtypes, restype) in sig.items():
            fn = getattr(L, name)
            fn.argtypes, fn.restype = argtypes, restype
        _lib = L
    return _lib


def check(code):
    if code != 0:
        raise RuntimeError(f'dist_gnn_b200 error {code}: {lib().dg_strerror(code).decode()}')


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dev_tensor(t, dtype, what):
    if not (isinstance(t, torch.Tensor) and t.is_cuda):
        raise RuntimeError(f'{what} must be a CUDA tensor: this library has no CPU path')
    if t.dtype != dtype or not t.is_contiguous():
        raise RuntimeError(f'{what} must be a contiguous {dtype} tensor, got {t.dtype} contiguous={t.is_contiguous()}')
    return t


def _row_major(t, what):
    """Row stride (in floats) of a 2-D fp32 CUDA matrix whose rows are dense but may lie further apart than their
    length - a column slice of a wider buffer, as the stage loop returns for operands it padded."""
    if not (isinstance(t, torch.Tensor) and t.is_cuda):
        raise RuntimeError(f'{what} must be a CUDA tensor: this library has no CPU path')
    if t.dtype != torch.float32 or t.dim() != 2 or (t.size(1) > 1 and t.stride(1) != 1) or (t.size(0) > 1 and t.stride(0) < t.size(1)):
        raise RuntimeError(f'{what} must be a row-major fp32 matrix, got {t.dtype} {tuple(t.shape)} strides {t.stride()}')
    return t.stride(0) if t.size(0) > 1 else max(t.size(1), 1)


class SpmmPlan:
    """Device CSR plan of one sparse block (dg_plan).  Keeps the int32 column ids and fp32 values alive."""

    def __init__(self, row_i32, col_i32, values, m, k, heavy_threshold=0, chunk=0):
        _dev_tensor(row_i32, torch.int32, 'row ids'), _dev_tensor(col_i32, torch.int32, 'column ids')
        _dev_tensor(values, torch.float32, 'values')
        if not (row_i32.numel() == col_i32.numel() == values.numel()):
            raise RuntimeError('row, col and value arrays differ in length')
        self.col, self.values, self.m, self.k, self.device = col_i32, values, int(m), int(k), values.device
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            check(lib().dg_plan_create_ex(row_i32.data_ptr(), col_i32.data_ptr(), values.numel(), self.m, self.k,
                                          heavy_threshold, chunk, _stream(), ctypes.byref(handle)))
        self.handle = handle

    @classmethod
    def from_coo(cls, A, heavy_threshold=0, chunk=0):
        """From a coalesced torch sparse COO tensor on a CUDA device (int64 indices are narrowed once, here)."""
        if not A.is_coalesced():
            A = A.coalesce()
        idx = A.indices()
        if max(A.shape) >= 2**31:
            raise RuntimeError('block dimensions must fit int32')
        return cls(idx[0].to(torch.int32), idx[1].to(torch.int32).contiguous(), A.values().contiguous(),
                   A.size(0), A.size(1), heavy_threshold, chunk)

    def stats(self):
        s = PlanStats()
        check(lib().dg_plan_get_stats(self.handle, ctypes.byref(s)))
        return {name: getattr(s, name) for name, _ in PlanStats._fields_}

    def rowptr(self):
        out = torch.empty(self.m + 1, dtype=torch.int64)
        with torch.cuda.device(self.device):
            check(lib().dg_plan_copy_rowptr(self.handle, out.data_ptr(), _stream()))
        return out

    def set_task_size(self, task_nnz):
        """Entries per warp task of the streaming kernel (default 1024; <= 0 restores it)."""
        with torch.cuda.device(self.device):
            check(lib().dg_plan_set_task_size(self.handle, int(task_nnz), _stream()))
        return self

    def device_status(self):
        """0, or non-zero if a kernel of this plan gave up on a bounded wait (its result is then invalid)."""
        out = ctypes.c_int(-1)
        with torch.cuda.device(self.device):
            check(lib().dg_plan_device_status(self.handle, ctypes.byref(out), _stream()))
        return out.value

    def spmm(self, B, C, alpha=1.0, beta=1.0, row_scale=None, bias=None, relu=False, values=None):
        """C <- epilogue(alpha * A @ B + beta * C) in place; B [k, F] and C [m, F] may be row-strided views."""
        val = self.values if values is None else _dev_tensor(values, torch.float32, 'values')
        for t, rows, what in ((B, self.k, 'B'), (C, self.m, 'C')):
            if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.float32 and t.dim() == 2):
                raise RuntimeError(f'{what} must be a 2-D fp32 CUDA tensor')
            if t.size(0) != rows or (t.size(1) > 1 and t.stride(1) != 1):
                raise RuntimeError(f'{what} has shape {tuple(t.shape)} / strides {t.stride()}, expected {rows} rows, unit column stride')
        if B.size(1) != C.size(1):
            raise RuntimeError('B and C differ in width')
        flags = (EPI_ROW_SCALE if row_scale is not None else 0) | (EPI_BIAS if bias is not None else 0) | (EPI_RELU if relu else 0)
        if row_scale is not None:
            _dev_tensor(row_scale, torch.float32, 'row_scale')
        if bias is not None:
            _dev_tensor(bias, torch.float32, 'bias')
        F = B.size(1)
        ldb = B.stride(0) if B.size(0) > 1 else max(F, 1)
        ldc = C.stride(0) if C.size(0) > 1 else max(F, 1)
        with torch.cuda.device(self.device):
            check(lib().dg_spmm_csr(self.handle, val.data_ptr(), B.data_ptr(), ldb, C.data_ptr(), ldc, F, alpha, beta, flags,
                                    row_scale.data_ptr() if row_scale is not None else None,
                                    bias.data_ptr() if bias is not None else None, _stream()))
        return C

    def algorithmic_bytes(self, F, beta_nonzero):
        """Compulsory HBM traffic of one product: CSR once, each touched row of B once, C written once (and read once
        when accumulating): 8*nnz + 4*(m+1) + 4*F*touched + 4*F*m*(1 + [beta != 0]).  (The row offsets are int64
        here, so the real compulsory figure is 4*(m+1) bytes larger; the smaller one is the one reported.)"""
        s = self.stats()
        return 8 * s['nnz'] + 4 * (s['m'] + 1) + 4 * F * s['touched_columns'] + 4 * F * s['m'] * (2 if beta_nonzero else 1)

    def __del__(self):
        h, self.handle = getattr(self, 'handle', None), None
        if h and _lib is not None:
            _lib.dg_plan_destroy(h)


def select_kernel(family):
    """0 automatic (row kernels), 1 row kernels only, 2 streaming kernel where eligible; process-wide."""
    check(lib().dg_select_kernel({'auto': 0, 'rows': 1, 'stream': 2}.get(family, family)))


dense_launches = 0      # kernels launched by dense_split / dense_nt / dense_tn since the last profile_begin


def profile_begin():
    """Start bracketing every local product with CUDA events (dg_profile_begin)."""
    global dense_launches
    dense_launches = 0
    check(lib().dg_profile_begin())


def profile_end():
    """Synchronise and return the summed product time, traffic models, flops and kernel-launch count."""
    p = Profile()
    check(lib().dg_profile_end(ctypes.byref(p)))
    out = {name: getattr(p, name) for name, _ in Profile._fields_}
    out['dense_launches'] = dense_launches
    return out


_plan_cache = {}


def plan_for(A):
    """The cached SpmmPlan of a sparse COO block, built on first use and dropped when the tensor dies."""
    import weakref
    key = id(A)
    hit = _plan_cache.get(key)
    if hit is not None and hit[0]() is A:
        return hit[1]
    plan = SpmmPlan.from_coo(A)
    _plan_cache[key] = (weakref.ref(A, lambda _ref, key=key: _plan_cache.pop(key, None)), plan)
    return plan


_dropin_plans = {}          # (values pointer, nnz, rows, cols, device) -> (SpmmPlan, row ids, column ids), most recent last
DROPIN_PLAN_CACHE = 64      # plans kept for the nine-argument route; 0 builds a transient plan on every call


def spmm_cusparse(A_row_idx, A_col_idx, A_values, A_row, A_col, B, C, alpha, beta):
    """Drop-in for the reference's native op: C = alpha * A_coo @ B + beta * C, in place, on the current stream.

    The reference's binding (light_dist_gnn/models/gcn.py:11) hands over fresh int32 copies of the indices on every call,
    so a plan cannot be recognised by their addresses.  The values of a coalesced block do keep their address, so the plan
    of a block is looked up by (values address, nnz, shape) and accepted only if the incoming row and column ids equal the
    ones it was built from (two device comparisons, one host synchronisation); anything else builds a new plan.  On a
    306 k-row stage block of the benchmark graph that is 0.3 ms per call instead of 1.9 ms for a transient plan."""
    _dev_tensor(A_row_idx, torch.int32, 'A_row_idx'), _dev_tensor(A_col_idx, torch.int32, 'A_col_idx')
    _dev_tensor(A_values, torch.float32, 'A_values'), _dev_tensor(B, torch.float32, 'B'), _dev_tensor(C, torch.float32, 'C')
    if B.dim() != 2 or C.dim() != 2 or B.size(0) != A_col or C.size(0) != A_row or B.size(1) != C.size(1):
        raise RuntimeError(f'shape mismatch: A {A_row}x{A_col}, B {tuple(B.shape)}, C {tuple(C.shape)}')
    nnz = A_values.numel()
    if not (A_row_idx.numel() == A_col_idx.numel() == nnz):
        raise RuntimeError('row, col and value arrays differ in length')
    if DROPIN_PLAN_CACHE > 0 and nnz > 0:
        key = (A_values.data_ptr(), nnz, int(A_row), int(A_col), C.device.index)
        hit = _dropin_plans.pop(key, None)
        if hit is not None and not (torch.equal(hit[1], A_row_idx) and torch.equal(hit[2], A_col_idx)):
            hit = None                                                # same address, another matrix: forget the old plan
        if hit is None:
            row, col = A_row_idx.clone(), A_col_idx.clone()           # the plan borrows its column ids: keep private copies
            hit = (SpmmPlan(row, col, A_values, int(A_row), int(A_col)), row, col)
        _dropin_plans[key] = hit                                      # (re-)inserted last: the oldest entry goes first
        while len(_dropin_plans) > DROPIN_PLAN_CACHE:
            _dropin_plans.pop(next(iter(_dropin_plans)))
        hit[0].spmm(B, C, float(alpha), float(beta), values=A_values)
        return
    with torch.cuda.device(C.device):
        check(lib().dg_spmm_coo(A_row_idx.data_ptr(), A_col_idx.data_ptr(), A_values.data_ptr(), nnz,
                                int(A_row), int(A_col), B.data_ptr(), C.data_ptr(), B.size(1), float(alpha), float(beta), _stream()))


class Comm:
    """One NCCL communicator with its side stream (dg_comm)."""

    def __init__(self, handle, device):
        self.handle, self.device = handle, device
        r, n = ctypes.c_int(), ctypes.c_int()
        check(lib().dg_comm_rank(handle, ctypes.byref(r), ctypes.byref(n)))
        self.rank, self.size = r.value, n.value

    @staticmethod
    def unique_id():
        buf = ctypes.create_string_buffer(128)
        check(lib().dg_comm_unique_id(buf))
        return buf.raw

    @classmethod
    def create(cls, unique_id, rank, size, device):
        handle = ctypes.c_void_p()
        with torch.cuda.device(device):
            check(lib().dg_comm_create(unique_id, rank, size, ctypes.byref(handle)))
        return cls(handle, device)

    def split(self, color, key):
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            check(lib().dg_comm_split(self.handle, color, key, ctypes.byref(handle)))
        return Comm(handle, self.device) if handle.value else None

    def all_reduce_sum(self, t):
        _dev_tensor(t, torch.float32, 'tensor')
        with torch.cuda.device(self.device):
            check(lib().dg_comm_allreduce_sum(self.handle, t.data_ptr(), t.numel(), _stream()))

    def broadcast(self, t, root):
        _dev_tensor(t, torch.float32, 'tensor')
        with torch.cuda.device(self.device):
            check(lib().dg_comm_broadcast(self.handle, t.data_ptr(), t.numel(), root, _stream()))

    def last_times(self):
        s = StageTimes()
        with torch.cuda.device(self.device):
            check(lib().dg_comm_last_times(self.handle, ctypes.byref(s)))
        return dict(comm_ms=s.comm_ms, spmm_ms=s.spmm_ms, total_ms=s.total_ms, stages=s.stages)

    def peer_alloc(self, floats):
        """Allocates this rank's two send buffers of the peer-copy loop; returns their CUDA IPC handles (128 bytes)."""
        buf = ctypes.create_string_buffer(128)
        with torch.cuda.device(self.device):
            check(lib().dg_comm_peer_alloc(self.handle, int(floats), buf))
        return buf.raw

    def peer_open(self, handles):
        """Maps every rank's send buffers; handles: the peer_alloc results of all ranks in communicator rank order."""
        blob = b''.join(handles)
        if len(blob) != 128 * self.size:
            raise RuntimeError(f'expected {self.size} handle records of 128 bytes')
        with torch.cuda.device(self.device):
            check(lib().dg_comm_peer_open(self.handle, blob))

    def peer_close(self):
        with torch.cuda.device(self.device):
            check(lib().dg_comm_peer_close(self.handle))

    def peer_capacity(self):
        return int(lib().dg_comm_peer_capacity(self.handle))

    def destroy(self):
        h, self.handle = self.handle, None
        if h and _lib is not None:
            _lib.dg_comm_destroy(h)


def bcast_spmm(comm, roots, plans, x_local, recv, z, row_comm=None, timed=False, group=1):
    """The pipelined stage loop (dg_bcast_spmm_1d / _15d): z <- sum_s A_s @ X_{roots[s]}.

    comm is a Comm or None (single rank).  `group` consecutive stages share one product: plans[g] is the plan of the
    joined sparse block of stages [g*group, (g+1)*group), and recv holds >= 2 fp32 CUDA buffers of group*n*F floats."""
    _dev_tensor(x_local, torch.float32, 'x_local'), _dev_tensor(z, torch.float32, 'z')
    n, F = x_local.shape
    S = len(roots)
    if len(plans) != (S + group - 1) // group:
        raise RuntimeError(f'{S} stages in groups of {group} need {(S + group - 1) // group} plans, got {len(plans)}')
    roots_arr = (ctypes.c_int32 * max(S, 1))(*roots)
    plan_arr = (ctypes.c_void_p * max(len(plans), 1))(*[p.handle for p in plans])
    val_arr = (ctypes.c_void_p * max(len(plans), 1))(*[p.values.data_ptr() for p in plans])
    recv = recv or []
    for b in recv:
        _dev_tensor(b, torch.float32, 'receive buffer')
        if b.numel() < min(group, S) * n * F:
            raise RuntimeError('receive buffer smaller than one group of blocks')
    recv_arr = (ctypes.c_void_p * max(len(recv), 1))(*[b.data_ptr() for b in recv])
    args = (S, roots_arr, group, plan_arr, val_arr, x_local.data_ptr(), n, F, recv_arr, len(recv), z.data_ptr(), int(timed), _stream())
    with torch.cuda.device(x_local.device):
        if row_comm is None:
            check(lib().dg_bcast_spmm_1d(comm.handle if comm else None, *args))
        else:
            check(lib().dg_bcast_spmm_15d(comm.handle if comm else None, row_comm.handle, *args))
    return z


def bcast_spmm_ordered(comm, roots, landing, products, x_local, z, row_comm=None, timed=False, bcast_group=1, peer_copies=False):
    """dg_bcast_spmm_ordered: every broadcast queued up front, products in the given order.

    roots[s]     root (rank inside comm) of broadcast s; the same list on every rank
    landing[s]   fp32 CUDA tensor (n x F) receiving block s here, or None at a stage this rank roots
    products     list of (plan, operand tensor, last_stage): operand is x_local or a (k*n) x F view of the landing area,
                 last_stage the index of the last broadcast the product reads (-1: none)"""
    _dev_tensor(x_local, torch.float32, 'x_local'), _dev_tensor(z, torch.float32, 'z')
    n, F = x_local.shape
    S, P = len(roots), len(products)
    roots_arr = (ctypes.c_int32 * max(S, 1))(*roots)
    land_arr = (ctypes.c_void_p * max(S, 1))(*[None if t is None else _dev_tensor(t, torch.float32, 'landing block').data_ptr() for t in landing])
    plan_arr = (ctypes.c_void_p * max(P, 1))(*[p.handle for p, _, _ in products])
    val_arr = (ctypes.c_void_p * max(P, 1))(*[p.values.data_ptr() for p, _, _ in products])
    for plan, operand, _ in products:
        _dev_tensor(operand, torch.float32, 'operand')
        if operand.size(0) != plan.k or operand.size(1) != F:
            raise RuntimeError(f'operand {tuple(operand.shape)} does not match a plan with {plan.k} columns and width {F}')
    op_arr = (ctypes.c_void_p * max(P, 1))(*[t.data_ptr() for _, t, _ in products])
    last_arr = (ctypes.c_int32 * max(P, 1))(*[l for _, _, l in products])
    with torch.cuda.device(x_local.device):
        if peer_copies:
            check(lib().dg_peer_spmm(comm.handle, row_comm.handle if row_comm else None, S, roots_arr, land_arr, P, plan_arr,
                                     val_arr, op_arr, last_arr, x_local.data_ptr(), n, F, z.data_ptr(), int(timed), _stream()))
        else:
            check(lib().dg_bcast_spmm_ordered(comm.handle, row_comm.handle if row_comm else None, S, roots_arr, bcast_group, land_arr, P,
                                              plan_arr, val_arr, op_arr, last_arr, x_local.data_ptr(), n, F, z.data_ptr(), int(timed),
                                              _stream()))
    return z


def peer_spmm(comm, roots, landing, products, x_local, z, row_comm=None, timed=False):
    """dg_peer_spmm: the arguments of bcast_spmm_ordered, but every remote block is pulled from its root's send buffer
    by a device-to-device copy (Comm.peer_alloc / peer_open come first) and the stage order may differ per rank."""
    return bcast_spmm_ordered(comm, roots, landing, products, x_local, z, row_comm=row_comm, timed=timed, peer_copies=True)


def peer_spmm_packed(comm, packs, roots, stage_offsets, stage_rows, landing, products, x_local, z, row_comm=None, timed=False):
    """dg_peer_spmm_packed: peer_spmm that moves only the operand rows each reader's sparse block touches.

    packs          list of (row-id tensor (int32, CUDA, ascending), first row inside this rank's send buffer), one per reader
    roots[s], stage_offsets[s], stage_rows[s]   root of stage s, first row of this rank's list inside the root's send
                   buffer, and its length;  landing[s]: (stage_rows[s] x F) tensor, or None at an own stage
    products       (plan, operand, last_stage) as for peer_spmm; the plans of remote blocks use the packed numbering"""
    _dev_tensor(x_local, torch.float32, 'x_local'), _dev_tensor(z, torch.float32, 'z')
    n, F = x_local.shape
    Q, S, P = len(packs), len(roots), len(products)
    for rows, _ in packs:
        _dev_tensor(rows, torch.int32, 'pack row ids')
    pr = (ctypes.c_void_p * max(Q, 1))(*[rows.data_ptr() if rows.numel() else None for rows, _ in packs])
    pc = (ctypes.c_int64 * max(Q, 1))(*[rows.numel() for rows, _ in packs])
    po = (ctypes.c_int64 * max(Q, 1))(*[int(off) for _, off in packs])
    roots_arr = (ctypes.c_int32 * max(S, 1))(*roots)
    so = (ctypes.c_int64 * max(S, 1))(*[int(v) for v in stage_offsets])
    sr = (ctypes.c_int64 * max(S, 1))(*[int(v) for v in stage_rows])
    land_arr = (ctypes.c_void_p * max(S, 1))(*[None if t is None or t.numel() == 0 else _dev_tensor(t, torch.float32, 'landing block').data_ptr()
                                                for t in landing])
    for plan, operand, _ in products:
        _dev_tensor(operand, torch.float32, 'operand')
        if operand.size(0) != plan.k or operand.size(1) != F:
            raise RuntimeError(f'operand {tuple(operand.shape)} does not match a plan with {plan.k} columns and width {F}')
    plan_arr = (ctypes.c_void_p * max(P, 1))(*[p.handle for p, _, _ in products])
    val_arr = (ctypes.c_void_p * max(P, 1))(*[p.values.data_ptr() for p, _, _ in products])
    op_arr = (ctypes.c_void_p * max(P, 1))(*[t.data_ptr() for _, t, _ in products])
    last_arr = (ctypes.c_int32 * max(P, 1))(*[l for _, _, l in products])
    with torch.cuda.device(x_local.device):
        check(lib().dg_peer_spmm_packed(comm.handle, row_comm.handle if row_comm else None, Q, pr, pc, po, S, roots_arr, so, sr, land_arr,
                                        P, plan_arr, val_arr, op_arr, last_arr, x_local.data_ptr(), n, F, z.data_ptr(), int(timed), _stream()))
    return z


def peer_spmm_gather(comm, roots, stage_lists, stage_rows, landing, products, x_local, z, row_comm=None, timed=False):
    """dg_peer_spmm_gather: peer_spmm whose reader gathers, out of each root's whole block, only the rows its sparse block
    touches (a small pull kernel on the side stream; the owners pack nothing).

    roots[s], stage_lists[s], stage_rows[s]   root of stage s, the ascending row ids to fetch (int32 CUDA tensor; None at an
                   own stage) and their count;  landing[s]: (stage_rows[s] x F) tensor, or None at an own stage
    products       (plan, operand, last_stage) as for peer_spmm; the plans of remote blocks use the packed numbering"""
    _dev_tensor(x_local, torch.float32, 'x_local'), _dev_tensor(z, torch.float32, 'z')
    n, F = x_local.shape
    S, P = len(roots), len(products)
    for rows in stage_lists:
        if rows is not None:
            _dev_tensor(rows, torch.int32, 'stage row ids')
    roots_arr = (ctypes.c_int32 * max(S, 1))(*roots)
    lists_arr = (ctypes.c_void_p * max(S, 1))(*[None if t is None or t.numel() == 0 else t.data_ptr() for t in stage_lists])
    sr = (ctypes.c_int64 * max(S, 1))(*[int(v) for v in stage_rows])
    land_arr = (ctypes.c_void_p * max(S, 1))(*[None if t is None or t.numel() == 0 else _dev_tensor(t, torch.float32, 'landing block').data_ptr()
                                                for t in landing])
    for plan, operand, _ in products:
        _dev_tensor(operand, torch.float32, 'operand')
        if operand.size(0) != plan.k or operand.size(1) != F:
            raise RuntimeError(f'operand {tuple(operand.shape)} does not match a plan with {plan.k} columns and width {F}')
    plan_arr = (ctypes.c_void_p * max(P, 1))(*[p.handle for p, _, _ in products])
    val_arr = (ctypes.c_void_p * max(P, 1))(*[p.values.data_ptr() for p, _, _ in products])
    op_arr = (ctypes.c_void_p * max(P, 1))(*[t.data_ptr() for _, t, _ in products])
    last_arr = (ctypes.c_int32 * max(P, 1))(*[l for _, _, l in products])
    with torch.cuda.device(x_local.device):
        check(lib().dg_peer_spmm_gather(comm.handle, row_comm.handle if row_comm else None, S, roots_arr, lists_arr, sr, land_arr,
                                        P, plan_arr, val_arr, op_arr, last_arr, x_local.data_ptr(), n, F, z.data_ptr(), int(timed), _stream()))
    return z


def chunk_widths(F, target=64):
    """Column chunks for allgather_spmm: widths that are multiples of 4 (16-byte aligned pieces) near `target`, last one
    takes the rest.  Narrow or odd operands stay in one piece."""
    if F < 2 * target or F % 4:
        return [F]
    widths = [target] * (F // target)
    if F % target:
        widths[-1] += F % target
    return widths


def allgather_spmm(comm, plan, x_local, pack, area, z, widths, timed=False):
    """dg_allgather_spmm: z <- A_rowblock @ allgather(x) pipelined over column chunks of the given widths.

    plan   SpmmPlan of the rank's whole n x (P*n) row block;  pack / area: two fp32 CUDA buffers each, of at least
    n * max(widths) and P * n * max(widths) floats."""
    _dev_tensor(x_local, torch.float32, 'x_local'), _dev_tensor(z, torch.float32, 'z')
    n, F = x_local.shape
    w_arr = (ctypes.c_int32 * len(widths))(*widths)
    for t, need, what in ((pack[0], n, 'pack'), (pack[1], n, 'pack'), (area[0], n * comm.size, 'area'), (area[1], n * comm.size, 'area')):
        _dev_tensor(t, torch.float32, what + ' buffer')
        if t.numel() < need * max(widths):
            raise RuntimeError(f'{what} buffer too small')
    pack_arr = (ctypes.c_void_p * 2)(pack[0].data_ptr(), pack[1].data_ptr())
    area_arr = (ctypes.c_void_p * 2)(area[0].data_ptr(), area[1].data_ptr())
    with torch.cuda.device(x_local.device):
        check(lib().dg_allgather_spmm(comm.handle, plan.handle, plan.values.data_ptr(), x_local.data_ptr(), n, F, len(widths), w_arr,
                                      pack_arr, area_arr, z.data_ptr(), int(timed), _stream()))
    return z


def dense_split(w):
    """TF32-exact head and residual tail of a small fp32 CUDA matrix (dg_dense_split); head + tail == w exactly."""
    _dev_tensor(w, torch.float32, 'matrix')
    global dense_launches
    dense_launches += 1
    head, tail = torch.empty_like(w), torch.empty_like(w)
    with torch.cuda.device(w.device):
        check(lib().dg_dense_split(w.data_ptr(), head.data_ptr(), tail.data_ptr(), w.numel(), _stream()))
    return head, tail


_split_cache = {}       # id(weight object) -> (weak reference to it, {transposed flag: (version, head, tail)})


def split_operand(w, transposed, cache_key=None):
    """The small operand of dense_nt, laid out [N x K] (rows padded to a multiple of 4 floats) and split into TF32 head
    and tail.  transposed=True takes w as [K x N] and transposes it.  With cache_key (the weight object the caller holds,
    e.g. the nn.Parameter) the result is kept until that tensor is modified in place - its version counter moves with every
    optimiser step - so a weight is transposed and split once per step, not once per product."""
    if cache_key is not None:
        import weakref
        ident = id(cache_key)
        entry = _split_cache.get(ident)
        if entry is None or entry[0]() is not cache_key:       # tensors compare element-wise, so the table is keyed by identity
            entry = _split_cache[ident] = (weakref.ref(cache_key, lambda _r, ident=ident: _split_cache.pop(ident, None)), {})
        slot = entry[1]
        hit = slot.get(transposed)
        if hit is not None and hit[0] == cache_key._version and hit[1].device == w.device:
            return hit[1], hit[2]
    bt = w.detach().t() if transposed else w.detach()
    N, K = bt.shape
    if K % 4 or not bt.is_contiguous():
        wide = torch.zeros((N, K + (-K) % 4), dtype=torch.float32, device=w.device)
        wide[:, :K] = bt
        bt = wide
    head, tail = dense_split(bt)
    if cache_key is not None:
        slot[transposed] = (cache_key._version, head, tail)
    return head, tail


def dense_nt(a, b, transposed=False, relu=False, mask=None, cache_key=None):
    """a [M x K] @ op(b) on the tensor cores with fp32 accuracy (dg_dense_nt): b is the small operand, [N x K] as given
    or [K x N] with transposed=True.  Returns None when the shapes or strides are outside what the kernel takes (the
    caller then uses a library GEMM).  relu applies max(x, 0) on the way out; mask [M x N] zeroes the result where
    mask <= 0 (the backward of a ReLU whose output is `mask`); cache_key: see split_operand."""
    lda = _row_major(a, 'a')
    if not (isinstance(b, torch.Tensor) and b.is_cuda and b.dtype == torch.float32 and b.dim() == 2):
        raise RuntimeError('b must be a 2-D fp32 CUDA tensor: this library has no CPU path')
    M, K = a.shape
    N = b.size(1) if transposed else b.size(0)
    if (b.size(0) if transposed else b.size(1)) != K:
        raise RuntimeError(f'inner dimensions differ: {tuple(a.shape)} x {tuple(b.shape)}{"" if transposed else "^T"}')
    ldm = _row_major(mask, 'mask') if mask is not None else 0
    if mask is not None and tuple(mask.shape) != (M, N):
        raise RuntimeError(f'mask is {tuple(mask.shape)}, the product {(M, N)}')
    ldb = K + (-K) % 4
    if M == 0 or N == 0 or not lib().dg_dense_supported(M, N, K, lda, ldb, a.data_ptr(), None, None):
        return None
    head, tail = split_operand(b, transposed, cache_key)
    global dense_launches
    dense_launches += (N + 255) // 256
    c = torch.empty((M, N), dtype=torch.float32, device=a.device)
    with torch.cuda.device(a.device):
        check(lib().dg_dense_nt_masked(a.data_ptr(), lda, head.data_ptr(), tail.data_ptr(), ldb, c.data_ptr(), N, M, N, K, int(relu),
                                       mask.data_ptr() if mask is not None else None, ldm, _stream()))
    return c


_tn_scratch = {}


def dense_tn(x, g):
    """x[n x Km]^T @ g[n x Nn] on the tensor cores with fp32 accuracy (dg_dense_tn), or None when the shapes or strides
    are outside what the kernel takes.  Both operands are streamed once; per-CTA partial results are added in CTA order."""
    ldx, ldg = _row_major(x, 'x'), _row_major(g, 'g')
    n, Km = x.shape
    Nn = g.size(1)
    if g.size(0) != n:
        raise RuntimeError(f'row counts differ: {tuple(x.shape)} vs {tuple(g.shape)}')
    if n == 0 or not lib().dg_dense_tn_supported(n, Km, Nn, ldx, ldg, x.data_ptr(), g.data_ptr()):
        return None
    ctas = torch.cuda.get_device_properties(x.device).multi_processor_count
    scratch = _tn_scratch.get(x.device)
    if scratch is None:
        scratch = _tn_scratch[x.device] = torch.empty(ctas * 256 * 256, dtype=torch.float32, device=x.device)
    global dense_launches
    dense_launches += 2 * ((Km + 255) // 256) * ((Nn + 255) // 256)      # per 256 x 256 panel: the product and the reduction over the CTAs' partials
    d = torch.empty((Km, Nn), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().dg_dense_tn(x.data_ptr(), ldx, g.data_ptr(), ldg, d.data_ptr(), Nn, n, Km, Nn, scratch.data_ptr(), scratch.numel(),
                                ctas, _stream()))
    return d


def dense_status(reset=False):
    """0, or non-zero if a dense-transform kernel gave up on one of its bounded waits since the last reset (its output is
    then invalid).  Synchronises the current stream.  reset=True clears the word after reading it."""
    out = ctypes.c_int(-1)
    check(lib().dg_dense_status(ctypes.byref(out), _stream()))
    if reset and out.value:
        check(lib().dg_dense_status_reset(_stream()))
    return out.value


def check_dense_status():
    """Raises if a dense kernel gave up since the last check (and clears the word, so the next check starts fresh)."""
    status = dense_status(reset=True)
    if status:
        raise RuntimeError('a dense-transform kernel gave up on a bounded wait: the activations or gradients of this step are invalid')


def dense_wait_selftest():
    """Runs the dense kernels' give-up path on purpose (dg_dense_wait_selftest); True if the bounded wait ran out as it must."""
    out = ctypes.c_int(-1)
    check(lib().dg_dense_wait_selftest(ctypes.byref(out), _stream()))
    return out.value == 1
