"""Process-group set-up and collective helpers with the surface of light_dist_gnn/dist_utils/env.py:10-54, plus the
replication groups of the 1.5D variant (1D_CAGNET/utils.py:21-49).

Two layers of communicators live here.  torch.distributed (NCCL or gloo) is the plumbing: rendezvous, object
exchange, the occasional all-gather of outputs for evaluation.  The hot path - the broadcasts of the stage loop,
the dW all-reduce and the 1.5D partial-sum all-reduce - runs on the library's own NCCL communicators
(``spmm_cpp.Comm``) created here when the ranks own CUDA devices.

Differences from the reference, on purpose: one visible GPU selects that GPU (the reference falls back to the CPU
unless it sees more than one, env.py:26-31); the O(P^2) two-rank groups of env.py:51-54, which no model of
light_dist_gnn uses, are not created (``p2p_group_dict`` stays empty); the timer's side channel is the process
group's own store instead of a fixed file under the temp folder, which went stale between runs.
"""
import os

import torch
import torch.distributed as dist

from . import schedule
from .logger import DistLogger
from .timer import DistTimer


class DistEnv:
    env = None

    def __init__(self, rank, world_size, backend='nccl', rep=1, stage_group=None, stage_order=None):
        assert rank >= 0
        assert world_size > 0
        schedule.check_layout(world_size, rep)
        self.rank, self.world_size, self.backend, self.rep = rank, world_size, backend, rep
        self.rank_grp, self.rank_col = rank // rep, rank % rep          # row block, replica index
        self.init_device()
        self.init_dist_groups()
        self.init_comms()
        self.logger = DistLogger(self)
        self.timer = DistTimer(self)
        self.store = dist.PrefixStore('dist_gnn_timer', dist.distributed_c10d._get_default_store())
        self._recv = {}
        # Order of the products inside a distributed SpMM:
        # 'reference':   ascending stage order (the reference's sum order), NCCL broadcasts into two receive buffers;
        # 'local_first': own block first, one receive area for all remote blocks, every broadcast queued up front;
        # 'feature_chunks' (1D): all-gather the operand one column chunk at a time, one full-row product per chunk;
        # 'peer_copy':   own block first, remote blocks pulled from their owners' send buffers by device-to-device copies.
        # 'peer_compact': peer_copy that moves only the operand rows each reader's sparse block touches (1D; less than half
        #                of the rows at 8 ranks on the benchmark graph): the owner packs them per reader, the reader copies.
        # 'peer_gather':  the same rows, gathered by the reader out of the owner's whole block with a small pull kernel; the
        #                owners pack nothing and nothing is exchanged beforehand.
        # Default: peer_compact for 1D (8 GPUs: 15.7 ms per epoch on the benchmark graph against 19.5 for peer_gather; the
        # broadcast loops and peer_copy were 25-30 ms with earlier kernels), reference for 1.5D (peer copies were slower there).
        default_order = 'peer_compact' if rep == 1 else 'reference'
        self.stage_order = stage_order if stage_order is not None else os.environ.get('DIST_GNN_STAGE_ORDER', default_order)
        if self.stage_order not in ('reference', 'local_first', 'feature_chunks', 'peer_copy', 'peer_compact', 'peer_gather'):
            raise ValueError(f'unknown stage order {self.stage_order!r}')
        # Stages fused into one product (1 = stage by stage, as the reference); the defaults and the measurements behind
        # them are in schedule.default_stage_group.
        chosen = stage_group if stage_group is not None else os.environ.get('DIST_GNN_STAGE_GROUP')
        if chosen is not None:
            # an integer, or for 'peer_compact' a list of group sizes such as "4,2,1" (arrivals per product, in pull order)
            sizes = [max(1, int(v)) for v in str(chosen).replace('(', '').replace(')', '').replace('[', '').replace(']', '').split(',') if v.strip()]
            self.stage_group = sizes[0] if len(sizes) == 1 else tuple(sizes)
        else:
            self.stage_group = schedule.default_stage_group(self.stage_order, rep, len(self.stages()))
        self.chunk_width = int(os.environ.get('DIST_GNN_CHUNK_WIDTH', 64))
        DistEnv.env = self

    def __repr__(self):
        return '<DistEnv %d/%d %s>' % (self.rank, self.world_size, self.backend)

    @property
    def group_k(self):
        """stage_group as one number, for the loops that fuse a fixed count of stages (a size list is 'peer_compact' only)."""
        return self.stage_group if isinstance(self.stage_group, int) else self.stage_group[0]

    def init_device(self):
        if torch.cuda.is_available() and self.backend == 'nccl':
            local = int(os.environ.get('LOCAL_RANK', self.rank)) % torch.cuda.device_count()
            self.device = torch.device('cuda', local)
            torch.cuda.set_device(self.device)
        else:
            self.device = torch.device('cpu')

    def init_dist_groups(self):
        if not dist.is_initialized():
            dist.init_process_group(backend=self.backend, rank=self.rank, world_size=self.world_size, init_method='env://')
        self.world_group = dist.new_group(list(range(self.world_size)))
        self.p2p_group_dict = {}
        self.row_procs = schedule.row_groups(self.world_size, self.rep)
        self.col_procs = schedule.col_groups(self.world_size, self.rep)
        self.row_groups, self.col_groups = [self.world_group], [self.world_group]
        if self.rep > 1:    # every rank creates every group, in the same order
            self.row_groups = [dist.new_group(p) for p in self.row_procs]
            self.col_groups = [dist.new_group(p) for p in self.col_procs]

    def init_comms(self):
        """Library communicators for the hot path: world, and for 1.5D the column (broadcast) and row (replica) groups."""
        self.comm = self.col_comm = self.row_comm = None
        if self.device.type != 'cuda' or self.world_size == 1:
            return
        import spmm_cpp
        box = [spmm_cpp.Comm.unique_id() if self.rank == 0 else None]
        dist.broadcast_object_list(box, src=0, group=self.world_group)
        self.comm = spmm_cpp.Comm.create(box[0], self.rank, self.world_size, self.device)
        self.col_comm = self.comm
        if self.rep > 1:
            self.col_comm = self.comm.split(self.rank_col, self.rank)
            self.row_comm = self.comm.split(self.rank_grp, self.rank)

    # ---- collective helpers (env.py:33-45) -------------------------------------------------------------------------
    def all_reduce_sum(self, tensor):
        """dW all-reduce of the layer backward: world group in 1D, column group in 1.5D."""
        if tensor.is_cuda and self.col_comm is not None:
            self.col_comm.all_reduce_sum(tensor)
        elif self.world_size > 1:
            dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=self.col_groups[self.rank_col] if self.rep > 1 else self.world_group)

    def broadcast(self, tensor, src):
        dist.broadcast(tensor, src=src, group=self.world_group)

    def all_gather_then_cat(self, src_t):
        """Row blocks of every rank stacked in block order (one replica per block in 1.5D)."""
        if self.rep == 1:
            group, size = self.world_group, self.world_size
        else:
            group, size = self.col_groups[self.rank_col], self.world_size // self.rep
        recv_list = [torch.zeros_like(src_t) for _ in range(size)]
        dist.all_gather(recv_list, src_t.contiguous(), group=group)
        return torch.cat(recv_list, dim=0)

    def all_gather_object(self, obj):
        out = [None] * self.world_size
        dist.all_gather_object(out, obj, group=self.world_group)
        return out

    def barrier_all(self):
        if self.device.type == 'cuda':
            dist.barrier(self.world_group, device_ids=[self.device.index])
        else:
            dist.barrier(self.world_group)

    # ---- stage-loop support ----------------------------------------------------------------------------------------
    def stages(self):
        return schedule.stages(self.rank, self.world_size, self.rep)

    def recv_buffers(self, n, F, nbuf=2, tag='recv'):
        """nbuf persistent buffers able to hold an n x F block each, reused by every stage loop; `tag` keeps apart the
        sets that are live at the same time (receive areas, pack buffers)."""
        need = n * F
        bufs = self._recv.get((tag, nbuf))
        if bufs is None or bufs[0].numel() < need:
            bufs = [torch.empty(need, dtype=torch.float32, device=self.device) for _ in range(nbuf)]
            self._recv[(tag, nbuf)] = bufs
        return [b[:need].view(n, F) for b in bufs]

    def ensure_peer_buffers(self, floats):
        """Send buffers of the 'peer_copy' stage order, mapped by every rank of the column communicator.  Collective
        over that communicator: every rank asks for the same sizes in the same order (they run the same model), so
        they all grow at the same call."""
        comm = self.col_comm
        if comm.peer_capacity() >= floats:
            return True
        group = self.world_group if self.rep == 1 else self.col_groups[self.rank_col]
        torch.cuda.synchronize(self.device)
        if comm.peer_capacity() > 0:
            comm.peer_close()
            dist.barrier(group, device_ids=[self.device.index])     # nobody frees a buffer a peer still maps
        ok, mine = True, b''
        try:
            mine = comm.peer_alloc(floats)
        except RuntimeError as e:                                   # e.g. CUDA IPC not permitted in this container
            ok, why = False, str(e)
        handles = [None] * comm.size
        dist.all_gather_object(handles, mine if ok else None, group=group)
        if all(h is not None for h in handles):
            try:
                comm.peer_open(handles)
            except RuntimeError as e:
                ok, why = False, str(e)
        else:
            ok, why = False, locals().get('why', 'a peer could not export its send buffers')
        agreed = [None] * comm.size
        dist.all_gather_object(agreed, ok, group=group)
        if not all(agreed):
            # every rank takes the same decision: back to the NCCL broadcast loop, which needs no peer mappings
            if comm.peer_capacity() > 0:
                comm.peer_close()
            if self.rank == 0:
                print(f"[dist-gnn] peer-copy stage order unavailable ({why if not ok else 'on a peer'}); using NCCL broadcasts", flush=True)
            self.stage_order = 'reference'
            self.stage_group = schedule.default_stage_group('reference', self.rep, len(self.stages()))
            return False
        dist.barrier(group, device_ids=[self.device.index])
        return True

    def shutdown(self, keep_process_group=False):
        """Closes the peer mappings and the library communicators; keep_process_group=True leaves torch.distributed
        initialised so that another DistEnv (another partition layout) can follow in the same process."""
        comms = list({id(c): c for c in (self.row_comm, self.col_comm, self.comm) if c is not None}.values())
        if any(c.peer_capacity() > 0 for c in comms):
            torch.cuda.synchronize(self.device)
            for c in comms:
                if c.peer_capacity() > 0:
                    c.peer_close()
            self.barrier_all()                                      # every mapping is gone before any owner frees its buffers
        for c in comms:
            c.destroy()
        self.comm = self.col_comm = self.row_comm = None
        self._recv = {}
        if dist.is_initialized() and not keep_process_group:
            dist.destroy_process_group()
        DistEnv.env = None
