"""Parameter registry, flat buffers, gradient reduction and optimizer state layout.

Counterpart of the reference's ParamStorage + GradConsolidation + the
distributed param / grad locators (src/comp/ParamStorage.cpp:33-191,195-216,
347-596,721-819,827-1232; src/comp/Distributed{Param,Grad}Locator.cpp).

Layout.  Parameters that share an owner rank set live in ONE flat buffer per
dtype (``flat_param``), with a matching flat gradient buffer (``flat_grad``,
fp32 under mixed precision) -- flat by construction, so there is no
pack/unpack copy around a collective, one collective (or one fused kernel)
covers a whole rank set, and gradient accumulation over micro-batches writes
straight into it.  Under mixed precision an fp32 master copy and the optimizer
moments sit in further flat buffers; with ``enable_zero`` each rank keeps only
its contiguous 1/n shard of those (aligned to 16 bytes x ranks, like the
reference's segments) and the optimizer sees the per-parameter intersections
with that shard.

Semantics kept from the reference: a parameter's owner set is the union of the
rank sets of the stages that use it; gradients are summed over the owner set
and averaged over the WORLD size; initial values come from the lowest owner
rank; a parameter shared by two stages on the same rank is an error.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import _core
from ..utils.config import conf
from ..utils.log import get_logger
from . import comm

logger = get_logger("ParamStorage")


def _align(n: int, unit: int) -> int:
    return (n + unit - 1) // unit * unit


class FlatGroup:
    """All parameters of one (owner rank set, dtype)."""

    def __init__(self, ranks: Tuple[int, ...], dtype: torch.dtype, device: torch.device):
        self.ranks = ranks
        self.dtype = dtype
        self.device = device
        self.names: List[str] = []
        self.params: List[torch.nn.Parameter] = []
        self.offsets: List[int] = []
        self.numels: List[int] = []
        self.opt_group: List[int] = []          # optimizer param_group index per param (-1: none)
        self.total = 0                           # aligned flat length
        self.flat_param: Optional[torch.Tensor] = None
        self.flat_grad: Optional[torch.Tensor] = None
        self.flat_master: Optional[torch.Tensor] = None  # fp32, full or shard
        self.master_params: List[Optional[torch.nn.Parameter]] = []
        self.shard: Tuple[int, int] = (0, 0)     # [lo, hi) of the flat buffer this rank updates
        self.symm = None                         # symmetric-memory handles of the fused gradient path
        self.slice_ranks: Optional[Tuple[int, ...]] = None  # tensor-partitioned weights: ranks holding the slices

    @property
    def nranks(self) -> int:
        return len(self.ranks)

    @property
    def my_index(self) -> int:
        return self.ranks.index(comm.get_rank())

    def add(self, name: str, p: torch.nn.Parameter, opt_group: int):
        self.names.append(name)
        self.params.append(p)
        self.opt_group.append(opt_group)

    def finalize(self, amp: bool, zero: bool, symmetric: bool = False):
        # 16-byte aligned slots so every parameter view can feed TMA / vector loads
        es = torch.empty((), dtype=self.dtype).element_size()
        unit = max(1, 16 // es)
        off = 0
        for p in self.params:
            self.offsets.append(off)
            self.numels.append(p.numel())
            off += _align(p.numel(), unit)
        # whole buffer divisible into equal 16-byte aligned shards
        self.total = _align(max(off, 1), unit * self.nranks * 8)
        gdtype = torch.float32 if amp else self.dtype
        self.symmetric = bool(symmetric and (self.nranks > 1 or self.slice_ranks) and self.device.type == "cuda")
        if self.symmetric:
            # peers read / write these buffers directly (fused gradient path)
            from .fused_reduce import symm_empty

            self.flat_param = symm_empty(self.total, self.dtype, self.device).zero_()
            self.flat_grad = symm_empty(self.total, gdtype, self.device).zero_()
        else:
            self.flat_param = torch.zeros(self.total, dtype=self.dtype, device=self.device)
            self.flat_grad = torch.zeros(self.total, dtype=gdtype, device=self.device)
        seg = self.total // self.nranks
        self.shard = (seg * self.my_index, seg * (self.my_index + 1)) if zero else (0, self.total)
        for p, o, n in zip(self.params, self.offsets, self.numels):
            view = self.flat_param[o:o + n].view(p.shape)
            view.copy_(p.data.to(device=self.device, dtype=self.dtype))
            p.data = view
            gview = self.flat_grad[o:o + n].view(p.shape)
            if amp:
                p.main_grad = gview
                p.grad = None
            elif p.requires_grad:
                p.grad = gview

    def param_range(self, i: int) -> Tuple[int, int]:
        return self.offsets[i], self.offsets[i] + self.numels[i]

    def local_range(self, i: int) -> Tuple[int, int]:
        """Intersection of parameter i with this rank's shard, in flat coordinates (may be empty)."""
        lo, hi = self.param_range(i)
        return max(lo, self.shard[0]), max(max(lo, self.shard[0]), min(hi, self.shard[1]))


class ParamStorage:
    def __init__(self, amp: bool, zero: bool, allreduce_amp_master_params: bool = False):
        self.amp = amp
        self.zero = zero
        self.allreduce_amp_master_params = allreduce_amp_master_params
        self.groups: List[FlatGroup] = []
        self.by_name: Dict[str, Tuple[FlatGroup, int]] = {}
        self.buffers: Dict[str, torch.Tensor] = {}
        self.param_ranks: Dict[str, Tuple[int, ...]] = {}
        self.sliced: Dict[str, Tuple[int, ...]] = {}   # weight sliced along dim 1 over these ranks
        self.global_order: Dict[str, int] = {}
        self.sync_on_init = True
        self.offload = False     # fp32 master copies and optimizer state in pinned host memory
        self._sumsq = None
        self._ctrl = None
        self._norm = None

    # ---------------------------------------------------------------- deploy
    def deploy(self, named_params: Dict[str, torch.nn.Parameter], owner_ranks: Dict[str, Sequence[int]],
               opt_group_of: Dict[int, int], device: torch.device, global_order: Dict[str, int],
               symmetric: bool = False, sliced: Optional[Dict[str, Sequence[int]]] = None,
               symmetric_slices: bool = False):
        """``sliced``: fqn -> ranks for weights stored as column slices (tensor-partitioned linear layers);
        such a parameter's local slice belongs to a flat buffer only this rank reduces and updates.
        ``named_params``: parameters used on this rank (fqn -> Parameter, tied names deduplicated);
        ``owner_ranks``: fqn -> ranks of every stage using it (for ALL parameters of the model, so that every
        rank can create the same communicators in the same order)."""
        me = comm.get_rank()
        self.global_order = dict(global_order)
        self.param_ranks = {k: tuple(sorted(set(v))) for k, v in owner_ranks.items()}
        self.sliced = {k: tuple(sorted(set(v))) for k, v in (sliced or {}).items()}
        comm.create_groups(list(self.param_ranks.values()) + list(self.sliced.values()))
        keyed: Dict[tuple, FlatGroup] = {}
        order = sorted(named_params.items(),
                       key=lambda kv: (opt_group_of.get(id(kv[1]), 1 << 30), global_order.get(kv[0], 0)))
        for name, p in order:
            ranks = self.param_ranks[name]
            if me not in ranks:
                continue
            dtype = p.dtype
            sl = self.sliced.get(name)
            key = ((me,), dtype, sl) if sl else (ranks, dtype, ())
            if key not in keyed:
                keyed[key] = FlatGroup(key[0], dtype, device)
                keyed[key].slice_ranks = sl
            keyed[key].add(name, p, opt_group_of.get(id(p), -1))
        # deterministic group order on every rank: smaller rank sets first
        self.groups = [keyed[k] for k in sorted(keyed, key=lambda k: (len(k[0]), k[0], str(k[1]), k[2]))]
        for g in self.groups:
            g.finalize(self.amp and g.dtype in (torch.float16, torch.bfloat16), self.zero,
                       symmetric_slices if g.slice_ranks else symmetric)
            for i, n in enumerate(g.names):
                self.by_name[n] = (g, i)
        if self.sync_on_init:
            self.sync_params_from_root()

    def sync_params_from_root(self):
        """Every owner starts from the lowest owner rank's values (reference: ParamStorage.cpp:1024-1057)."""
        for g in self.groups:
            if g.nranks > 1:
                comm.bcast(g.flat_param, g.ranks[0], g.ranks)

    def setup_master(self):
        """fp32 master copies (whole buffer, or this rank's shard under ZeRO)."""
        for g in self.groups:
            if g.dtype not in (torch.float16, torch.bfloat16) or not self.amp:
                g.master_params = [None] * len(g.params)
                continue
            lo, hi = g.shard
            g.flat_master = g.flat_param[lo:hi].float()
            host = self.offload and g.flat_master.is_cuda
            if host:
                g.flat_master = g.flat_master.cpu().pin_memory()
            g.master_params = []
            for i, p in enumerate(g.params):
                a, b = g.local_range(i)
                if b <= a:
                    g.master_params.append(None)
                    continue
                full = (a, b) == g.param_range(i)
                mview = g.flat_master[a - lo:b - lo]
                mp = torch.nn.Parameter(mview.view(p.shape) if full else mview, requires_grad=p.requires_grad)
                if not host:
                    mp.grad = g.flat_grad[a:b].view(mp.shape)
                g.master_params.append(mp)

    # ---------------------------------------------------------------- gradients
    def zero_grad(self):
        for g in self.groups:
            g.flat_grad.zero_()
            for p in g.params:
                if not self.amp or g.flat_master is None:
                    if p.requires_grad and p.grad is None:
                        lo, hi = g.param_range(g.params.index(p))
                        p.grad = g.flat_grad[lo:hi].view(p.shape)

    def fold_model_grads(self):
        """Mixed precision: gradients autograd left in ``p.grad`` (operators without a fused wgrad) are added
        into the fp32 buffer."""
        from ..ops import kernels as K

        for g in self.groups:
            if g.flat_master is None and not (self.amp and g.dtype in (torch.float16, torch.bfloat16)):
                continue
            for p in g.params:
                if p.grad is not None and p.grad.data_ptr() != p.main_grad.data_ptr():
                    if p.grad.is_cuda and p.grad.dtype in (torch.float16, torch.bfloat16):
                        K.accum_f32(p.main_grad, p.grad.contiguous())
                    else:
                        p.main_grad.add_(p.grad.float())
                    p.grad = None

    def allreduce_grads(self):
        """Baseline gradient path: NCCL all-reduce of each flat buffer, averaged over the world size
        (reference: one ncclAllReduce per parameter with PreMulSum(1/world), ParamStorage.cpp:347-394)."""
        world = comm.get_world_size()
        self.fold_model_grads()
        for g in self.groups:
            if world > 1:
                g.flat_grad.mul_(1.0 / world)
            if g.nranks > 1:
                comm.allreduce(g.flat_grad, "sum", g.ranks)
        self._sync_if_asked()

    def allreduce_grads_zero(self, only=None):
        """ZeRO baseline: reduce-scatter so each rank holds the reduced gradient of its shard
        (reference: bucketed ncclReduceScatter, ParamStorage.cpp:396-520).  ``only``: a subset of the groups."""
        world = comm.get_world_size()
        self.fold_model_grads()
        for g in self.groups:
            if only is not None and g not in only:
                continue
            if world > 1:
                g.flat_grad.mul_(1.0 / world)
            if g.nranks > 1:
                lo, hi = g.shard
                out = torch.empty(hi - lo, dtype=g.flat_grad.dtype, device=g.device)
                comm.reduce_scatter_into(out, g.flat_grad, g.ranks)
                g.flat_grad[lo:hi].copy_(out)
        self._sync_if_asked()

    @staticmethod
    def _sync_if_asked():
        """``sync_allreduce``: the host waits for the reduction before it launches anything else (debugging aid;
        reference: ParamStorage.cpp, syncStream after the all-reduce)."""
        if bool(conf("sync_allreduce")) and comm.is_cuda():
            torch.cuda.synchronize()

    def allgather_params_zero(self, only=None):
        """Refreshes the full 16-bit parameters from the updated shards (reference: ParamStorage.cpp:559-596)."""
        for g in self.groups:
            if only is not None and g not in only:
                continue
            if g.nranks > 1 and self.zero:
                lo, hi = g.shard
                comm.allgather_into(g.flat_param, g.flat_param[lo:hi].clone(), g.ranks)

    # ---------------------------------------------------------------- norms
    def _norm_bufs(self, device):
        if self._sumsq is None or self._sumsq.device != device:
            self._sumsq = torch.zeros(1, dtype=torch.float32, device=device)
            self._ctrl = torch.zeros(2, dtype=torch.float32, device=device)
            self._norm = torch.zeros(1, dtype=torch.float32, device=device)
        return self._sumsq, self._ctrl, self._norm

    def grad_sumsq(self) -> torch.Tensor:
        """Sum of squares of the gradients this rank is responsible for, as a device scalar.  Each element is
        counted once across the job: a rank counts its shard under ZeRO, otherwise the lowest owner counts."""
        me = comm.get_rank()
        dev = self.groups[0].device if self.groups else comm.device()
        ss, _, _ = self._norm_bufs(dev)
        ss.zero_()
        for g in self.groups:
            if self.zero:
                lo, hi = g.shard
            elif g.ranks[0] == me:
                lo, hi = 0, g.total
            else:
                continue
            seg = g.flat_grad[lo:hi]
            if seg.is_cuda:
                from ..ops import kernels as K

                K.sumsq(seg, ss)
            else:
                ss.add_(seg.float().pow(2).sum())
        if comm.get_world_size() > 1:
            comm.allreduce(ss, "sum")
        return ss

    def calc_grad_norm(self) -> float:
        return float(self.grad_sumsq().sqrt().item())

    def clip_grad_norm(self, max_norm: float) -> float:
        ss = self.grad_sumsq()
        norm = float(ss.sqrt().item())
        coef = max_norm / (norm + 1e-6)
        if coef < 1.0:
            for g in self.groups:
                g.flat_grad.mul_(coef)
        return norm

    # ---------------------------------------------------------------- access for checkpoints / tests
    def load_param(self, name: str, value: torch.Tensor) -> bool:
        """Overwrites a deployed parameter with ``value`` (the full tensor): the 16-bit / working copy in the flat
        buffer and, under mixed precision, the part of the fp32 master copy this rank keeps.  Every rank that
        holds the parameter must call it with the same value.  Returns False if this rank does not hold it."""
        if name not in self.by_name:
            return False
        g, i = self.by_name[name]
        v = value.detach()
        sl = self.sliced.get(name)
        if sl:
            # tensor-partitioned weight: this rank keeps one block of columns
            ks = v.shape[1] // len(sl)
            idx = sl.index(comm.get_rank())
            v = v[:, idx * ks:(idx + 1) * ks]
        flat = v.contiguous().reshape(-1)
        o, e = g.param_range(i)
        if flat.numel() != e - o:
            raise RuntimeError(f"{name}: got {flat.numel()} elements for a parameter of {e - o}")
        g.flat_param[o:e].copy_(flat.to(device=g.device, dtype=g.dtype))
        if g.flat_master is not None:
            a, b = g.local_range(i)
            if b > a:
                lo = g.shard[0]
                g.flat_master[a - lo:b - lo].copy_(flat[a - o:b - o].to(torch.float32))
        return True

    def _root_of(self, name: str) -> int:
        return self.param_ranks[name][0]

    def get_param(self, name: str, shape, dtype, amp_master: bool = False) -> torch.Tensor:
        """Collective over the world: the value from the lowest owner rank, on the CPU
        (reference: ParamStorage::syncParam / gatherParamZero, ParamStorage.cpp:1079-1232)."""
        return self._fetch(name, shape, dtype, grad=False, amp_master=amp_master)

    def get_param_grad(self, name: str, shape, dtype, amp_master: bool = False) -> torch.Tensor:
        return self._fetch(name, shape, dtype, grad=True, amp_master=amp_master)

    def _fetch(self, name, shape, dtype, grad: bool, amp_master: bool) -> torch.Tensor:
        root = self._root_of(name)
        me = comm.get_rank()
        dev = comm.device()
        use_master = amp_master and self.amp
        out_dtype = torch.float32 if (use_master or (grad and self.amp and dtype in (torch.float16, torch.bfloat16))) \
            else dtype
        numel = 1
        for d in shape:
            numel *= d
        sl = self.sliced.get(name)
        if name in self.by_name:
            g, i = self.by_name[name]
            lo, hi = g.param_range(i)
            if grad:
                if self.zero and g.nranks > 1:
                    full = self._gather_sharded(g, g.flat_grad, lo, hi)
                else:
                    full = g.flat_grad[lo:hi]
            elif use_master and g.flat_master is not None:
                if self.zero and g.nranks > 1:
                    full = self._gather_sharded(g, None, lo, hi, master=True)
                else:
                    full = g.flat_master[lo - g.shard[0]:hi - g.shard[0]]
            else:
                full = g.flat_param[lo:hi]
            if sl:
                # this rank's column block of the full weight; the blocks are summed below
                ks = shape[1] // len(sl)
                idx = sl.index(me)
                val = torch.zeros(shape, dtype=out_dtype, device=full.device)
                val[:, idx * ks:(idx + 1) * ks] = full.to(out_dtype).reshape(shape[0], ks)
            else:
                val = full.to(out_dtype).reshape(shape).clone()
        elif sl:
            val = torch.zeros(shape, dtype=out_dtype, device=dev)
        else:
            val = torch.empty(shape, dtype=out_dtype, device=dev)
        if sl:
            if comm.get_world_size() > 1:
                val = val.to(dev)
                comm.allreduce(val, "sum")
            return val.cpu()
        if comm.get_world_size() > 1:
            if val.device != dev:
                val = val.to(dev)
            comm.bcast(val, root)
        return val.cpu()

    def _gather_sharded(self, g: FlatGroup, flat: Optional[torch.Tensor], lo: int, hi: int, master: bool = False):
        """All-gather of the shards of a ZeRO-sharded buffer inside the owner set, then the [lo, hi) slice."""
        seg = g.total // g.nranks
        slo, shi = g.shard
        mine = (g.flat_master if master else flat[slo:shi]).float().contiguous()
        full = torch.empty(g.total, dtype=torch.float32, device=g.device)
        comm.allgather_into(full, mine, g.ranks)
        return full[lo:hi]
