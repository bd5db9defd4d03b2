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
one 1/n slice of every gradient bucket of those (aligned to 16 bytes x ranks,
like the reference's segments) and the optimizer sees the per-parameter
intersections with its slices.

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


def _host_zeros(n: int, dtype: torch.dtype) -> torch.Tensor:
    """Host buffer the device can copy from / to asynchronously (pinned when there is a CUDA device)."""
    t = torch.zeros(n, dtype=dtype)
    return t.pin_memory() if torch.cuda.is_available() else t


def _align(n: int, unit: int) -> int:
    return (n + unit - 1) // unit * unit


class FlatGroup:
    """All parameters of one (owner rank set, dtype).

    The flat buffer is a sequence of *buckets*: runs of whole parameters, each padded so that it splits into
    equal 16-byte aligned slices, one per rank.  Without ZeRO there is one bucket and every rank updates all of
    it.  With ZeRO rank r updates slice r of EVERY bucket (``pieces``), so that each bucket can be reduced as
    soon as backward has produced its gradients, with every rank taking an equal part of the work; the fp32
    master copy and the optimizer moments of a rank are the concatenation of its slices (``local_len``
    elements, ``to_local`` maps flat coordinates into it).  Because buckets end at parameter boundaries a
    parameter meets this rank's slices in at most one contiguous piece (``local_range``).
    (Reference: 128 MiB reduce-scatter buckets, src/comp/ParamStorage.cpp:21,396-520; per-parameter aligned
    segments, src/comp/DistributedGradLocator.cpp:10-86.)"""

    def __init__(self, ranks: Tuple[int, ...], dtype: torch.dtype, device: torch.device):
        self.ranks = ranks
        self.dtype = dtype
        self.device = device
        self.names: List[str] = []
        self.params: List[torch.nn.Parameter] = []
        self.offsets: List[int] = []
        self.numels: List[int] = []
        self.opt_group: List[int] = []          # optimizer param_group index per param (-1: none)
        self.units: List[Optional[str]] = []    # parameters with the same key stay adjacent in one bucket
        self.total = 0                           # aligned flat length
        self.flat_param: Optional[torch.Tensor] = None
        self.flat_grad: Optional[torch.Tensor] = None
        self.flat_master: Optional[torch.Tensor] = None  # fp32, full or this rank's slices
        self.master_params: List[Optional[torch.nn.Parameter]] = []
        self.buckets: List[Tuple[int, int]] = []          # [lo, hi) in flat coordinates
        self.bucket_of: List[int] = []                    # bucket index per parameter
        self.pieces: List[Tuple[int, int, int]] = []      # (flat lo, flat hi, local offset) this rank updates
        self.local_len = 0
        self.zero = False
        self.symm = None                         # symmetric-memory handles of the fused gradient path
        self.slice_ranks: Optional[Tuple[int, ...]] = None  # tensor-partitioned weights: ranks holding the slices
        # streamed: the 16-bit parameters and their fp32 gradients live in (pinned) host memory and only the
        # operators about to run have theirs on the device (parallel/param_stream.py)
        self.streamed = False

    @property
    def nranks(self) -> int:
        return len(self.ranks)

    @property
    def my_index(self) -> int:
        return self.ranks.index(comm.get_rank())

    @property
    def shard(self) -> Tuple[int, int]:
        """[lo, hi) this rank updates when that is ONE interval (no ZeRO, or a single bucket)."""
        if len(self.pieces) != 1:
            raise RuntimeError("this rank's part of the flat buffer is not one interval; use pieces / to_local")
        return self.pieces[0][0], self.pieces[0][1]

    def add(self, name: str, p: torch.nn.Parameter, opt_group: int, unit: Optional[str] = None):
        self.names.append(name)
        self.params.append(p)
        self.opt_group.append(opt_group)
        self.units.append(unit)

    def finalize(self, amp: bool, zero: bool, symmetric: bool = False, bucket_numel: int = 0,
                 streamed: bool = False):
        # 16-byte aligned slots so every parameter view can feed TMA / vector loads
        es = torch.empty((), dtype=self.dtype).element_size()
        unit = max(1, 16 // es)
        balign = unit * self.nranks * 8          # a bucket divides into equal 16-byte aligned slices
        self.zero = bool(zero)
        off, bstart = 0, 0
        n = len(self.params)
        for i, p in enumerate(self.params):
            self.offsets.append(off)
            self.numels.append(p.numel())
            self.bucket_of.append(len(self.buckets))
            off += _align(p.numel(), unit)
            same_unit = i + 1 < n and self.units[i] is not None and self.units[i + 1] == self.units[i]
            if zero and bucket_numel > 0 and off - bstart >= bucket_numel and not same_unit and i + 1 < n:
                off = bstart + _align(off - bstart, balign)
                self.buckets.append((bstart, off))
                bstart = off
        off = bstart + _align(max(off - bstart, 1), balign)
        self.buckets.append((bstart, off))
        self.total = off
        gdtype = torch.float32 if amp else self.dtype
        self.streamed = bool(streamed and amp and not self.slice_ranks)
        self.symmetric = bool(symmetric and (self.nranks > 1 or self.slice_ranks) and self.device.type == "cuda"
                              and not self.streamed)
        if self.streamed:
            self.flat_param = _host_zeros(self.total, self.dtype)
            self.flat_grad = _host_zeros(self.total, gdtype)
        elif self.symmetric:
            # peers read / write these buffers directly (fused gradient path)
            from .fused_reduce import symm_empty

            self.flat_param = symm_empty(self.total, self.dtype, self.device).zero_()
            self.flat_grad = symm_empty(self.total, gdtype, self.device).zero_()
        else:
            self.flat_param = torch.zeros(self.total, dtype=self.dtype, device=self.device)
            self.flat_grad = torch.zeros(self.total, dtype=gdtype, device=self.device)
        if zero:
            loc = 0
            for lo, hi in self.buckets:
                seg = (hi - lo) // self.nranks
                a = lo + seg * self.my_index
                self.pieces.append((a, a + seg, loc))
                loc += seg
            self.local_len = loc
        else:
            self.pieces = [(0, self.total, 0)]
            self.local_len = self.total
        for p, o, n_ in zip(self.params, self.offsets, self.numels):
            view = self.flat_param[o:o + n_].view(p.shape)
            if self.streamed:
                view.copy_(p.data.to(dtype=self.dtype))
                # the Parameter keeps its identity (the optimizer and the stage graphs refer to it); between
                # uses it holds no device memory.  ``fetch`` / ``release`` of the streamer swap the data in and out.
                p._rannc_host = view
                p._rannc_host_grad = self.flat_grad[o:o + n_].view(p.shape)
                p._rannc_shape = tuple(p.shape)
                p._rannc_flat = (self, o, n_)     # where it lives in the host buffers
                p._rannc_grad_valid = False
                p.data = torch.empty(0, dtype=self.dtype, device=self.device)
                p.main_grad = None
                p.grad = None
                continue
            view.copy_(p.data.to(device=self.device, dtype=self.dtype))
            p.data = view
            gview = self.flat_grad[o:o + n_].view(p.shape)
            if amp:
                p.main_grad = gview
                p.grad = None
            elif p.requires_grad:
                p.grad = gview

    def param_range(self, i: int) -> Tuple[int, int]:
        return self.offsets[i], self.offsets[i] + self.numels[i]

    def local_range(self, i: int) -> Tuple[int, int]:
        """Intersection of parameter i with the part this rank updates, in flat coordinates (may be empty)."""
        lo, hi = self.param_range(i)
        if not self.zero:
            return lo, hi
        a, b, _ = self.pieces[self.bucket_of[i]]
        return max(lo, a), max(max(lo, a), min(hi, b))

    def to_local(self, x: int) -> int:
        """Index into this rank's master / moment buffers of flat coordinate ``x`` (inside, or at the end of,
        one of its pieces)."""
        for a, b, loc in self.pieces:
            if a <= x <= b:
                return loc + (x - a)
        raise IndexError(f"flat offset {x} is not in this rank's part of the buffer")

    def gather_local(self, flat: torch.Tensor) -> torch.Tensor:
        """This rank's pieces of a flat buffer, concatenated (the layout of the master / moment buffers)."""
        if len(self.pieces) == 1:
            a, b, _ = self.pieces[0]
            return flat[a:b]
        return torch.cat([flat[a:b] for a, b, _ in self.pieces])

    def scatter_local(self, flat: torch.Tensor, local: torch.Tensor) -> None:
        """Inverse of ``gather_local``: writes a local buffer into this rank's pieces of ``flat``."""
        for a, b, loc in self.pieces:
            flat[a:b].copy_(local[loc:loc + (b - a)])


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
        self.stream16 = False    # ... and the 16-bit parameters + fp32 gradients too (offload_param_window_mb > 0)
        self.streamer = None     # parallel/param_stream.ParamStreamer when stream16
        self._sumsq = None
        self._ctrl = None
        self._norm = None

    # ---------------------------------------------------------------- deploy
    def deploy(self, named_params: Dict[str, torch.nn.Parameter], owner_ranks: Dict[str, Sequence[int]],
               opt_group_of: Dict[int, int], device: torch.device, global_order: Dict[str, int],
               symmetric: bool = False, sliced: Optional[Dict[str, Sequence[int]]] = None,
               symmetric_slices: bool = False, adjacent: Optional[Sequence[Sequence[str]]] = None):
        """``sliced``: fqn -> ranks for weights stored as column slices (tensor-partitioned linear layers);
        such a parameter's local slice belongs to a flat buffer only this rank reduces and updates.
        ``named_params``: parameters used on this rank (fqn -> Parameter, tied names deduplicated);
        ``owner_ranks``: fqn -> ranks of every stage using it (for ALL parameters of the model, so that every
        rank can create the same communicators in the same order).
        ``adjacent``: lists of fqns to lay out back to back, in the given order (the three projection weights of
        a fused QKV block, so that one GEMM serves them); honoured when the parameters share a group."""
        me = comm.get_rank()
        self.global_order = dict(global_order)
        self.param_ranks = {k: tuple(sorted(set(v))) for k, v in owner_ranks.items()}
        self.sliced = {k: tuple(sorted(set(v))) for k, v in (sliced or {}).items()}
        comm.create_groups(list(self.param_ranks.values()) + list(self.sliced.values()))
        keyed: Dict[tuple, FlatGroup] = {}
        unit_of: Dict[str, Tuple[str, int, int]] = {}     # fqn -> (unit key, order of the unit's first member, pos)
        for names in (adjacent or ()):
            names = [n for n in names if n in named_params]
            ogs = {opt_group_of.get(id(named_params[n]), 1 << 30) for n in names}
            dts = {named_params[n].dtype for n in names}
            if len(names) < 2 or len(ogs) != 1 or len(dts) != 1 or any(n in unit_of for n in names):
                continue
            first = min(global_order.get(n, 0) for n in names)
            for pos, n in enumerate(names):
                unit_of[n] = ("u:" + names[0], first, pos)

        def sort_key(kv):
            name, p = kv
            u = unit_of.get(name)
            og = opt_group_of.get(id(p), 1 << 30)
            if u is not None:
                return (og, u[1], 0, u[2])
            return (og, global_order.get(name, 0), 1, 0)

        order = sorted(named_params.items(), key=sort_key)
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
            keyed[key].add(name, p, opt_group_of.get(id(p), -1), unit_of[name][0] if name in unit_of else None)
        # deterministic group order on every rank: smaller rank sets first
        self.groups = [keyed[k] for k in sorted(keyed, key=lambda k: (len(k[0]), k[0], str(k[1]), k[2]))]
        bucket_bytes = float(conf("grad_bucket_mb")) * (1 << 20)
        for g in self.groups:
            g_amp = self.amp and g.dtype in (torch.float16, torch.bfloat16)
            ges = 4 if g_amp else torch.empty((), dtype=g.dtype).element_size()
            g.finalize(g_amp, self.zero and not g.slice_ranks,
                       symmetric_slices if g.slice_ranks else symmetric,
                       bucket_numel=int(bucket_bytes // ges) if g.nranks > 1 else 0,
                       streamed=self.stream16)
            for i, n in enumerate(g.names):
                self.by_name[n] = (g, i)
        if self.sync_on_init:
            self.sync_params_from_root()

    def sync_params_from_root(self):
        """Every owner starts from the lowest owner rank's values (reference: ParamStorage.cpp:1024-1057)."""
        for g in self.groups:
            if g.nranks > 1 and g.streamed:
                for lo, hi in self._chunks(0, g.total):
                    d = g.flat_param[lo:hi].to(g.device)
                    comm.bcast(d, g.ranks[0], g.ranks)
                    g.flat_param[lo:hi].copy_(d)
            elif g.nranks > 1:
                comm.bcast(g.flat_param, g.ranks[0], g.ranks)

    @staticmethod
    def _chunks(lo: int, hi: int):
        """[lo, hi) in pieces of at most ``offload_chunk_numel`` elements (device staging of host buffers)."""
        step = max(1 << 16, int(conf("offload_chunk_numel")))
        for a in range(lo, hi, step):
            yield a, min(hi, a + step)

    def wait_streamed(self, host: bool = False) -> None:
        """Copies of streamed gradients / parameters still in flight are ordered before what the current stream
        does next (``host``: before what the host does next)."""
        if self.streamer is not None:
            self.streamer.wait(host)

    def setup_master(self):
        """fp32 master copies (whole buffer, or this rank's slices of every bucket under ZeRO)."""
        for g in self.groups:
            if g.dtype not in (torch.float16, torch.bfloat16) or not self.amp:
                g.master_params = [None] * len(g.params)
                continue
            g.flat_master = g.gather_local(g.flat_param).float()
            host = self.offload and g.flat_master.is_cuda
            if host:
                g.flat_master = g.flat_master.cpu().pin_memory()
            elif g.streamed and torch.cuda.is_available():
                g.flat_master = g.flat_master.pin_memory()
            g.master_params = []
            for i, p in enumerate(g.params):
                a, b = g.local_range(i)
                if b <= a:
                    g.master_params.append(None)
                    continue
                full = (a, b) == g.param_range(i)
                la = g.to_local(a)
                mview = g.flat_master[la:la + (b - a)]
                mp = torch.nn.Parameter(mview.view(getattr(p, "_rannc_shape", p.shape)) if full else mview, requires_grad=p.requires_grad)
                if not host:
                    mp.grad = g.flat_grad[a:b].view(mp.shape)
                g.master_params.append(mp)

    # ---------------------------------------------------------------- gradients
    def zero_grad(self):
        for g in self.groups:
            if g.streamed:
                # nothing is cleared on the host: the first gradient written for a parameter in the next
                # backward overwrites, later ones (further micro-batches) accumulate
                for p in g.params:
                    p._rannc_grad_valid = False
                continue
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
            if g.streamed:
                continue    # folded segment by segment, while the gradient window is on the device
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
            # the divisor is the world size whatever the size of the owner set: every rank saw its share of
            # the global batch.  The scaling rides inside the collective where NCCL's PreMulSum is available.
            if g.streamed:
                self._reduce_streamed(g, 1.0 / world)
                continue
            comm.allreduce(g.flat_grad, "sum", g.ranks, scale=1.0 / world)
        self._sync_if_asked()

    def _reduce_streamed(self, g: FlatGroup, scale: float) -> None:
        """Host-resident gradients: chunk by chunk onto the device, all-reduce there, and back.  Under ZeRO only
        the slices this rank updates are written back (the rest of the host buffer is not read again)."""
        self.wait_streamed()
        if g.nranks == 1 and scale == 1.0:
            return
        spans = g.buckets if g.zero else [(0, g.total)]
        for bi, (blo, bhi) in enumerate(spans):
            for lo, hi in self._chunks(blo, bhi):
                d = g.flat_grad[lo:hi].to(g.device, non_blocking=True)
                comm.allreduce(d, "sum", g.ranks, scale=scale)
                if g.zero:
                    a, b, _ = g.pieces[bi]
                    a, b = max(a, lo), min(b, hi)
                    if b > a:
                        g.flat_grad[a:b].copy_(d[a - lo:b - lo], non_blocking=True)
                else:
                    g.flat_grad[lo:hi].copy_(d, non_blocking=True)
        if g.device.type == "cuda":
            torch.cuda.current_stream().synchronize()   # the optimizer (host or device) reads the host buffer next

    def allreduce_grads_zero(self, only=None):
        """ZeRO baseline: reduce-scatter, bucket by bucket, so each rank holds the reduced gradient of its slices
        (reference: bucketed ncclReduceScatter, ParamStorage.cpp:396-520).  ``only``: a subset of the groups."""
        world = comm.get_world_size()
        self.fold_model_grads()
        for g in self.groups:
            if only is not None and g not in only:
                continue
            scale = 1.0 / world
            if g.streamed:
                self._reduce_streamed(g, scale)
            elif g.nranks > 1 and g.zero:
                for (lo, hi), (a, b, _) in zip(g.buckets, g.pieces):
                    out = torch.empty(b - a, dtype=g.flat_grad.dtype, device=g.device)
                    comm.reduce_scatter_into(out, g.flat_grad[lo:hi], g.ranks, scale=scale)
                    g.flat_grad[a:b].copy_(out)
            else:
                comm.allreduce(g.flat_grad, "sum", g.ranks, scale=scale)
        self._sync_if_asked()

    @staticmethod
    def _sync_if_asked():
        """``sync_allreduce``: the host waits for the reduction before it launches anything else (debugging aid;
        reference: ParamStorage.cpp, syncStream after the all-reduce)."""
        if bool(conf("sync_allreduce")) and comm.is_cuda():
            comm.sync_with_error_check()

    def allgather_params_zero(self, only=None):
        """Refreshes the full 16-bit parameters from the updated slices (reference: ParamStorage.cpp:559-596)."""
        for g in self.groups:
            if only is not None and g not in only:
                continue
            if g.nranks > 1 and g.zero and g.streamed:
                # host-resident parameters: each bucket is assembled on the device and copied back whole
                for (lo, hi), (a, b, _) in zip(g.buckets, g.pieces):
                    out = torch.empty(hi - lo, dtype=g.dtype, device=g.device)
                    comm.allgather_into(out, g.flat_param[a:b].to(g.device, non_blocking=True), g.ranks)
                    g.flat_param[lo:hi].copy_(out, non_blocking=True)
                if g.device.type == "cuda":
                    torch.cuda.current_stream().synchronize()
            elif g.nranks > 1 and g.zero:
                for (lo, hi), (a, b, _) in zip(g.buckets, g.pieces):
                    comm.allgather_into(g.flat_param[lo:hi], g.flat_param[a:b].clone(), g.ranks)

    # ---------------------------------------------------------------- norms
    def _norm_bufs(self, device):
        if self._sumsq is None or self._sumsq.device != device:
            self._sumsq = torch.zeros(1, dtype=torch.float32, device=device)
            self._ctrl = torch.zeros(2, dtype=torch.float32, device=device)
            self._norm = torch.zeros(1, dtype=torch.float32, device=device)
        return self._sumsq, self._ctrl, self._norm

    def _ensure_reduced(self, sticky: bool = True) -> None:
        """The fused gradient path reduces inside (or right before) the optimizer step; anything that reads
        gradients earlier first makes sure the reduction has happened.  ``sticky``: the request comes from user
        code (``clip_grad_norm``, ``get_param_grad``), which will ask again in later steps."""
        red = getattr(self, "reducer", None)
        if red is not None:
            red.ensure_reduced(sticky)

    def grad_sumsq(self, sticky: bool = False) -> torch.Tensor:
        """Sum of squares of the gradients this rank is responsible for, as a device scalar.  Each element is
        counted once across the job: a rank counts its slices under ZeRO, otherwise the lowest owner counts."""
        self._ensure_reduced(sticky)
        self.wait_streamed(host=True)
        me = comm.get_rank()
        dev = self.groups[0].device if self.groups else comm.device()
        ss, _, _ = self._norm_bufs(dev)
        ss.zero_()
        red = getattr(self, "reducer", None)
        for g in self.groups:
            if red is not None and red.adds_sumsq(g, ss):
                continue   # the reduction kernels already summed the squares of this group's reduced gradients
            if g.zero:
                segs = [g.flat_grad[a:b] for a, b, _ in g.pieces]
            elif g.ranks[0] == me:
                segs = [g.flat_grad]
            else:
                continue
            for seg in segs:
                if seg.is_cuda:
                    from ..ops import kernels as K

                    K.sumsq(seg, ss)
                else:
                    ss.add_(seg.float().pow(2).sum())
        if comm.get_world_size() > 1:
            comm.allreduce(ss, "sum")
        return ss

    def calc_grad_norm(self) -> float:
        return float(self.grad_sumsq(sticky=True).sqrt().item())

    def clip_grad_norm(self, max_norm: float) -> float:
        """Global L2 norm of the reduced gradients, then scale them (reference: ParamStorage.cpp:721-819)."""
        ss = self.grad_sumsq(sticky=True)
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
                la = g.to_local(a)
                g.flat_master[la:la + (b - a)].copy_(flat[a - o:b - o].to(torch.float32))
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
                self._ensure_reduced()
                if g.zero and g.nranks > 1:
                    full = self._gather_sharded(g, i, g.flat_grad)
                else:
                    full = g.flat_grad[lo:hi]
            elif use_master and g.flat_master is not None:
                if g.zero and g.nranks > 1:
                    full = self._gather_sharded(g, i, None)
                else:
                    full = g.flat_master[lo:hi]
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

    def _gather_sharded(self, g: FlatGroup, i: int, flat: Optional[torch.Tensor]) -> torch.Tensor:
        """Parameter i of a ZeRO-sharded group, assembled inside the owner set: every rank contributes the part
        of the parameter that lies in its slice of the parameter's bucket (``flat`` = a full-length buffer such
        as the gradients; None = the fp32 master slices).  Only the parameter's own range travels: an
        all-reduce of a zero-filled [numel] buffer (reference: gatherParamZero, ParamStorage.cpp:1143-1232)."""
        lo, hi = g.param_range(i)
        a, b = g.local_range(i)
        out = torch.zeros(hi - lo, dtype=torch.float32, device=g.device)
        if b > a:
            if flat is None:
                la = g.to_local(a)
                out[a - lo:b - lo] = g.flat_master[la:la + (b - a)].to(g.device, torch.float32)
            else:
                out[a - lo:b - lo] = flat[a:b].float()
        comm.allreduce(out, "sum", g.ranks)
        return out
