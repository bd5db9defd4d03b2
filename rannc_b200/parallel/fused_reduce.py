"""Host side of the fused gradient path: reduce-scatter + optimizer update + all-gather over peer memory,
bucket by bucket, while backward is still running.

The flat gradient and parameter buffers of a rank set are allocated in
symmetric memory (``torch.distributed._symmetric_memory``: CUDA VMM allocations
whose handles are exchanged once, so every rank holds every peer's base pointer
and, when the fabric offers it, a multicast address for NVLS).  A flat buffer is
a sequence of buckets (``FlatGroup.buckets``) and every rank owns one slice of
each.  For a bucket, ``rs_adam.cu`` pulls and reduces this rank's slice of every
peer's gradients, updates the fp32 master slice and pushes the new 16-bit
parameters into every peer's buffer -- the work the reference spreads over a
per-parameter ncclAllReduce (or bucketed ncclReduceScatter), scaling kernels, the
optimizer and an ncclAllGather before the next forward
(src/comp/ParamStorage.cpp:347-596).

When it runs.  The fused operators report, at the end of their backward, the
parameters whose gradients they have just written (``ops.functional.notify_grads``).
The first backward only counts those reports per bucket; from the second step on a
bucket is launched, on a side stream and with a small CTA budget, as soon as its
count is reached during the last micro-batch's backward -- so the reduction, and
the update itself, overlap the rest of backward (the reference reduces after the
whole backward, src/comp/Backward.cpp:100-107).  Each launch is preceded by a
one-warp barrier kernel over the owner set ("this bucket's gradients are final on
every rank"), so the reduction kernel itself never waits and never holds SMs idle;
one more barrier at the optimizer step separates the peers' writes into this
rank's parameters from the next forward.  Buckets are launched in one fixed order
on every rank.

Two ways to split the work:
  * update in backward (default when nothing needs the reduced gradients): one launch per bucket does
    reduce + update + publish;
  * reduce in backward, update at the step: used when gradient clipping, fp16 loss scaling or a reader of
    gradients (``clip_grad_norm``, ``get_param_grad``) needs the reduced gradients first.  The reduction
    launches write the reduced slice back into this rank's own gradient buffer and accumulate its sum of
    squares; the step launches the update with the [multiplier, skip] pair computed from it.

Used when: mixed precision (fp32 master), ZeRO, Adam / AdamW / SGD without amsgrad, a CUDA device, more than
one rank in the owner set, every parameter of the group handed to the optimizer and trainable.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional

import torch

from ..ops import _lib
from ..utils.config import conf
from ..utils.log import get_logger
from . import comm

logger = get_logger("FusedReduce")

MAX_PEERS = 8
RS_BEGIN, RS_END, RS_PULL, RS_UPDATE, RS_STORE_GRAD = 1, 2, 4, 8, 16


class _Args(ctypes.Structure):
    _fields_ = [
        ("peer_grad", ctypes.c_void_p * MAX_PEERS), ("peer_param", ctypes.c_void_p * MAX_PEERS),
        ("peer_flags", ctypes.c_void_p * MAX_PEERS),
        ("mc_grad", ctypes.c_void_p), ("mc_param", ctypes.c_void_p),
        ("master", ctypes.c_void_p), ("m", ctypes.c_void_p), ("v", ctypes.c_void_p),
        ("done_counter", ctypes.c_void_p),
        ("lo", ctypes.c_int64), ("len", ctypes.c_int64),
        ("nranks", ctypes.c_int32), ("my_idx", ctypes.c_int32),
        ("epoch", ctypes.c_uint32), ("grad_mul", ctypes.c_float),
        ("lr", ctypes.c_float), ("beta1", ctypes.c_float), ("beta2", ctypes.c_float), ("eps", ctypes.c_float),
        ("weight_decay", ctypes.c_float), ("bias_corr1", ctypes.c_float), ("bias_corr2", ctypes.c_float),
        ("adamw", ctypes.c_int32), ("dtype16", ctypes.c_int32), ("num_ctas", ctypes.c_int32),
        ("mode", ctypes.c_int32),
        ("ctrl", ctypes.c_void_p), ("max_polls", ctypes.c_uint64),
        ("sumsq", ctypes.c_void_p),
    ]


def symm_empty(numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    import torch.distributed._symmetric_memory as symm_mem

    return symm_mem.empty(numel, dtype=dtype, device=device)


class _GroupState:
    def __init__(self):
        self.grad_hdl = None
        self.param_hdl = None
        self.flags = None
        self.flags_hdl = None
        self.flag_ptrs = None
        self.done = None
        self.epoch = [0, 0]                 # barrier counters of the two flag rows
        self.sumsq = None                   # device scalar: squared norm of this rank's reduced slices
        self.expected: List[int] = []       # reports per bucket in one backward (learned in the first one)
        self.seen: List[int] = []
        self.reduced: List[bool] = []       # bucket already reduced in this step
        self.updated: List[bool] = []       # bucket already updated + published in this step
        self.next = 0                       # position in ``order`` of the next bucket to launch
        self.order: List[int] = []          # fixed launch order (last bucket first: backward produces it first)


class FusedGradReducer:
    """One instance per RaNNCModule; owns the symmetric-memory handles of every flat group."""

    def __init__(self, storage, optimizer):
        self.storage = storage
        self.optimizer = optimizer
        self.states: Dict[int, _GroupState] = {}
        self.handles_reduce = True
        self.pending = False                # local gradients are final, (part of) the reduction is still to come
        self.plain_groups = []
        # multimem.ld_reduce / multimem.st through the switch, or plain peer loads / stores.  Measured on two and
        # on eight B200s the peer-load path is the faster one for this access pattern (every thread keeps
        # 2 x nranks 16-byte loads in flight), so it is the default; RANNC_USE_MULTIMEM=1 selects the other.
        self.use_multimem = bool(int(os.environ.get("RANNC_USE_MULTIMEM", "0")))
        self.stream: Optional[torch.cuda.Stream] = None
        self.overlap = bool(conf("overlap_grad_reduce"))
        self.update_in_backward = bool(conf("fused_update_in_backward"))
        self.need_grads = False             # a reader of reduced gradients was seen: keep reduce and update apart
        self.learned = False
        self.armed = False                  # the running backward is the last one before the step
        self.step_begun = False             # hyper-parameters / step counters of this step already advanced
        self.bucket_of_param: Dict[int, tuple] = {}
        self.launched_in_backward = 0

    # ------------------------------------------------------------------ set-up
    @staticmethod
    def eligible(storage, optimizer) -> Optional[str]:
        if optimizer is None or type(optimizer) not in (torch.optim.Adam, torch.optim.AdamW, torch.optim.SGD):
            return "the optimizer is not Adam / AdamW / SGD"
        for g in optimizer.param_groups:
            if g.get("amsgrad") or g.get("maximize"):
                return "amsgrad / maximize are not supported"
        if not storage.amp or not storage.zero:
            return "needs mixed precision with enable_zero (sharded fp32 master)"
        for g in storage.groups:
            if g.flat_master is None:
                continue   # a full-precision group (batch-norm state): reduced and updated on the library path
            if g.nranks > MAX_PEERS:
                return f"more than {MAX_PEERS} ranks in an owner set"
            if any(og < 0 or not p.requires_grad for og, p in zip(g.opt_group, g.params)):
                # the kernel updates whole slices: a frozen parameter would still receive weight decay
                return "a flat buffer holds parameters that are frozen or not handed to the optimizer"
            if len({og for og in g.opt_group if og >= 0}) > 1:
                hp = [optimizer.param_groups[og] for og in sorted({og for og in g.opt_group if og >= 0})]
                keys = ("lr", "betas", "eps", "weight_decay") if "betas" in hp[0] else \
                    ("lr", "momentum", "dampening", "nesterov", "weight_decay")
                if any(tuple(h[k] for k in keys) != tuple(hp[0][k] for k in keys) for h in hp):
                    return "param groups with different hyper-parameters share a flat buffer"
        return None

    @classmethod
    def create(cls, storage, optimizer) -> "FusedGradReducer":
        why = cls.eligible(storage, optimizer)
        if why is not None:
            raise RuntimeError(why)
        import torch.distributed._symmetric_memory as symm_mem

        self = cls(storage, optimizer)
        self.plain_groups = [g for g in storage.groups if g.flat_master is None]
        for g in storage.groups:
            if g.flat_master is None:
                continue
            st = _GroupState()
            if g.nranks > 1:
                if not getattr(g, "symmetric", False):
                    raise RuntimeError("flat buffers were not allocated in symmetric memory")
                pg = comm.group(g.ranks)
                st.grad_hdl = symm_mem.rendezvous(g.flat_grad, pg)
                st.param_hdl = symm_mem.rendezvous(g.flat_param, pg)
                st.flags = symm_empty(2 * MAX_PEERS, torch.int32, g.device)
                st.flags.zero_()
                st.flags_hdl = symm_mem.rendezvous(st.flags, pg)
                st.flag_ptrs = (ctypes.c_void_p * MAX_PEERS)()
                for r in range(g.nranks):
                    st.flag_ptrs[r] = st.flags_hdl.buffer_ptrs[r]
            st.done = torch.zeros(1, dtype=torch.int32, device=g.device)
            st.sumsq = torch.zeros(1, dtype=torch.float32, device=g.device)
            nb = len(g.buckets)
            st.expected = [0] * nb
            st.seen = [0] * nb
            st.reduced = [False] * nb
            st.updated = [False] * nb
            st.order = list(range(nb - 1, -1, -1))
            self.states[id(g)] = st
            for i, p in enumerate(g.params):
                self.bucket_of_param[id(p)] = (g, g.bucket_of[i])
        if torch.cuda.is_available():
            self.stream = torch.cuda.Stream(device=storage.groups[0].device, priority=-1)
        torch.cuda.synchronize()
        comm.barrier()
        return self

    # ------------------------------------------------------------------ facts for reports
    def multimem_active(self) -> bool:
        for st in self.states.values():
            if st.grad_hdl is not None and self.use_multimem and (getattr(st.grad_hdl, "multicast_ptr", 0) or 0) \
                    and (getattr(st.param_hdl, "multicast_ptr", 0) or 0):
                return True
        return False

    def num_buckets(self) -> int:
        return sum(len(st.expected) for st in self.states.values())

    # ------------------------------------------------------------------ backward-time protocol
    def begin_backward(self, last: bool) -> None:
        """Called by the runtime before a backward pass; ``last``: it is the one right before the optimizer
        step (the last micro-batch, no gradient accumulation pending)."""
        self.armed = bool(last and self.overlap and self.learned and self.stream is not None and
                          self.handles_reduce)
        counting = not self.learned
        for st in self.states.values():
            st.seen = [0] * len(st.seen)
            if counting:
                st.expected = [0] * len(st.expected)
        self._counting = counting

    def on_grads(self, params) -> None:
        """Report from a fused operator's backward (or a gradient hook): the gradients of ``params`` have been
        written for this use of the parameters."""
        for p in params:
            hit = self.bucket_of_param.get(id(p))
            if hit is None:
                continue
            g, b = hit
            st = self.states[id(g)]
            if self._counting:
                st.expected[b] += 1
                continue
            st.seen[b] += 1
            if self.armed and st.seen[b] == st.expected[b]:
                self._launch_ready(g, st)

    def _launch_ready(self, g, st) -> None:
        """Launches, in the fixed order, every bucket whose gradients are complete."""
        while st.next < len(st.order):
            b = st.order[st.next]
            if st.seen[b] < st.expected[b]:
                return
            self._launch_bucket(g, st, b, overlapped=True)
            self.launched_in_backward += 1
            st.next += 1

    def end_backward(self) -> None:
        if getattr(self, "_counting", False):
            self.learned = True
            self._counting = False
        self.armed = False

    def mark_ready(self):
        """Called at the end of the last backward: the local gradients are final."""
        self.pending = True
        if self.plain_groups:
            # groups without a 16-bit / fp32-master pair take the collective path right away
            self.storage.allreduce_grads_zero(only=self.plain_groups)

    # ------------------------------------------------------------------ launches
    def _moments(self, g):
        """The flat Adam moments are shared with the non-fused optimizer step (``opt._FlatState``)."""
        from ..opt import _FlatState

        fs = self.optimizer._rannc_flat_state.get(id(g))
        if fs is None:
            kind = "sgd" if type(self.optimizer) is torch.optim.SGD else "adam"
            fs = self.optimizer._rannc_flat_state[id(g)] = _FlatState(g.local_len, g.device, kind)
        return fs

    def _begin_step(self) -> None:
        """Advances the step counters once per optimizer step, before the first update launch of the step."""
        if self.step_begun:
            return
        self.step_begun = True
        for g in self.storage.groups:
            if g.flat_master is not None:
                self._moments(g).step += 1

    def _split_mode(self) -> bool:
        """True: reduce now, update at the step (something needs the reduced gradients in between)."""
        mod = getattr(self.optimizer, "_rannc_module", None)
        needs_norm = bool(mod is not None and mod._needs_grad_norm())
        return self.need_grads or needs_norm or not self.update_in_backward

    def _fill_common(self, a: _Args, g, st) -> None:
        if g.nranks > 1:
            for r in range(g.nranks):
                a.peer_grad[r] = st.grad_hdl.buffer_ptrs[r]
                a.peer_param[r] = st.param_hdl.buffer_ptrs[r]
                a.peer_flags[r] = st.flags_hdl.buffer_ptrs[r]
            mcg = getattr(st.grad_hdl, "multicast_ptr", 0) or 0
            mcp = getattr(st.param_hdl, "multicast_ptr", 0) or 0
            if self.use_multimem and mcg and mcp:
                a.mc_grad, a.mc_param = mcg, mcp
        else:
            a.peer_grad[0] = g.flat_grad.data_ptr()
            a.peer_param[0] = g.flat_param.data_ptr()
            if st.flags is None:
                st.flags = torch.zeros(2 * MAX_PEERS, dtype=torch.int32, device=g.device)
            a.peer_flags[0] = st.flags.data_ptr()
        a.done_counter = st.done.data_ptr()
        a.nranks, a.my_idx = g.nranks, g.my_index
        a.dtype16 = 1 if g.dtype == torch.bfloat16 else 0
        a.max_polls = 0

    def _fill_hyper(self, a: _Args, g, fs) -> bool:
        ogs = sorted({og for og in g.opt_group if og >= 0})
        if not ogs:
            return False
        hp = self.optimizer.param_groups[ogs[0]]
        sgd = type(self.optimizer) is torch.optim.SGD
        a.weight_decay = float(hp["weight_decay"])
        if sgd:
            a.lr, a.beta1, a.beta2 = float(hp["lr"]), float(hp["momentum"]), float(hp.get("dampening", 0.0))
            a.eps = 1.0 if hp.get("nesterov") else 0.0
            a.bias_corr1, a.bias_corr2 = (0.0 if fs.step == 1 else 1.0), 1.0
            a.adamw = 2
        else:
            b1, b2 = hp["betas"]
            a.lr, a.beta1, a.beta2, a.eps = float(hp["lr"]), float(b1), float(b2), float(hp["eps"])
            a.bias_corr1, a.bias_corr2 = 1.0 - b1 ** fs.step, 1.0 - b2 ** fs.step
            a.adamw = 1 if type(self.optimizer) is torch.optim.AdamW else 0
        return True

    def _barrier(self, g, st, row: int) -> None:
        if g.nranks <= 1:
            return
        st.epoch[row] += 1
        _lib.check(_lib.lib().rb_peer_barrier(st.flag_ptrs, ctypes.c_int(g.nranks), ctypes.c_int(g.my_index),
                                              ctypes.c_int(row), ctypes.c_uint(st.epoch[row]),
                                              ctypes.c_ulonglong(0), _lib.stream_ptr()), "rb_peer_barrier")

    def _launch_bucket(self, g, st, b: int, overlapped: bool, ctrl: Optional[torch.Tensor] = None) -> None:
        """Reduction (and, unless something needs the reduced gradients first, the update) of bucket ``b``."""
        split = self._split_mode()
        fs = self._moments(g)
        if not split:
            self._begin_step()
        a = _Args()
        self._fill_common(a, g, st)
        pa, pb, loc = g.pieces[b]
        a.lo, a.len = pa, pb - pa
        a.master = g.flat_master.data_ptr() + 4 * loc
        a.m = fs.m.data_ptr() + 4 * loc
        a.v = (fs.v.data_ptr() if fs.v is not None else fs.m.data_ptr()) + 4 * loc
        a.grad_mul = 1.0 / comm.get_world_size()
        a.ctrl = None if (ctrl is None or split) else ctrl.data_ptr()
        if split:
            a.mode = RS_PULL | RS_STORE_GRAD
            a.sumsq = st.sumsq.data_ptr()
        else:
            if not self._fill_hyper(a, g, fs):
                st.reduced[b] = st.updated[b] = True
                return
            a.mode = RS_PULL | RS_UPDATE
        a.num_ctas = max(1, int(conf("fused_reduce_ctas"))) if overlapped else 0
        if overlapped:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                self.stream.wait_event(ev)
                self._barrier(g, st, 0)
                _lib.check(_lib.lib().rb_rs_adam_ag(ctypes.byref(a), _lib.stream_ptr()), "rb_rs_adam_ag")
        else:
            self._barrier(g, st, 0)
            _lib.check(_lib.lib().rb_rs_adam_ag(ctypes.byref(a), _lib.stream_ptr()), "rb_rs_adam_ag")
        st.reduced[b] = True
        st.updated[b] = not split

    def _join_side_stream(self) -> None:
        if self.stream is not None:
            ev = torch.cuda.Event()
            ev.record(self.stream)
            torch.cuda.current_stream().wait_event(ev)

    def ensure_reduced(self, sticky: bool = True) -> None:
        """For readers of gradients between backward and the step (``clip_grad_norm``, ``get_param_grad``):
        finishes the reduction without updating.  A bucket that was already updated during backward cannot be
        read any more; from the first such request on (``sticky``), reduction and update are kept apart."""
        if not self.pending:
            return
        if sticky:
            self.need_grads = True
        for g in self.storage.groups:
            st = self.states.get(id(g))
            if st is None:
                continue
            if any(st.updated):
                raise RuntimeError(
                    "the gradients of this step were already consumed by the update that overlaps backward; "
                    "gradient readers (clip_grad_norm, get_param_grad) must be used from the first step on, or "
                    "set RANNC_FUSED_UPDATE_IN_BACKWARD=false")
            self._join_side_stream()
            for b in st.order:
                if not st.reduced[b]:
                    self._launch_bucket(g, st, b, overlapped=False)

    def adds_sumsq(self, g, out: torch.Tensor) -> bool:
        """Adds the squared norm of this rank's reduced slices of ``g`` to ``out`` when the reduction launches
        have accumulated it.  False: the caller computes it."""
        st = self.states.get(id(g))
        if st is None or not self.pending or not all(st.reduced) or any(st.updated):
            return False
        self._join_side_stream()
        out.add_(st.sumsq)
        return True

    def step(self, ctrl: Optional[torch.Tensor] = None):
        """Optimizer step: whatever the backward-time launches have not done yet, then the closing barrier."""
        lib = _lib.lib()
        self._join_side_stream()
        self._begin_step()
        for g in self.storage.groups:
            if g.flat_master is None:
                continue
            st = self.states[id(g)]
            fs = self._moments(g)
            for b in st.order:
                if st.updated[b]:
                    continue
                if not st.reduced[b] and not self._split_mode():
                    self._launch_bucket(g, st, b, overlapped=False, ctrl=ctrl)
                    continue
                if not st.reduced[b]:
                    self._launch_bucket(g, st, b, overlapped=False)
                # update from the reduced slice in this rank's own gradient buffer
                a = _Args()
                self._fill_common(a, g, st)
                pa, pb, loc = g.pieces[b]
                a.lo, a.len = pa, pb - pa
                a.master = g.flat_master.data_ptr() + 4 * loc
                a.m = fs.m.data_ptr() + 4 * loc
                a.v = (fs.v.data_ptr() if fs.v is not None else fs.m.data_ptr()) + 4 * loc
                a.grad_mul = 1.0
                a.ctrl = None if ctrl is None else ctrl.data_ptr()
                a.mode = RS_UPDATE
                if self._fill_hyper(a, g, fs):
                    _lib.check(lib.rb_rs_adam_ag(ctypes.byref(a), _lib.stream_ptr()), "rb_rs_adam_ag")
                st.updated[b] = True
            # every peer has finished reading this rank's gradients and writing its parameters
            self._barrier(g, st, 1)
            st.reduced = [False] * len(st.reduced)
            st.updated = [False] * len(st.updated)
            st.next = 0
            st.sumsq.zero_()
        self.pending = False
        self.step_begun = False

    def skip_step(self) -> None:
        """An overflow step: nothing is updated, but the peers still have to agree that this rank's buffers
        may be overwritten (zero_grad) -- same closing barrier as a real step."""
        self._join_side_stream()
        for g in self.storage.groups:
            st = self.states.get(id(g))
            if st is None:
                continue
            self._barrier(g, st, 1)
            st.reduced = [False] * len(st.reduced)
            st.updated = [False] * len(st.updated)
            st.next = 0
            st.sumsq.zero_()
        self.pending = False
        self.step_begun = False

    def publish_state(self):
        """Per-parameter views of the flat moments in ``optimizer.state`` (torch's layout)."""
        for g in self.storage.groups:
            if g.flat_master is None:
                continue
            self.optimizer._rannc_publish_state(g, self._moments(g))


def compare_with_collectives(module, optimizer, run_step) -> float:
    """Value check of the fused path against NCCL collectives: from the same parameters, moments and dropout
    counters, ``run_step()`` (forward + backward + optimizer step + zero_grad) runs once down each path; returns
    the largest |difference| of the updated fp32 master values relative to the largest update, over all ranks.
    The state is put back afterwards.  Collective over the world."""
    from ..ops import functional as RF

    storage = module._storage
    red = module._fused_reducer
    groups = [g for g in storage.groups if g.flat_master is not None]

    def snapshot():
        snap = []
        for g in groups:
            fs = optimizer._rannc_flat_state.get(id(g))
            snap.append((g.flat_param.clone(), g.flat_master.clone(),
                         None if fs is None else (fs.m.clone(), None if fs.v is None else fs.v.clone(), fs.step)))
        return snap, RF.rng.get_state()

    def restore(snap):
        s, rng = snap
        for g, (fp, fm, mom) in zip(groups, s):
            g.flat_param.copy_(fp)
            g.flat_master.copy_(fm)
            fs = optimizer._rannc_flat_state.get(id(g))
            if fs is not None and mom is not None:
                fs.m.copy_(mom[0])
                if fs.v is not None:
                    fs.v.copy_(mom[1])
                fs.step = mom[2]
        RF.rng.set_state(rng)
        RF.bump_param_epoch()

    torch.cuda.synchronize()
    comm.barrier()
    snap = snapshot()
    run_step()
    torch.cuda.synchronize()
    comm.barrier()
    fused = [g.flat_master.clone() for g in groups]
    restore(snap)
    torch.cuda.synchronize()
    comm.barrier()
    red.handles_reduce = False
    try:
        run_step()
        torch.cuda.synchronize()
    finally:
        red.handles_reduce = True
    comm.barrier()
    err = torch.zeros(2, dtype=torch.float32, device=groups[0].device)
    for g, f, (fp, fm, _) in zip(groups, fused, snap[0]):
        err[0] = torch.maximum(err[0], (f - g.flat_master).abs().max())
        err[1] = torch.maximum(err[1], (g.flat_master - fm).abs().max())
    comm.allreduce(err, "max")
    restore(snap)
    torch.cuda.synchronize()
    comm.barrier()
    return float(err[0] / err[1].clamp_min(1e-30))
