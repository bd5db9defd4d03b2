"""Host side of the fused gradient path: reduce-scatter + Adam + all-gather in one kernel per rank.

The flat gradient and parameter buffers of a rank set are allocated in
symmetric memory (``torch.distributed._symmetric_memory``: CUDA VMM allocations
whose handles are exchanged once, so every rank holds every peer's base pointer
and, when the fabric offers it, a multicast address for NVLS).  At the
optimizer step ``rs_adam.cu`` pulls and reduces this rank's shard of every
peer's gradients, updates the fp32 master shard and pushes the new 16-bit
parameters into every peer's buffer -- the work the reference spreads over a
per-parameter ncclAllReduce (or bucketed ncclReduceScatter), scaling kernels, the
optimizer and an ncclAllGather before the next forward
(src/comp/ParamStorage.cpp:347-596).

Used when: mixed precision (fp32 master), Adam / AdamW without amsgrad, a CUDA
device, more than one rank in the owner set, no gradient clipping and no fp16
loss scaling (those need the reduced norm first and take the NCCL path).
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional

import torch

from ..ops import _lib
from ..utils.config import conf
from ..utils.log import get_logger
from . import comm

logger = get_logger("FusedReduce")

MAX_PEERS = 8


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
        ("pad_", ctypes.c_int32),
        ("ctrl", ctypes.c_void_p), ("max_polls", ctypes.c_uint64),
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
        self.done = None
        self.epoch = 0


class FusedGradReducer:
    """One instance per RaNNCModule; owns the symmetric-memory handles of every flat group."""

    def __init__(self, storage, optimizer):
        self.storage = storage
        self.optimizer = optimizer
        self.states: Dict[int, _GroupState] = {}
        self.handles_reduce = True
        self.pending = False
        self.plain_groups = []
        self.use_multimem = bool(int(__import__("os").environ.get("RANNC_USE_MULTIMEM", "1")))

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
            st.done = torch.zeros(1, dtype=torch.int32, device=g.device)
            self.states[id(g)] = st
        torch.cuda.synchronize()
        comm.barrier()
        return self

    def mark_ready(self):
        """Called at the end of backward: the local gradients are final; the reduction itself happens
        inside the optimizer step's kernel."""
        self.pending = True
        if self.plain_groups:
            # groups without a 16-bit / fp32-master pair take the collective path right away
            self.storage.allreduce_grads_zero(only=self.plain_groups)

    def _moments(self, g):
        """The flat Adam moments are shared with the non-fused optimizer step (``opt._FlatState``)."""
        from ..opt import _FlatState

        fs = self.optimizer._rannc_flat_state.get(id(g))
        if fs is None:
            kind = "sgd" if type(self.optimizer) is torch.optim.SGD else "adam"
            fs = self.optimizer._rannc_flat_state[id(g)] = _FlatState(g.shard[1] - g.shard[0], g.device, kind)
        return fs

    def step(self, ctrl: Optional[torch.Tensor] = None):
        world = comm.get_world_size()
        lib = _lib.lib()
        for g in self.storage.groups:
            if g.flat_master is None:
                continue
            st = self.states[id(g)]
            fs = self._moments(g)
            fs.step += 1
            st.epoch += 1
            ogs = sorted({og for og in g.opt_group if og >= 0})
            if not ogs:
                continue
            hp = self.optimizer.param_groups[ogs[0]]
            sgd = type(self.optimizer) is torch.optim.SGD
            b1, b2 = (float(hp["momentum"]), float(hp.get("dampening", 0.0))) if sgd else hp["betas"]
            a = _Args()
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
            a.master, a.m = g.flat_master.data_ptr(), fs.m.data_ptr()
            a.v = fs.v.data_ptr() if fs.v is not None else fs.m.data_ptr()
            a.done_counter = st.done.data_ptr()
            a.lo, a.len = g.shard[0], g.shard[1] - g.shard[0]
            a.nranks, a.my_idx = g.nranks, g.my_index
            a.epoch = st.epoch
            a.grad_mul = 1.0 / world
            a.weight_decay = float(hp["weight_decay"])
            if sgd:
                a.lr, a.beta1, a.beta2 = float(hp["lr"]), float(b1), float(b2)
                a.eps = 1.0 if hp.get("nesterov") else 0.0
                a.bias_corr1, a.bias_corr2 = (0.0 if fs.step == 1 else 1.0), 1.0
                a.adamw = 2
            else:
                a.lr, a.beta1, a.beta2, a.eps = float(hp["lr"]), float(b1), float(b2), float(hp["eps"])
                a.bias_corr1, a.bias_corr2 = 1.0 - b1 ** fs.step, 1.0 - b2 ** fs.step
                a.adamw = 1 if type(self.optimizer) is torch.optim.AdamW else 0
            a.dtype16 = 1 if g.dtype == torch.bfloat16 else 0
            a.num_ctas = int(conf("fused_reduce_ctas")) if _has_conf("fused_reduce_ctas") else 0
            a.ctrl = None if ctrl is None else ctrl.data_ptr()
            a.max_polls = 0
            _lib.check(lib.rb_rs_adam_ag(ctypes.byref(a), _lib.stream_ptr()), "rb_rs_adam_ag")
        self.pending = False

    def publish_state(self):
        """Per-parameter views of the flat moments in ``optimizer.state`` (torch's layout)."""
        for g in self.storage.groups:
            if g.flat_master is None:
                continue
            fs = self._moments(g)
            lo = g.shard[0]
            for i, mp in enumerate(g.master_params):
                if mp is None or g.opt_group[i] < 0:
                    continue
                a, b = g.local_range(i)
                s = self.optimizer.state[mp]
                if fs.v is None:
                    s["momentum_buffer"] = fs.m[a - lo:b - lo].view(mp.shape)
                    continue
                s["step"] = torch.tensor(float(fs.step))
                s["exp_avg"] = fs.m[a - lo:b - lo].view(mp.shape)
                s["exp_avg_sq"] = fs.v[a - lo:b - lo].view(mp.shape)


def _has_conf(name: str) -> bool:
    try:
        conf(name)
        return True
    except Exception:  # noqa: BLE001
        return False
