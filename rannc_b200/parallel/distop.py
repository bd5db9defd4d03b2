"""Tensor-partitioned linear layer (``distop``): the weight of ``aten::linear`` is sliced along its input
dimension over the replicas of a stage, so each rank stores 1/n of it.

Same semantics as the reference's ``rannc::linear_dist`` (src/distop/PartitionTensor.cpp:9-10,230-298,
src/distop/DistMatmul.cpp:97-304): every member of the group works on its own batch slice with the FULL
weight, which is re-assembled on the fly --

* forward        Y  = X  gather(W)^T     all-gather -> GEMM
* input gradient dX = dY gather(W)       all-gather -> GEMM
* weight gradient dW_j = sum_r (dY_r^T X_r)[:, block j]     GEMM -> reduce-scatter

Here each of the three is ONE kernel launch per rank (``csrc/cuda/gemm_tcgen05.cu``): the all-gather is
a prologue in which the epilogue warps copy the peers' shards into a local buffer with plain peer loads
while the tensor core already works on the shard that is local, and the reduce-scatter is the GEMM
epilogue adding each column block into its owner's fp32 gradient buffer over NVLink.  No library GEMM
sees peer memory and no TMA reads it: the TMA loads read the local buffer only.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from ..ops import _lib
from ..ops.gemm import gemm
from ..ops import kernels as K
from . import comm

MAX_PEERS = 8


class DistGroup:
    """Buffers a rank set shares for its tensor-partitioned layers.

    ``local=True`` builds an emulated group inside one process (every "rank's" memory is on this GPU), which is
    how the kernels are tested on a single device."""

    def __init__(self, ranks: Sequence[int], max_weight_numel: int, dtype=torch.bfloat16, device=None,
                 local: bool = False, kernels: Optional[bool] = None):
        self.ranks = tuple(sorted(ranks))
        self.n = len(self.ranks)
        self.local = local
        self.device = device or comm.device()
        self.dtype = dtype
        self.my_idx = 0 if local else self.ranks.index(comm.get_rank())
        # without the kernels (CPU ranks, or fused_kernels=false) the same operator runs on collectives
        self.kernels = self.device.type == "cuda" if kernels is None else bool(kernels)
        self.epoch = 0
        self._flag_ptrs = None
        if not self.kernels:
            return
        self.staging = torch.empty(max_weight_numel, dtype=dtype, device=self.device)
        self.ag_flags = torch.zeros(8, dtype=torch.int32, device=self.device)
        if not local and self.n > 1:
            import torch.distributed._symmetric_memory as symm_mem

            self.flags = symm_mem.empty(2 * MAX_PEERS, dtype=torch.int32, device=self.device).zero_()
            torch.cuda.synchronize(self.device)   # zeroed before any peer can learn the address
            hdl = symm_mem.rendezvous(self.flags, comm.group(self.ranks))
            self._flag_ptrs = [int(p) for p in hdl.buffer_ptrs]
            self._keep = [hdl]

    def alloc_shared(self, numel: int, dtype) -> "SharedTensor":
        return SharedTensor(self, numel, dtype)

    def barrier(self):
        """Stream-ordered barrier over the group (flag handshake kernel; bounded waits)."""
        if self.local or self.n == 1 or not self.kernels:
            return
        self.epoch += 1
        arr = (ctypes.c_void_p * 8)(*([ctypes.c_void_p(p) for p in self._flag_ptrs] + [None] * (8 - self.n)))
        _lib.check(_lib.lib().rb_peer_barrier(arr, ctypes.c_int(self.n), ctypes.c_int(self.my_idx), ctypes.c_int(0),
                                              ctypes.c_uint(self.epoch), ctypes.c_ulonglong(0), _lib.stream_ptr()),
                   "rb_peer_barrier")


class SharedTensor:
    """A tensor every rank of the group allocates with the same size in symmetric memory; ``ptrs[r]`` is
    rank r's copy as seen from this rank."""

    def __init__(self, grp: DistGroup, numel: int, dtype):
        self.grp = grp
        if grp.local or grp.n == 1:
            self.t = torch.zeros(numel, dtype=dtype, device=grp.device)
            self.ptrs = [self.t.data_ptr()]
        else:
            import torch.distributed._symmetric_memory as symm_mem

            self.t = symm_mem.empty(numel, dtype=dtype, device=grp.device).zero_()
            torch.cuda.synchronize(grp.device)
            self.hdl = symm_mem.rendezvous(self.t, comm.group(grp.ranks))
            self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]


def _gather_spec(grp: DistGroup, shard_ptrs: List[int], rows: int, cols: int):
    return {"nranks": grp.n, "my_idx": grp.my_idx, "rows": rows, "cols": cols, "flags": grp.ag_flags.data_ptr(),
            "src": shard_ptrs}


class _LinearDist(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_shard, bias, grp, shard_ptrs, grad_ptrs, w_main_grad, grad_scale):
        # w_shard: [N, K / n]; shard_ptrs[r]: rank r's shard; grad_ptrs[r]: rank r's fp32 [N, K / n] gradient
        N, Ks = w_shard.shape
        Kfull = Ks * grp.n
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        wfull = grp.staging[: N * Kfull].view(N, Kfull)
        y = gemm(x2, wfull, bias=bias, gather=_gather_spec(grp, shard_ptrs, N, Ks))
        ctx.save_for_backward(x2)
        ctx.meta = (grp, shard_ptrs, grad_ptrs, N, Ks, bias, w_main_grad, x.shape, grad_scale)
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        grp, shard_ptrs, grad_ptrs, N, Ks, bias, w_mg, x_shape, grad_scale = ctx.meta
        Kfull = Ks * grp.n
        dy2 = dy.reshape(-1, N)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        wfull = grp.staging[: N * Kfull].view(N, Kfull)
        dx = None
        if ctx.needs_input_grad[0]:
            # the weight is gathered again (it is not kept between forward and backward)
            dx = gemm(dy2, wfull, trans_b=False, gather=_gather_spec(grp, shard_ptrs, N, Ks)).view(x_shape)
        # dW = dy^T x for this rank's batch slice; column block j is added into rank j's gradient buffer
        _gemm_rs(dy2, x2, N, Kfull, grad_ptrs, Ks, grad_scale)
        db = None
        if bias is not None and ctx.needs_input_grad[2]:
            mg = getattr(bias, "main_grad", None)
            if mg is not None:
                K.colsum(dy2, out=mg)
            else:
                db = K.colsum(dy2).to(bias.dtype)
        return dx, None, db, None, None, None, None, None


class _LinearDistCollective(torch.autograd.Function):
    """The same operator on library collectives (gloo on CPU ranks, NCCL when the kernels are switched off):
    all-gather of the slices, a plain matmul, and an all-reduce of the full weight gradient of which each
    rank keeps its block -- the way the reference runs it (src/distop/DistMatmul.cpp:97-214)."""

    @staticmethod
    def _gather(w, grp):
        import torch.distributed as dist

        if grp.n == 1:
            return w.detach()
        parts = [torch.empty_like(w) for _ in range(grp.n)]
        dist.all_gather(parts, w.detach().contiguous(), group=comm.group(grp.ranks))
        return torch.cat(parts, dim=1)

    @staticmethod
    def forward(ctx, x, w_shard, bias, grp, grad_scale):
        wfull = _LinearDistCollective._gather(w_shard, grp)
        ctx.save_for_backward(x, w_shard)
        ctx.meta = (grp, bias is not None, grad_scale)
        return torch.nn.functional.linear(x, wfull, bias)

    @staticmethod
    def backward(ctx, dy):
        x, w_shard = ctx.saved_tensors
        grp, has_bias, grad_scale = ctx.meta
        wfull = _LinearDistCollective._gather(w_shard, grp)
        dx = dy @ wfull if ctx.needs_input_grad[0] else None
        dy2, x2 = dy.reshape(-1, dy.shape[-1]), x.reshape(-1, x.shape[-1])
        dw = (dy2.t() @ x2) * grad_scale
        if grp.n > 1:
            comm.allreduce(dw, "sum", grp.ranks)
        ks = w_shard.shape[1]
        gw = dw[:, grp.my_idx * ks:(grp.my_idx + 1) * ks].contiguous()
        db = dy2.sum(0) if has_bias and ctx.needs_input_grad[2] else None
        return dx, gw, db, None, None


def _gemm_rs(dy2, x2, N, Kfull, grad_ptrs, Ks, alpha):
    """dW[N, Kfull] = dy2^T x2, scattered by column blocks of width Ks into the fp32 buffers grad_ptrs[j]."""
    from ..ops.gemm import _Args, _dt, _mat, ACCUM

    a, ar, ac, lda, _, _ = _mat(dy2)   # stored [M, N] -> op(A) = A^T : [N, M]
    b, br, bc, ldb, _, _ = _mat(x2)    # stored [M, Kfull] -> MN-major B
    M = ar
    args = _Args(_lib.ptr(a), _lib.ptr(b), grad_ptrs[0], None, None, None, None, N, Kfull, M, 1, lda, ldb, Ks, 0, 0,
                 0, 1, 1, _dt(a), 1, ACCUM, 0, float(alpha), 0)
    if len(grad_ptrs) > 1:
        args.rs_nranks = len(grad_ptrs)
        for i, p in enumerate(grad_ptrs):
            args.rs_peer[i] = int(p)
    _lib.check(_lib.lib().rb_gemm(ctypes.byref(args), _lib.stream_ptr()), "rb_gemm (reduce-scatter)")


def linear_dist(x, w_shard, bias, grp: DistGroup, shard_ptrs: List[int], grad_ptrs: List[int],
                grad_scale: Optional[float] = None):
    """``x @ gather(w_shards).T + bias`` for a weight sliced along its input dimension over ``grp``.

    The weight gradient is the SUM over the group's batch slices times ``grad_scale``; by default that is
    1 / world size, the data-parallel average (reference: ParamStorage.cpp:377-379).  Inside RaNNCModule
    the storage applies that average to every gradient buffer itself, so it passes 1."""
    if grad_scale is None:
        grad_scale = 1.0 / (comm.get_world_size() if not grp.local else 1)
    if not grp.kernels:
        return _LinearDistCollective.apply(x, w_shard, bias, grp, grad_scale)
    return _LinearDist.apply(x, w_shard, bias, grp, shard_ptrs, grad_ptrs, getattr(w_shard, "main_grad", None),
                             grad_scale)


class LinearDistSite:
    """What one rewritten ``linear`` node of a stage graph needs at run time."""

    def __init__(self, grp: DistGroup, shard_ptrs: List[int], grad_ptrs: List[int]):
        self.grp, self.shard_ptrs, self.grad_ptrs = grp, shard_ptrs, grad_ptrs


_SITES: dict = {}


def register_site(site: LinearDistSite) -> int:
    key = len(_SITES) + 1
    _SITES[key] = site
    return key


def clear_sites() -> None:
    _SITES.clear()


def linear_dist_op(x, w_shard, bias, key: int):
    """Graph-level form of ``linear_dist``: ``key`` names a registered site (graphs hold plain values only)."""
    st = _SITES[key]
    return linear_dist(x, w_shard, bias, st.grp, st.shard_ptrs, st.grad_ptrs, 1.0)


class DistLinear(torch.nn.Module):
    """``nn.Linear`` whose weight is stored as [out, in / n] per rank.  ``from_linear`` slices an existing
    layer; the gradient of the local slice accumulates (already reduced over the group and averaged over
    the world) in ``weight.main_grad`` (fp32)."""

    def __init__(self, grp: DistGroup, out_features: int, in_features: int, bias: bool = True, dtype=torch.bfloat16):
        super().__init__()
        if in_features % (256 * grp.n):
            raise ValueError("in_features must be a multiple of 256 x group size")
        self.grp = grp
        self.in_features, self.out_features = in_features, out_features
        ks = in_features // grp.n
        self._w = grp.alloc_shared(out_features * ks, dtype)
        self._g = grp.alloc_shared(out_features * ks, torch.float32)
        self.weight = torch.nn.Parameter(self._w.t.view(out_features, ks))
        self.weight.main_grad = self._g.t.view(out_features, ks)
        self.bias = torch.nn.Parameter(torch.zeros(out_features, dtype=dtype, device=grp.device)) if bias else None

    @classmethod
    def from_linear(cls, grp: DistGroup, lin: torch.nn.Linear, idx: Optional[int] = None) -> "DistLinear":
        m = cls(grp, lin.out_features, lin.in_features, lin.bias is not None, lin.weight.dtype)
        i = grp.my_idx if idx is None else idx
        ks = lin.in_features // grp.n
        with torch.no_grad():
            m.weight.copy_(lin.weight[:, i * ks:(i + 1) * ks])
            if lin.bias is not None:
                m.bias.copy_(lin.bias)
        return m

    def shard_ptrs(self):
        return self._w.ptrs

    def grad_ptrs(self):
        return self._g.ptrs

    def forward(self, x):
        return linear_dist(x, self.weight, self.bias, self.grp, self.shard_ptrs(), self.grad_ptrs())
