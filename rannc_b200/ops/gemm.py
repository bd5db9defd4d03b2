"""tcgen05 GEMM wrapper (``csrc/cuda/gemm_tcgen05.cu``)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib

BIAS, GELU, DGELU, RESIDUAL, ACCUM, AUX_OUT = 1, 2, 4, 8, 16, 32


class _Args(ctypes.Structure):
    _fields_ = [
        ("A", ctypes.c_void_p), ("B", ctypes.c_void_p), ("D", ctypes.c_void_p),
        ("bias", ctypes.c_void_p), ("residual", ctypes.c_void_p),
        ("aux_in", ctypes.c_void_p), ("aux_out", ctypes.c_void_p),
        ("M", ctypes.c_int64), ("N", ctypes.c_int64), ("K", ctypes.c_int64), ("batch", ctypes.c_int64),
        ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldd", ctypes.c_int64),
        ("strideA", ctypes.c_int64), ("strideB", ctypes.c_int64), ("strideD", ctypes.c_int64),
        ("a_major", ctypes.c_int32), ("b_major", ctypes.c_int32),
        ("in_dtype", ctypes.c_int32), ("out_dtype", ctypes.c_int32),
        ("flags", ctypes.c_int32), ("max_ctas", ctypes.c_int32),
        ("alpha", ctypes.c_float), ("rs_nranks", ctypes.c_int32),
        ("rs_peer", ctypes.c_void_p * 8),
        ("ag_nranks", ctypes.c_int32), ("ag_my_idx", ctypes.c_int32), ("ag_rows", ctypes.c_int32),
        ("ag_cols", ctypes.c_int32), ("ag_flags", ctypes.c_void_p), ("ag_src", ctypes.c_void_p * 8),
        ("conv_taps", ctypes.c_int32), ("conv_c", ctypes.c_int32), ("conv_b_tap_cols", ctypes.c_int32),
        ("b_row_shift", ctypes.c_int32), ("conv_shift", ctypes.c_int32 * 49),
        ("map_hp", ctypes.c_int32), ("map_wp", ctypes.c_int32), ("map_h", ctypes.c_int32),
        ("map_w", ctypes.c_int32), ("map_pad", ctypes.c_int32),
    ]


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float16:
        return 0
    raise TypeError(f"gemm: unsupported input dtype {t.dtype}")


def _tma_ready(t: torch.Tensor) -> torch.Tensor:
    """TMA wants a 16-byte aligned base and row strides that are multiples of 16 bytes.  Operands that do
    not qualify (e.g. a [M, 2] gradient) are copied into a buffer whose rows are padded to 8 elements; the
    logical extents stay the same, so the padding is never read as data."""
    ok = t.data_ptr() % 16 == 0 and t.stride(-1) == 1 and t.stride(-2) % 8 == 0 and \
        (t.dim() == 2 or t.stride(0) % 8 == 0)
    if ok:
        return t
    cols = t.shape[-1]
    pc = (cols + 7) // 8 * 8
    buf = torch.zeros(*t.shape[:-1], pc, dtype=t.dtype, device=t.device)
    view = buf[..., :cols]
    view.copy_(t)
    return view


def _mat(t: torch.Tensor):
    """Returns (tensor, rows, cols, ld, batch, batch_stride) for a 2-D/3-D tensor whose last dim is contiguous."""
    if t.dim() == 2:
        t = _tma_ready(t)
        return t, t.shape[0], t.shape[1], t.stride(0), 1, 0
    if t.dim() == 3:
        t = _tma_ready(t)
        return t, t.shape[1], t.shape[2], t.stride(1), t.shape[0], t.stride(0)
    raise ValueError("gemm operands must be 2-D or 3-D")


def gemm(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = True,
         bias=None, residual=None, aux_in=None, aux_out=None, gelu: bool = False,
         dgelu: bool = False, out: torch.Tensor | None = None, accumulate: bool = False,
         out_dtype: torch.dtype | None = None, alpha: float = 1.0, max_ctas: int = 0,
         rs_peers=None, rs_ld: int = 0, gather=None, conv=None, b_row_shift: int = 0,
         row_map=None) -> torch.Tensor:
    """``out = epilogue(alpha * op(a) @ op(b))``.

    ``a`` is stored ``[M, K]`` (``trans_a=False``) or ``[K, M]`` (``trans_a=True``).
    ``b`` is stored ``[N, K]`` (``trans_b=True``, the ``nn.Linear`` weight layout) or
    ``[K, N]`` (``trans_b=False``).  A leading batch dimension is allowed on both.

    ``conv = {"taps": T, "shifts": [...], "b_tap_cols": n}``: implicit-GEMM convolution.  ``a`` is the padded
    channels-last activation as ``[rows, C]``; the product runs over K = T x C, k-block by k-block reading the
    rows shifted by ``shifts[tap]`` (rows outside ``a`` read as zero).  ``b`` is ``[N, T*C]`` (``trans_b=True``) or
    ``[C, T*b_tap_cols]`` with tap t's ``[C, N]`` block at column ``t * b_tap_cols`` (``trans_b=False``).
    ``b_row_shift`` (``trans_b=False`` only): the rows of ``b`` a k-block reads are shifted by this many.
    ``row_map = (Hp, Wp, H, W, pad)``: the M rows are positions of a padded image grid; only the interior is
    stored, at the un-padded row index (``out`` has N_img * H * W rows).
    """
    a, ar, ac, lda, ba, sa = _mat(a)
    b, br, bc, ldb, bb, sb = _mat(b)
    M, K = (ac, ar) if trans_a else (ar, ac)
    N, Kb = (br, bc) if trans_b else (bc, br)
    if conv is not None:
        T = int(conv["taps"])
        if trans_a or a.dim() != 2 or b.dim() != 2 or len(conv["shifts"]) != T or lda != ac:
            raise ValueError("gemm: a convolution wants a contiguous 2-D [rows, C] activation")
        if trans_b:
            if bc != T * ac:
                raise ValueError(f"gemm: weight matrix has {bc} columns, expected {T} x {ac}")
        else:
            N = int(conv["n"])
            if br != ac or bc < (T - 1) * int(conv["b_tap_cols"]) + N:
                raise ValueError("gemm: weight matrix does not hold the taps' blocks")
        K = Kb = T * ac
    if K != Kb:
        raise ValueError(f"gemm: inner dimensions differ ({K} vs {Kb})")
    batch = max(ba, bb)
    if ba != bb and min(ba, bb) != 1:
        raise ValueError("gemm: batch sizes differ")
    if ba == 1 and batch > 1:
        sa = 0
    if bb == 1 and batch > 1:
        sb = 0
    odt = out_dtype or (out.dtype if out is not None else a.dtype)
    if out is None:
        if row_map is not None:
            raise ValueError("gemm: row_map needs an explicit output")
        shape = (M, N) if batch == 1 and a.dim() == 2 and b.dim() == 2 else (batch, M, N)
        out = torch.empty(shape, dtype=odt, device=a.device)
    ldd = out.stride(-2)
    sd = out.stride(0) if out.dim() == 3 else 0
    flags = 0
    if bias is not None:
        flags |= BIAS
    if gelu:
        flags |= GELU
    if dgelu:
        flags |= DGELU
    if residual is not None:
        flags |= RESIDUAL
    if accumulate:
        flags |= ACCUM
    if aux_out is not None:
        flags |= AUX_OUT
    args = _Args(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(residual),
        _lib.ptr(aux_in), _lib.ptr(aux_out), M, N, K, batch, lda, ldb, ldd, sa, sb, sd,
        1 if trans_a else 0, 0 if trans_b else 1, _dt(a), 0 if odt == a.dtype else 1, flags,
        max_ctas, float(alpha), 0)
    if rs_peers is not None and len(rs_peers) > 1:
        # reduce-scatter epilogue: column block j of the product is added into rank j's buffer
        args.rs_nranks = len(rs_peers)
        for i, ptr in enumerate(rs_peers):
            args.rs_peer[i] = int(ptr)
        if rs_ld:
            args.ldd = int(rs_ld)
    if gather is not None:
        args.ag_nranks = gather["nranks"]
        args.ag_my_idx = gather["my_idx"]
        args.ag_rows = gather["rows"]
        args.ag_cols = gather["cols"]
        args.ag_flags = gather["flags"]
        for i, ptr in enumerate(gather["src"]):
            args.ag_src[i] = int(ptr)
    if conv is not None:
        args.conv_taps = int(conv["taps"])
        args.conv_c = ac
        args.conv_b_tap_cols = int(conv.get("b_tap_cols", 0))
        for i, sh in enumerate(conv["shifts"]):
            args.conv_shift[i] = int(sh)
    if b_row_shift:
        if trans_b:
            raise ValueError("gemm: b_row_shift needs b stored [K, N]")
        args.b_row_shift = int(b_row_shift)
    if row_map is not None:
        args.map_hp, args.map_wp, args.map_h, args.map_w, args.map_pad = (int(v) for v in row_map)
    rc = _lib.lib().rb_gemm(ctypes.byref(args), _lib.stream_ptr())
    _lib.check(rc, "rb_gemm")
    return out
