"""Thin ctypes wrappers over the C ABI of ``_kernels.so`` (everything but the GEMM).

Every function launches on the current CUDA stream and returns immediately.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint64, c_void_p

import torch

from . import _lib


def dt_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float16:
        return 0
    if t.dtype == torch.float32:
        return 2
    raise TypeError(f"unsupported dtype {t.dtype}")


# ------------------------------------------------------------------ layer norm
def ln_supported(H: int) -> bool:
    return bool(_lib.lib().rb_ln_supported(c_int(H)))


def ln_fwd(x, residual, gamma, beta, eps, p=0.0, seed=0, offset=0, need_z=True):
    """Returns (y, z, mean, rstd); z is x itself when there is neither residual nor dropout."""
    H = x.shape[-1]
    rows = x.numel() // H
    y = torch.empty_like(x)
    fused = residual is not None or p > 0.0
    z = torch.empty_like(x) if (fused and need_z) else None
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    rc = _lib.lib().rb_ln_fwd(_lib.vp(x), _lib.vp(residual), _lib.vp(gamma), _lib.vp(beta), _lib.vp(y),
                              _lib.vp(z), _lib.vp(mean), _lib.vp(rstd), c_int(rows), c_int(H),
                              c_float(eps), c_float(p), c_uint64(seed), c_uint64(offset),
                              c_int(dt_code(x)), _lib.stream_ptr())
    _lib.check(rc, "rb_ln_fwd")
    return y, (z if z is not None else x), mean, rstd


def ln_bwd(dy, z, gamma, mean, rstd, p=0.0, seed=0, offset=0, dgamma=None, dbeta=None, accumulate=False):
    """Returns (dz, dx, dgamma, dbeta); dx is dz when p == 0; dgamma/dbeta are fp32."""
    H = z.shape[-1]
    rows = z.numel() // H
    dz = torch.empty_like(z)
    dx = torch.empty_like(z) if p > 0.0 else None
    if dgamma is None:
        dgamma = torch.empty(H, dtype=torch.float32, device=z.device)
        dbeta = torch.empty(H, dtype=torch.float32, device=z.device)
        accumulate = False
    grid = _lib.lib().rb_ln_bwd_grid(c_int(rows))
    partial = torch.empty(grid * 2 * H, dtype=torch.float32, device=z.device)
    rc = _lib.lib().rb_ln_bwd(_lib.vp(dy), _lib.vp(z), _lib.vp(gamma), _lib.vp(mean), _lib.vp(rstd),
                              _lib.vp(dz), _lib.vp(dx), _lib.vp(dgamma), _lib.vp(dbeta), _lib.vp(partial),
                              c_int(rows), c_int(H), c_float(p), c_uint64(seed), c_uint64(offset),
                              c_int(1 if accumulate else 0), c_int(dt_code(z)), _lib.stream_ptr())
    _lib.check(rc, "rb_ln_bwd")
    return dz, (dx if dx is not None else dz), dgamma, dbeta


# ------------------------------------------------------------------ element-wise
def gelu(x):
    y = torch.empty_like(x)
    _lib.check(_lib.lib().rb_gelu(_lib.vp(x), c_void_p(0), _lib.vp(y), c_longlong(x.numel()), c_int(0),
                                  c_int(dt_code(x)), _lib.stream_ptr()), "rb_gelu")
    return y


def gelu_bwd(x, dy):
    y = torch.empty_like(x)
    _lib.check(_lib.lib().rb_gelu(_lib.vp(x), _lib.vp(dy), _lib.vp(y), c_longlong(x.numel()), c_int(1),
                                  c_int(dt_code(x)), _lib.stream_ptr()), "rb_gelu")
    return y


def dropout(x, p, seed, offset):
    y = torch.empty_like(x)
    _lib.check(_lib.lib().rb_dropout(_lib.vp(x), _lib.vp(y), c_longlong(x.numel()), c_float(p), c_uint64(seed),
                                     c_uint64(offset), c_int(dt_code(x)), _lib.stream_ptr()), "rb_dropout")
    return y


def colsum(x2d, out=None):
    """fp32 column sums of a [M, N] 16-bit matrix; adds into ``out`` when given."""
    M, N = x2d.shape
    if out is None:
        out = torch.zeros(N, dtype=torch.float32, device=x2d.device)
    _lib.check(_lib.lib().rb_colsum(_lib.vp(x2d), _lib.vp(out), c_int(M), c_int(N), c_longlong(x2d.stride(0)),
                                    c_int(dt_code(x2d)), _lib.stream_ptr()), "rb_colsum")
    return out


def accum_f32(dst, src, scale=1.0):
    _lib.check(_lib.lib().rb_accum_f32(_lib.vp(dst), _lib.vp(src), c_longlong(src.numel()), c_float(scale),
                                       c_int(dt_code(src)), _lib.stream_ptr()), "rb_accum_f32")


def cast_from_f32(dst, src, scale=1.0):
    _lib.check(_lib.lib().rb_cast_from_f32(_lib.vp(dst), _lib.vp(src), c_longlong(src.numel()), c_float(scale),
                                           c_int(dt_code(dst)), _lib.stream_ptr()), "rb_cast_from_f32")


def embed_fwd(ids, table):
    H = table.shape[1]
    out = torch.empty(*ids.shape, H, dtype=table.dtype, device=table.device)
    _lib.check(_lib.lib().rb_embed_fwd(_lib.vp(ids), _lib.vp(table), _lib.vp(out), c_int(ids.numel()), c_int(H),
                                       c_longlong(table.shape[0]), c_int(dt_code(table)), _lib.stream_ptr()),
               "rb_embed_fwd")
    return out


def embed_bwd(ids, dout, dtable_f32, padding_idx=-1):
    H = dout.shape[-1]
    _lib.check(_lib.lib().rb_embed_bwd(_lib.vp(ids), _lib.vp(dout), _lib.vp(dtable_f32), c_int(ids.numel()),
                                       c_int(H), c_longlong(dtable_f32.shape[0]), c_longlong(padding_idx),
                                       c_int(dt_code(dout)), _lib.stream_ptr()), "rb_embed_bwd")


def rowcopy(src, dst, rows, bytes_per_row, src_stride, dst_stride):
    _lib.check(_lib.lib().rb_rowcopy(_lib.vp(src), _lib.vp(dst), c_longlong(rows), c_longlong(bytes_per_row),
                                     c_longlong(src_stride), c_longlong(dst_stride), _lib.stream_ptr()),
               "rb_rowcopy")


# ------------------------------------------------------------------ loss
def xent_fwd(logits2d, labels, V, ignore_index=-100, weight=1.0):
    rows = logits2d.shape[0]
    lse = torch.empty(rows, dtype=torch.float32, device=logits2d.device)
    acc = torch.zeros(2, dtype=torch.float32, device=logits2d.device)
    loss = torch.empty((), dtype=torch.float32, device=logits2d.device)
    _lib.check(_lib.lib().rb_xent_fwd(_lib.vp(logits2d), _lib.vp(labels), _lib.vp(lse), _lib.vp(acc), _lib.vp(loss),
                                      c_int(rows), c_int(V), c_longlong(logits2d.stride(0)),
                                      c_longlong(ignore_index), c_float(weight), c_int(dt_code(logits2d)),
                                      _lib.stream_ptr()), "rb_xent_fwd")
    return loss, lse, acc


def xent_bwd(logits2d, labels, lse, acc, gout, V, ignore_index=-100, weight=1.0, inplace=True):
    d = logits2d if inplace else torch.empty_like(logits2d)
    _lib.check(_lib.lib().rb_xent_bwd(_lib.vp(logits2d), _lib.vp(labels), _lib.vp(lse), _lib.vp(acc), _lib.vp(gout),
                                      _lib.vp(d), c_int(logits2d.shape[0]), c_int(V),
                                      c_longlong(logits2d.stride(0)), c_longlong(ignore_index), c_float(weight),
                                      c_int(dt_code(logits2d)), _lib.stream_ptr()), "rb_xent_bwd")
    return d


# ------------------------------------------------------------------ optimizer
def adam_flat(master, grad, m, v, model16, lr, beta1, beta2, eps, weight_decay, step, adamw, ctrl=None):
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    _lib.check(_lib.lib().rb_adam_flat(_lib.vp(master), _lib.vp(grad), _lib.vp(m), _lib.vp(v), _lib.vp(model16),
                                       c_longlong(master.numel()), c_float(lr), c_float(beta1), c_float(beta2),
                                       c_float(eps), c_float(weight_decay), c_float(bc1), c_float(bc2),
                                       c_int(1 if adamw else 0), _lib.vp(ctrl),
                                       c_int(dt_code(model16) if model16 is not None else 1),
                                       _lib.stream_ptr()), "rb_adam_flat")


def sgd_flat(master, grad, mom, model16, lr, momentum, dampening, weight_decay, nesterov, first_step, ctrl=None):
    _lib.check(_lib.lib().rb_sgd_flat(_lib.vp(master), _lib.vp(grad), _lib.vp(mom), _lib.vp(model16),
                                      c_longlong(master.numel()), c_float(lr), c_float(momentum),
                                      c_float(dampening), c_float(weight_decay), c_int(1 if nesterov else 0),
                                      c_int(1 if first_step else 0), _lib.vp(ctrl),
                                      c_int(dt_code(model16) if model16 is not None else 1),
                                      _lib.stream_ptr()), "rb_sgd_flat")


def sumsq(x, out):
    _lib.check(_lib.lib().rb_sumsq(_lib.vp(x), c_longlong(x.numel()), _lib.vp(out), c_int(dt_code(x)),
                                   _lib.stream_ptr()), "rb_sumsq")


def finalize_ctrl(sumsq_t, inv_scale, max_norm, ctrl, norm_out=None):
    _lib.check(_lib.lib().rb_finalize_ctrl(_lib.vp(sumsq_t), c_float(inv_scale), c_float(max_norm), _lib.vp(ctrl),
                                           _lib.vp(norm_out), _lib.stream_ptr()), "rb_finalize_ctrl")


def scale_(x, s):
    _lib.check(_lib.lib().rb_scale(_lib.vp(x), c_longlong(x.numel()), c_float(s), c_int(dt_code(x)),
                                   _lib.stream_ptr()), "rb_scale")


# ------------------------------------------------------------------ attention
class _AttnArgs(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in ("Q", "K", "V", "O", "lse", "key_bias", "dO", "dQ", "dK", "dV", "delta",
                                        "dq_accum")] + \
               [(f"{t}_{s}", ctypes.c_int64) for t in ("q", "k", "v", "o", "do", "dq", "dk", "dv")
                for s in ("sb", "ss", "sh")] + \
               [("B", ctypes.c_int32), ("H", ctypes.c_int32), ("S", ctypes.c_int32), ("D", ctypes.c_int32),
                ("dtype", ctypes.c_int32), ("pad_", ctypes.c_int32), ("scale", c_float), ("p_drop", c_float),
                ("seed", c_uint64), ("offset", c_uint64)]


def _bshd_strides(t):
    """t is [B, S, H, D] with D contiguous; returns (sb, ss, sh)."""
    if t.stride(3) != 1:
        raise ValueError("attention operands need a contiguous head dimension")
    return t.stride(0), t.stride(1), t.stride(2)


def _attn_ok(t):
    return (t.data_ptr() % 16 == 0) and all(s % 8 == 0 for s in t.stride()[:3])


def attn_fwd(q, k, v, key_bias=None, scale=None, p_drop=0.0, seed=0, offset=0):
    """q, k, v: [B, S, H, 64] views (any strides with D contiguous).  Returns (o [B,S,H,64], lse [B,H,S])."""
    B, S, H, D = q.shape
    scale = float(scale if scale is not None else D ** -0.5)
    o = torch.empty(B, S, H, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
    a = _AttnArgs()
    a.Q, a.K, a.V, a.O, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr()
    a.key_bias = None if key_bias is None else key_bias.data_ptr()
    a.q_sb, a.q_ss, a.q_sh = _bshd_strides(q)
    a.k_sb, a.k_ss, a.k_sh = _bshd_strides(k)
    a.v_sb, a.v_ss, a.v_sh = _bshd_strides(v)
    a.o_sb, a.o_ss, a.o_sh = _bshd_strides(o)
    a.B, a.H, a.S, a.D, a.dtype = B, H, S, D, dt_code(q)
    a.scale, a.p_drop, a.seed, a.offset = scale, float(p_drop), int(seed), int(offset)
    _lib.check(_lib.lib().rb_attn_fwd(ctypes.byref(a), _lib.stream_ptr()), "rb_attn_fwd")
    return o, lse


def attn_bwd(q, k, v, o, lse, do, key_bias=None, scale=None, p_drop=0.0, seed=0, offset=0, dq=None, dk=None,
             dv=None):
    B, S, H, D = q.shape
    scale = float(scale if scale is not None else D ** -0.5)
    if do.stride(3) != 1 or not _attn_ok(do):
        do = do.contiguous()
    dq = torch.empty(B, S, H, D, dtype=q.dtype, device=q.device) if dq is None else dq
    dk = torch.empty(B, S, H, D, dtype=q.dtype, device=q.device) if dk is None else dk
    dv = torch.empty(B, S, H, D, dtype=q.dtype, device=q.device) if dv is None else dv
    delta = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
    dq_acc = torch.empty(B, S, H, D, dtype=torch.float32, device=q.device)
    a = _AttnArgs()
    a.Q, a.K, a.V, a.O, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr()
    a.key_bias = None if key_bias is None else key_bias.data_ptr()
    a.dO, a.dQ, a.dK, a.dV = do.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.delta, a.dq_accum = delta.data_ptr(), dq_acc.data_ptr()
    a.q_sb, a.q_ss, a.q_sh = _bshd_strides(q)
    a.k_sb, a.k_ss, a.k_sh = _bshd_strides(k)
    a.v_sb, a.v_ss, a.v_sh = _bshd_strides(v)
    a.o_sb, a.o_ss, a.o_sh = _bshd_strides(o)
    a.do_sb, a.do_ss, a.do_sh = _bshd_strides(do)
    a.dq_sb, a.dq_ss, a.dq_sh = _bshd_strides(dq)
    a.dk_sb, a.dk_ss, a.dk_sh = _bshd_strides(dk)
    a.dv_sb, a.dv_ss, a.dv_sh = _bshd_strides(dv)
    a.B, a.H, a.S, a.D, a.dtype = B, H, S, D, dt_code(q)
    a.scale, a.p_drop, a.seed, a.offset = scale, float(p_drop), int(seed), int(offset)
    _lib.check(_lib.lib().rb_attn_bwd(ctypes.byref(a), _lib.stream_ptr()), "rb_attn_bwd")
    return dq, dk, dv


# ------------------------------------------------------------------ convolution support, batch norm (NHWC)
def conv_out_size(H: int, k: int, s: int, pad: int) -> int:
    return (H + 2 * pad - k) // s + 1


def im2col(x_nhwc, k: int, s: int, pad: int):
    """[N, H, W, C] (contiguous) -> [N * Ho * Wo, k * k * C], taps outermost within a row."""
    N, H, W, C = x_nhwc.shape
    Ho, Wo = conv_out_size(H, k, s, pad), conv_out_size(W, k, s, pad)
    cols = torch.empty(N * Ho * Wo, k * k * C, dtype=x_nhwc.dtype, device=x_nhwc.device)
    _lib.check(_lib.lib().rb_im2col(_lib.vp(x_nhwc), _lib.vp(cols), c_int(N), c_int(H), c_int(W), c_int(C), c_int(k),
                                    c_int(s), c_int(pad), c_int(dt_code(x_nhwc)), _lib.stream_ptr()), "rb_im2col")
    return cols


def col2im(dcols, N: int, H: int, W: int, C: int, k: int, s: int, pad: int):
    """Adjoint of ``im2col``: [N * Ho * Wo, k * k * C] -> [N, H, W, C]."""
    dx = torch.empty(N, H, W, C, dtype=dcols.dtype, device=dcols.device)
    _lib.check(_lib.lib().rb_col2im(_lib.vp(dcols), _lib.vp(dx), c_int(N), c_int(H), c_int(W), c_int(C), c_int(k),
                                    c_int(s), c_int(pad), c_int(dt_code(dcols)), _lib.stream_ptr()), "rb_col2im")
    return dx


def bn_fwd(x2d, residual2d, gamma32, beta32, run_mean32, run_var32, eps: float, momentum: float, relu: bool):
    """Training-mode batch norm over the rows of [R, C] (+ residual, + ReLU).  Returns (y, mean, rstd);
    the running statistics (fp32, may be None) are updated in place."""
    R, C = x2d.shape
    y = torch.empty_like(x2d)
    part = torch.empty(2, C, dtype=torch.float32, device=x2d.device)
    mean = torch.empty(C, dtype=torch.float32, device=x2d.device)
    rstd = torch.empty(C, dtype=torch.float32, device=x2d.device)
    _lib.check(_lib.lib().rb_bn_fwd(_lib.vp(x2d), _lib.vp(residual2d), _lib.vp(gamma32), _lib.vp(beta32), _lib.vp(y),
                                    _lib.vp(part), _lib.vp(mean), _lib.vp(rstd), _lib.vp(run_mean32),
                                    _lib.vp(run_var32), c_longlong(R), c_int(C), c_float(eps), c_float(momentum),
                                    c_int(1 if relu else 0), c_int(dt_code(x2d)), _lib.stream_ptr()), "rb_bn_fwd")
    return y, mean, rstd


def bn_bwd(x2d, dy2d, y2d, mean, rstd, gamma32, relu: bool, want_dres: bool):
    """Returns (dx, dres or None, dgamma fp32, dbeta fp32)."""
    R, C = x2d.shape
    dx = torch.empty_like(x2d)
    dres = torch.empty_like(x2d) if want_dres else None
    part = torch.empty(5, C, dtype=torch.float32, device=x2d.device)   # two sums + three coefficient rows
    _lib.check(_lib.lib().rb_bn_bwd(_lib.vp(x2d), _lib.vp(dy2d), _lib.vp(y2d), _lib.vp(mean), _lib.vp(rstd),
                                    _lib.vp(gamma32), _lib.vp(part), _lib.vp(dx), _lib.vp(dres), c_longlong(R),
                                    c_int(C), c_int(1 if relu else 0), c_int(dt_code(x2d)), _lib.stream_ptr()),
               "rb_bn_bwd")
    return dx, dres, part[1], part[0]
