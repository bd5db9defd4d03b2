"""Host side of the implicit-GEMM convolution, checked without a GPU.

``ops.functional._Conv2d`` describes a stride-1 "same" convolution to the GEMM kernel as row shifts per filter tap
over the zero-padded channels-last activation, a padded-grid-to-output row map, and tap blocks of the weight matrix.
Here the GEMM is replaced by a plain PyTorch function that follows the kernel's documented addressing rules (rows
outside the matrix read as zero, tap t's block of a [K, N] operand starts ``b_tap_cols * t`` columns further right,
``b_row_shift`` shifts the rows of the [K, N] operand, only interior rows of the padded grid are stored), and the
Function's forward, input gradient and weight gradient are compared with ``torch.nn.functional.conv2d``."""
import pytest
import torch

from rannc_b200.ops import functional as RF
from rannc_b200.utils.config import set_conf


def _shifted_rows(m: torch.Tensor, shift: int) -> torch.Tensor:
    """out[i] = m[i + shift], zero where i + shift falls outside m (the TMA fill of an out-of-range box)."""
    rows = m.shape[0]
    out = torch.zeros_like(m)
    lo, hi = max(0, -shift), min(rows, rows - shift)
    if hi > lo:
        out[lo:hi] = m[lo + shift:hi + shift]
    return out


def _gemm_by_the_rules(a, b, *, trans_a=False, trans_b=True, bias=None, out=None, accumulate=False, out_dtype=None,
                       conv=None, b_row_shift=0, row_map=None, **_):
    a32, b32 = a.float(), b.float()
    if conv is not None:
        taps, chans = conv["taps"], a.shape[1]
        lhs = torch.cat([_shifted_rows(a32, conv["shifts"][t]) for t in range(taps)], 1)      # [rows, taps * C]
        if trans_b:
            rhs = b32.t()
        else:
            n, step = conv["n"], conv["b_tap_cols"]
            assert b32.shape[0] == chans
            rhs = torch.cat([b32[:, t * step:t * step + n] for t in range(taps)], 0)          # [taps * C, n]
        res = lhs @ rhs
    else:
        lhs = a32.t() if trans_a else a32
        rhs = b32.t() if trans_b else (_shifted_rows(b32, b_row_shift) if b_row_shift else b32)
        res = lhs @ rhs
    if bias is not None:
        res = res + bias.float()
    if row_map is not None:
        hp, wp, h, w, pad = row_map
        n_img = res.shape[0] // (hp * wp)
        res = res.view(n_img, hp, wp, -1)[:, pad:pad + h, pad:pad + w].reshape(n_img * h * w, -1)
    odt = out_dtype or (out.dtype if out is not None else a.dtype)
    if out is None:
        return res.to(odt)
    if accumulate:
        out.add_(res.to(out.dtype))
    else:
        out.copy_(res.to(out.dtype))
    return out


@pytest.mark.parametrize("N,C,Co,H,W,k", [(2, 64, 128, 5, 7, 3), (1, 64, 64, 4, 4, 5), (3, 128, 64, 6, 3, 3)])
def test_tap_shifts_row_map_and_weight_blocks_reproduce_conv2d(monkeypatch, N, C, Co, H, W, k):
    monkeypatch.setattr(RF, "gemm", _gemm_by_the_rules)
    monkeypatch.setattr(RF.K, "conv_out_size", lambda size, kk, s, p: (size + 2 * p - kk) // s + 1)
    monkeypatch.setattr(RF.K, "colsum", lambda d, out=None: d.float().sum(0) if out is None
                        else out.add_(d.float().sum(0)))
    set_conf("conv_implicit_gemm", True)
    set_conf("conv_implicit_max_overhead", 100.0)
    try:
        torch.manual_seed(0)
        pad = (k - 1) // 2
        assert RF._Conv2d._implicit(k, 1, pad, C, Co, H, W)
        x = torch.randn(N, C, H, W, requires_grad=True)
        w = torch.randn(Co, C, k, k, requires_grad=True)
        b = torch.randn(Co, requires_grad=True)
        y = RF._Conv2d.apply(x, w, b, 1, pad)
        ref = torch.nn.functional.conv2d(x, w, b, 1, pad)
        go = torch.randn_like(ref)
        gx, gw, gb = torch.autograd.grad(y, (x, w, b), go)
        rx, rw, rb = torch.autograd.grad(ref, (x, w, b), go)
        for got, want in ((y, ref), (gx, rx), (gw, rw), (gb, rb)):
            assert torch.allclose(got, want, rtol=1e-4, atol=1e-4 * float(want.abs().max()))
    finally:
        set_conf("conv_implicit_gemm", True)
        set_conf("conv_implicit_max_overhead", 1.2)


def test_small_feature_maps_keep_the_gathered_matrix():
    set_conf("conv_implicit_gemm", True)
    set_conf("conv_implicit_max_overhead", 1.2)
    assert RF._Conv2d._implicit(3, 1, 1, 256, 256, 56, 56)
    assert RF._Conv2d._implicit(3, 1, 1, 256, 256, 28, 28)
    assert not RF._Conv2d._implicit(3, 1, 1, 256, 256, 14, 14)      # 31 % more positions than outputs
    assert not RF._Conv2d._implicit(3, 2, 1, 256, 256, 56, 56)      # strided
    assert not RF._Conv2d._implicit(3, 1, 1, 24, 256, 56, 56)       # channels not a multiple of the k step
