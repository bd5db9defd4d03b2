"""Memory-bound and attention kernels against plain fp32 PyTorch references."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _close(a, b, tol):
    err = (a.float() - b.float()).abs().max().item()
    scale = b.float().abs().max().item() + 1e-6
    assert err / scale < tol, f"rel err {err / scale:.4g} (abs {err:.4g})"


@pytest.mark.parametrize("H", [256, 768, 1024, 2048, 4096])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_layernorm_fwd_bwd(H, dtype):
    from rannc_b200.ops import kernels as K

    torch.manual_seed(0)
    rows = 517
    x = torch.randn(rows, H, device="cuda", dtype=dtype)
    res = torch.randn(rows, H, device="cuda", dtype=dtype)
    g = (torch.randn(H, device="cuda") * 0.1 + 1).to(dtype)
    b = (torch.randn(H, device="cuda") * 0.1).to(dtype)
    y, z, mean, rstd = K.ln_fwd(x, res, g, b, 1e-5)
    zr = (x.float() + res.float()).to(dtype).float().requires_grad_(True)
    yr = F.layer_norm(zr, (H,), g.float(), b.float(), 1e-5)
    _close(z, zr, 1e-2)
    _close(y, yr, 2e-2)
    dy = torch.randn(rows, H, device="cuda", dtype=dtype)
    dz, dx, dg, db = K.ln_bwd(dy, z, g, mean, rstd)
    gg = g.float().requires_grad_(True)
    bb = b.float().requires_grad_(True)
    yr = F.layer_norm(zr, (H,), gg, bb, 1e-5)
    yr.backward(dy.float())
    _close(dz, zr.grad, 2e-2)
    _close(dg, gg.grad, 2e-2)
    _close(db, bb.grad, 2e-2)
    assert dx is dz


def test_layernorm_dropout_consistency():
    from rannc_b200.ops import kernels as K

    torch.manual_seed(0)
    rows, H, p = 300, 1024, 0.25
    x = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16)
    res = torch.zeros(rows, H, device="cuda", dtype=torch.bfloat16)
    g = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(H, device="cuda", dtype=torch.bfloat16)
    y, z, mean, rstd = K.ln_fwd(x, res, g, b, 1e-5, p=p, seed=7, offset=3)
    # z is dropout(x): same mask as the standalone kernel with the same counter
    d = K.dropout(x, p, 7, 3)
    assert torch.equal(z, d)
    keep = (z != 0).float().mean().item()
    assert abs(keep - (1 - p)) < 0.01
    nz = z != 0
    _close(z[nz], x[nz].float() / (1 - p), 1e-2)
    # backward regenerates the mask
    dy = torch.randn_like(x)
    dz, dx, _, _ = K.ln_bwd(dy, z, g, mean, rstd, p=p, seed=7, offset=3)
    ref = torch.where(nz, dz.float() / (1 - p), torch.zeros_like(dz.float()))
    _close(dx, ref, 1e-2)
    # a different offset gives a different mask
    d2 = K.dropout(x, p, 7, 4)
    assert not torch.equal(d, d2)


def test_gelu_colsum_embed():
    from rannc_b200.ops import kernels as K

    torch.manual_seed(0)
    x = torch.randn(1000, 333, device="cuda", dtype=torch.bfloat16)
    _close(K.gelu(x), F.gelu(x.float()), 1e-2)
    dy = torch.randn_like(x)
    xr = x.float().requires_grad_(True)
    F.gelu(xr).backward(dy.float())
    _close(K.gelu_bwd(x, dy), xr.grad, 2e-2)
    _close(K.colsum(x), x.float().sum(0), 1e-2)
    table = torch.randn(1000, 256, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, 1000, (7, 31), device="cuda")
    out = K.embed_fwd(ids, table)
    assert torch.equal(out, table[ids])
    dt = torch.zeros(1000, 256, device="cuda", dtype=torch.float32)
    dout = torch.randn(7, 31, 256, device="cuda", dtype=torch.bfloat16)
    K.embed_bwd(ids, dout, dt)
    ref = torch.zeros_like(dt).index_add_(0, ids.flatten(), dout.float().view(-1, 256))
    _close(dt, ref, 1e-3)


@pytest.mark.parametrize("V,ld", [(30522, 30528), (1000, 1000), (77, 80)])
def test_xent(V, ld):
    from rannc_b200.ops import kernels as K

    torch.manual_seed(0)
    rows = 257
    buf = torch.randn(rows, ld, device="cuda", dtype=torch.bfloat16) * 3
    logits = buf[:, :ld]
    labels = torch.randint(0, V, (rows,), device="cuda")
    labels[torch.rand(rows, device="cuda") < 0.7] = -100
    lr = logits[:, :V].float().requires_grad_(True)
    ref = F.cross_entropy(lr, labels, ignore_index=-100)
    loss, lse, acc = K.xent_fwd(logits, labels, V)
    _close(loss, ref, 1e-3)
    ref.backward()
    gout = torch.ones((), device="cuda", dtype=torch.float32)
    d = K.xent_bwd(logits, labels, lse, acc, gout, V, inplace=False)
    _close(d[:, :V], lr.grad, 2e-2)
    assert (d[:, V:] == 0).all()


def test_adam_and_norm():
    from rannc_b200.ops import kernels as K

    torch.manual_seed(0)
    n = 100003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    ref_p = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref_p], lr=1e-2, weight_decay=0.01)
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    for step in range(1, 4):
        ref_p.grad = g.clone()
        opt.step()
        K.adam_flat(p, g, m, v, p16, 1e-2, 0.9, 0.999, 1e-8, 0.01, step, True)
    _close(p, ref_p.detach(), 1e-4)
    _close(p16, ref_p.detach(), 1e-2)
    ss = torch.zeros(1, device="cuda")
    K.sumsq(g, ss)
    _close(ss, (g.double() ** 2).sum().float(), 1e-4)
    ctrl = torch.zeros(2, device="cuda")
    norm = torch.zeros(1, device="cuda")
    K.finalize_ctrl(ss, 0.5, 1.0, ctrl, norm)
    nref = g.norm().item() * 0.5
    assert abs(norm.item() - nref) / nref < 1e-3
    assert abs(ctrl[0].item() - 0.5 / nref) / (0.5 / nref) < 1e-2 and ctrl[1].item() == 0
    g[5] = float("inf")
    ss.zero_()
    K.sumsq(g, ss)
    K.finalize_ctrl(ss, 0.5, 1.0, ctrl, norm)
    assert ctrl[1].item() == 1
    before = p.clone()
    K.adam_flat(p, g, m, v, p16, 1e-2, 0.9, 0.999, 1e-8, 0.01, 4, True, ctrl)
    assert torch.equal(before, p)  # overflow: step skipped


def _attn_ref(q, k, v, bias, scale):
    # q,k,v [B,S,H,D] fp32
    s = torch.einsum("bqhd,bkhd->bhqk", q, k) * scale
    if bias is not None:
        s = s + bias[:, None, None, :]
    p = s.softmax(-1)
    return torch.einsum("bhqk,bkhd->bqhd", p, v)


@pytest.mark.parametrize("B,S,H", [(2, 512, 4), (1, 128, 2), (2, 200, 3), (1, 384, 1)])
@pytest.mark.parametrize("use_bias", [False, True])
def test_attention_fwd_bwd(B, S, H, use_bias):
    from rannc_b200.ops import _lib
    from rannc_b200.ops import kernels as K

    torch.manual_seed(0)
    D = 64
    qkv = torch.randn(B, S, 3, H, D, device="cuda", dtype=torch.bfloat16)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    bias = None
    if use_bias:
        bias = torch.zeros(B, S, device="cuda", dtype=torch.float32)
        bias[:, S - S // 4:] = -10000.0
    o, lse = K.attn_fwd(q, k, v, key_bias=bias)
    torch.cuda.synchronize()
    assert _lib.read_error() == 0
    qr, kr, vr = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    ref = _attn_ref(qr, kr, vr, bias, D ** -0.5)
    _close(o, ref, 2e-2)
    do = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16)
    dq, dk, dv = K.attn_bwd(q, k, v, o, lse, do, key_bias=bias)
    torch.cuda.synchronize()
    assert _lib.read_error() == 0
    ref.backward(do.float())
    _close(dv, vr.grad, 3e-2)
    _close(dk, kr.grad, 3e-2)
    _close(dq, qr.grad, 3e-2)


@pytest.mark.parametrize("use_bias", [False, True])
def test_attention_dropout_forward_backward_consistency(use_bias):
    """The backward regenerates the forward's dropout mask.  The mask depends on (seed, b, h, q, key) only,
    so it can be read out with uniform attention over one-hot values, and then used in an fp32 reference."""
    from rannc_b200.ops import _lib
    from rannc_b200.ops import kernels as K

    torch.manual_seed(1)
    B, S, H, D, pd = 2, 64, 3, 64, 0.25
    z = torch.zeros(B, S, H, D, device="cuda", dtype=torch.bfloat16)
    eye = torch.eye(S, device="cuda", dtype=torch.bfloat16)[None, :, None, :].expand(B, S, H, D).contiguous()
    o, _ = K.attn_fwd(z, z, eye, p_drop=pd, seed=21, offset=2)
    mask = (o.float() > 0).permute(0, 2, 1, 3).float()          # [B, H, q, key]
    assert abs(mask.mean().item() - (1 - pd)) < 0.03
    qkv = torch.randn(B, S, 3, H, D, device="cuda", dtype=torch.bfloat16)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    bias = None
    if use_bias:
        bias = torch.zeros(B, S, device="cuda", dtype=torch.float32)
        bias[:, S - 9:] = -10000.0
    o, lse = K.attn_fwd(q, k, v, key_bias=bias, p_drop=pd, seed=21, offset=2)
    qr, kr, vr = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    sc = torch.einsum("bqhd,bkhd->bhqk", qr, kr) * D ** -0.5
    if bias is not None:
        sc = sc + bias[:, None, None, :]
    a = sc.softmax(-1) * mask / (1 - pd)
    ref = torch.einsum("bhqk,bkhd->bqhd", a, vr)
    _close(o, ref, 2e-2)
    do = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16)
    dq, dk, dv = K.attn_bwd(q, k, v, o, lse, do, key_bias=bias, p_drop=pd, seed=21, offset=2)
    torch.cuda.synchronize()
    assert _lib.read_error() == 0
    ref.backward(do.float())
    _close(dv, vr.grad, 3e-2)
    _close(dk, kr.grad, 3e-2)
    _close(dq, qr.grad, 3e-2)


def test_attention_dropout_statistics():
    from rannc_b200.ops import kernels as K

    torch.manual_seed(0)
    B, S, H, D = 1, 256, 2, 64
    q = torch.zeros(B, S, H, D, device="cuda", dtype=torch.bfloat16)
    k = torch.zeros(B, S, H, D, device="cuda", dtype=torch.bfloat16)
    v = torch.ones(B, S, H, D, device="cuda", dtype=torch.bfloat16)
    # uniform attention over ones: each output = (kept fraction) / (1 - p)
    o, _ = K.attn_fwd(q, k, v, p_drop=0.5, seed=11, offset=1)
    mean = o.float().mean().item()
    assert abs(mean - 1.0) < 0.02
    assert o.float().std().item() > 0.01
    o2, _ = K.attn_fwd(q, k, v, p_drop=0.5, seed=11, offset=1)
    assert torch.equal(o, o2)
    # keep decisions of neighbouring rows / keys are uncorrelated, and another offset gives another mask
    vv = torch.eye(64, device="cuda", dtype=torch.bfloat16)[None, :, None, :].expand(1, 64, 2, 64).contiguous()
    zz = torch.zeros(1, 64, 2, 64, device="cuda", dtype=torch.bfloat16)
    m1 = (K.attn_fwd(zz, zz, vv, p_drop=0.5, seed=11, offset=1)[0].float() > 0).float()   # [1, q, h, key]
    m2 = (K.attn_fwd(zz, zz, vv, p_drop=0.5, seed=11, offset=2)[0].float() > 0).float()
    c = lambda a, b: ((a - a.mean()) * (b - b.mean())).mean().item() / 0.25  # noqa: E731
    assert abs(c(m1[:, :-1], m1[:, 1:])) < 0.06 and abs(c(m1[..., :-1], m1[..., 1:])) < 0.06
    assert abs(c(m1[:, :, 0], m1[:, :, 1])) < 0.06 and abs(c(m1, m2)) < 0.06
