"""Convolution (GEMM over channels-last activations) and batch-norm kernels against fp32 PyTorch."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _close(a, b, tol=2e-2):
    err = (a.float() - b.float()).abs().max().item()
    scale = b.float().abs().max().item() + 1e-6
    assert err / scale < tol, f"rel err {err / scale:.4g}"


@pytest.mark.parametrize("k,s,p", [(1, 1, 0), (1, 2, 0), (3, 1, 1), (3, 2, 1), (7, 2, 3)])
@pytest.mark.parametrize("bias", [False, True])
def test_conv2d_forward_backward(k, s, p, bias):
    from rannc_b200.ops import _lib
    from rannc_b200.ops import functional as RF

    torch.manual_seed(0)
    N, Ci, Co, H, W = 3, 16, 24, 14, 18
    x = torch.randn(N, Ci, H, W, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    w = (torch.randn(Co, Ci, k, k, device="cuda") * 0.1).bfloat16().requires_grad_(True)
    b = torch.randn(Co, device="cuda", dtype=torch.bfloat16).requires_grad_(True) if bias else None
    y = RF.conv2d(x, w, b, s, p)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    br = b.detach().float().requires_grad_(True) if bias else None
    ref = F.conv2d(xr, wr, br, s, p)
    assert y.shape == ref.shape
    _close(y, ref)
    dy = torch.randn_like(ref)
    y.backward(dy.to(y.dtype))
    ref.backward(dy.to(y.dtype).float())
    torch.cuda.synchronize()
    assert _lib.read_error() == 0
    _close(x.grad, xr.grad, 3e-2)
    _close(w.grad, wr.grad, 3e-2)
    if bias:
        _close(b.grad, br.grad, 3e-2)


def test_conv2d_accumulates_into_main_grad():
    from rannc_b200.ops import functional as RF

    torch.manual_seed(1)
    x = torch.randn(2, 32, 8, 8, device="cuda", dtype=torch.bfloat16)
    for k, p in ((1, 0), (3, 1)):
        w = (torch.randn(16, 32, k, k, device="cuda") * 0.1).bfloat16().requires_grad_(True)
        w.main_grad = torch.ones(16, 32, k, k, device="cuda")
        y = RF.conv2d(x, w, None, 1, p)
        dy = torch.randn_like(y)
        y.backward(dy)
        wr = w.detach().float().requires_grad_(True)
        F.conv2d(x.float(), wr, None, 1, p).backward(dy.float())
        assert w.grad is None
        _close(w.main_grad, wr.grad + 1.0, 3e-2)


@pytest.mark.parametrize("relu,res", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_batch_norm_act(relu, res, dtype):
    from rannc_b200.ops import functional as RF

    torch.manual_seed(2)
    N, C, H, W = 6, 64, 9, 7
    x = (torch.randn(N, C, H, W, device="cuda") * 2 + 0.5).to(dtype).requires_grad_(True)
    r = torch.randn(N, C, H, W, device="cuda").to(dtype).requires_grad_(True) if res else None
    g = (torch.rand(C, device="cuda") + 0.5).requires_grad_(True)
    b = torch.randn(C, device="cuda").requires_grad_(True)
    rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
    y = RF.batch_norm_act(x, g, b, rm, rv, True, 0.1, 1e-5, relu, r)
    xr = x.detach().float().requires_grad_(True)
    rr = r.detach().float().requires_grad_(True) if res else None
    gr, br = g.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    rmr, rvr = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
    ref = F.batch_norm(xr, rmr, rvr, gr, br, True, 0.1, 1e-5)
    if res:
        ref = ref + rr
    if relu:
        ref = torch.relu(ref)
    _close(y, ref)
    assert torch.allclose(rm, rmr, rtol=1e-2, atol=1e-3) and torch.allclose(rv, rvr, rtol=1e-2, atol=1e-3)
    dy = torch.randn_like(ref)
    y.backward(dy.to(dtype))
    ref.backward(dy.to(dtype).float())
    _close(x.grad, xr.grad, 3e-2)
    _close(g.grad, gr.grad, 3e-2)
    _close(b.grad, br.grad, 3e-2)
    if res:
        _close(r.grad, rr.grad, 3e-2)


def test_tiny_resnet_trains_through_the_engine():
    """Convolutions, batch norms with their buffers, pooling and the classifier through RaNNCModule with
    mixed precision; the loss must fall and the running statistics must move."""
    import rannc_b200 as pyrannc
    from rannc_b200.models.resnet import ResNetWithLoss, tiny_resnet

    torch.manual_seed(0)
    net = ResNetWithLoss(tiny_resnet())
    opt = torch.optim.SGD(net.parameters(), lr=0.05, momentum=0.9)
    model = pyrannc.RaNNCModule(net, opt, enable_apex_amp=True)
    x = torch.randn(16, 3, 64, 64, device="cuda")
    yl = torch.randint(0, 10, (16,), device="cuda")
    losses = []
    for _ in range(12):
        loss = model(x, yl)
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(float(loss))
    assert losses[-1] < 0.7 * losses[0], losses
    sd = model.state_dict()
    assert float(sd["net.bn1.num_batches_tracked"]) == 12
    assert sd["net.bn1.running_mean"].abs().sum() > 0
    stats = model._traced.rewrite_stats
    assert stats.get("conv2d", 0) >= 16 and stats.get("batch_norm_act", 0) >= 16
    pyrannc.clear()


@pytest.mark.parametrize("N,Ci,Co,H,W,k", [(4, 64, 128, 14, 14, 3), (2, 128, 64, 9, 7, 3), (2, 64, 64, 8, 8, 5),
                                           (3, 192, 320, 28, 28, 3)])
@pytest.mark.parametrize("main_grad", [False, True])
def test_conv2d_implicit_gemm_matches_fp32(N, Ci, Co, H, W, k, main_grad):
    """conv_implicit_gemm: stride-1 "same" convolutions read the zero-padded activation tap by tap inside the
    GEMM's producer (forward, input gradient) and with a row shift per tap (weight gradient): no im2col matrix."""
    from rannc_b200.ops import _lib
    from rannc_b200.ops import functional as RF
    from rannc_b200.utils.config import set_conf

    set_conf("conv_implicit_gemm", True)
    set_conf("conv_implicit_max_overhead", 10.0)
    try:
        torch.manual_seed(0)
        p = (k - 1) // 2
        assert RF._Conv2d._implicit(k, 1, p, Ci, Co, H, W)
        x = torch.randn(N, Ci, H, W, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
        w = (torch.randn(Co, Ci, k, k, device="cuda") * 0.05).bfloat16().requires_grad_(True)
        b = torch.randn(Co, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
        if main_grad:
            w.main_grad = torch.ones(Co, Ci, k, k, device="cuda")
        y = RF.conv2d(x, w, b, 1, p)
        xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
        br = b.detach().float().requires_grad_(True)
        ref = F.conv2d(xr, wr, br, 1, p)
        assert y.shape == ref.shape
        _close(y, ref)
        dy = torch.randn_like(ref)
        y.backward(dy.to(y.dtype))
        ref.backward(dy.to(y.dtype).float())
        torch.cuda.synchronize()
        assert _lib.read_error() == 0
        _close(x.grad, xr.grad, 3e-2)
        if main_grad:
            assert w.grad is None
            _close(w.main_grad, wr.grad + 1.0, 3e-2)
        else:
            _close(w.grad, wr.grad, 3e-2)
        _close(b.grad, br.grad, 3e-2)
    finally:
        set_conf("conv_implicit_gemm", False)
        set_conf("conv_implicit_max_overhead", 1.2)
