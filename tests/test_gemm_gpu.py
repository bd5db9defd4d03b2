"""tcgen05 GEMM against an fp32 PyTorch reference of the same product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, trans_a, trans_b):
    a32, b32 = a.float(), b.float()
    if trans_a:
        a32 = a32.transpose(-1, -2)
    if trans_b:
        b32 = b32.transpose(-1, -2)
    return a32 @ b32


def _check(out, ref, tol=2e-2, elementwise=True):
    """Two criteria.  The largest error relative to the largest reference value (catches a wrong tile), and --
    for outputs that were rounded once to 16 bits from an fp32 accumulator -- every element on its own:
    |err| <= atol + rtol * |ref| with atol a tenth of the first criterion's, so that an error confined to
    small-magnitude outputs does not hide behind the large ones."""
    d = (out.float() - ref).abs()
    scale = ref.abs().max().item() + 1e-6
    assert d.max().item() / scale < tol, f"rel err {d.max().item() / scale}"
    if elementwise:
        bound = 0.1 * tol * scale + tol * ref.abs()
        bad = d > bound
        assert not bad.any(), f"{int(bad.sum())} element(s) outside atol + rtol|ref|, worst {float((d - bound).max())}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 264, 136), (1024, 1024, 1024), (129, 40, 72)])
def test_gemm_layouts(dtype, trans_a, trans_b, M, N, K):
    from rannc_b200.ops import _lib
    from rannc_b200.ops.gemm import gemm

    torch.manual_seed(0)
    a = torch.randn((K, M) if trans_a else (M, K), device="cuda", dtype=dtype)
    b = torch.randn((N, K) if trans_b else (K, N), device="cuda", dtype=dtype)
    out = gemm(a, b, trans_a=trans_a, trans_b=trans_b)
    torch.cuda.synchronize()
    assert _lib.read_error() == 0
    _check(out, _ref(a, b, trans_a, trans_b))


def test_gemm_epilogues():
    from rannc_b200.ops.gemm import gemm

    torch.manual_seed(1)
    M, N, K = 512, 768, 320
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    pre = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    out = gemm(x, w, bias=bias, gelu=True, aux_out=pre)
    z = x.float() @ w.float().t() + bias.float()
    _check(pre, z)
    _check(out, torch.nn.functional.gelu(z))
    out = gemm(x, w, bias=bias, residual=res)
    _check(out, z + res.float())
    # dgelu: v * gelu'(aux)
    zz = z.clone().requires_grad_(True)
    torch.nn.functional.gelu(zz).sum().backward()
    out = gemm(x, w, dgelu=True, aux_in=pre)
    _check(out, (x.float() @ w.float().t()) * zz.grad, tol=3e-2)
    # fp32 output with accumulation
    acc = torch.ones(M, N, device="cuda", dtype=torch.float32)
    gemm(x, w, out=acc, accumulate=True, alpha=0.5)
    _check(acc, 0.5 * (x.float() @ w.float().t()) + 1.0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(4096, 4096, 256), (4360, 2120, 328), (2304, 2048, 1024)])
def test_gemm_pair_kernel_layouts(dtype, trans_a, trans_b, M, N, K):
    """Shapes with enough 256 x 256 tiles for the two-CTA kernel (both SMs of a TPC on one tile),
    including ragged edges where the second CTA's rows or columns run past the matrix."""
    from rannc_b200.ops import _lib
    from rannc_b200.ops.gemm import gemm

    torch.manual_seed(0)
    a = torch.randn((K, M) if trans_a else (M, K), device="cuda", dtype=dtype)
    b = torch.randn((N, K) if trans_b else (K, N), device="cuda", dtype=dtype)
    out = gemm(a, b, trans_a=trans_a, trans_b=trans_b)
    torch.cuda.synchronize()
    assert _lib.read_error() == 0
    _check(out, _ref(a, b, trans_a, trans_b))


def test_gemm_pair_kernel_epilogues():
    from rannc_b200.ops import _lib
    from rannc_b200.ops.gemm import gemm

    torch.manual_seed(1)
    M, N, K = 4232, 3080, 320
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    pre = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    out = gemm(x, w, bias=bias, gelu=True, aux_out=pre)
    z = x.float() @ w.float().t() + bias.float()
    _check(pre, z)
    _check(out, torch.nn.functional.gelu(z))
    out = gemm(x, w, bias=bias, residual=res)
    _check(out, z + res.float())
    out32 = gemm(x, w, out_dtype=torch.float32, alpha=0.5)
    _check(out32, 0.5 * (x.float() @ w.float().t()))
    # many tiles per cluster (both accumulator buffers and every ring stage wrap several times)
    out = gemm(x, w, max_ctas=8)
    _check(out, x.float() @ w.float().t())
    a3 = torch.randn(40, 512, 64, device="cuda", dtype=torch.bfloat16)
    b3 = torch.randn(40, 512, 64, device="cuda", dtype=torch.bfloat16)
    _check(gemm(a3, b3), a3.float() @ b3.float().transpose(1, 2))
    torch.cuda.synchronize()
    assert _lib.read_error() == 0


@pytest.mark.parametrize("M,N,K", [(1024, 1024, 8192), (3072, 1024, 4100), (1024, 4096, 2048), (384, 520, 16384)])
def test_gemm_wgrad_split_k_pair(M, N, K):
    """Weight-gradient shape: few output tiles, long K, fp32 accumulation into an existing buffer."""
    from rannc_b200.ops import _lib
    from rannc_b200.ops.gemm import gemm

    torch.manual_seed(3)
    dy = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    acc = torch.full((M, N), 2.0, device="cuda", dtype=torch.float32)
    gemm(dy, x, trans_a=True, trans_b=False, out=acc, accumulate=True)
    gemm(dy, x, trans_a=True, trans_b=False, out=acc, accumulate=True, alpha=0.5)
    torch.cuda.synchronize()
    assert _lib.read_error() == 0
    _check(acc, 1.5 * (dy.float().t() @ x.float()) + 2.0)


def test_gemm_batched():
    from rannc_b200.ops.gemm import gemm

    torch.manual_seed(2)
    a = torch.randn(6, 200, 64, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(6, 320, 64, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, b)
    _check(out, a.float() @ b.float().transpose(1, 2))
    c = torch.randn(6, 64, 136, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, c, trans_b=False)
    _check(out, a.float() @ c.float())


def test_gemm_large_perf_shape():
    from rannc_b200.ops.gemm import gemm

    torch.manual_seed(3)
    a = torch.randn(4096, 1024, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(4096, 1024, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, b)
    _check(out, a.float() @ b.float().t())
