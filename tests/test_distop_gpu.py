"""Tensor-partitioned linear: all-gather -> GEMM and GEMM -> reduce-scatter kernels.  On one device the ranks
of the group are emulated inside one kernel launch (every shard lives on this GPU), which exercises the same
code: shard copies into the local buffer, readiness counters, rotated k order, scattered reductions."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, tol=2e-2):
    err = (a.float() - b.float()).abs().max().item()
    scale = b.float().abs().max().item() + 1e-6
    assert err / scale < tol, f"rel err {err / scale:.4g}"


@pytest.mark.parametrize("n", [2, 4])
@pytest.mark.parametrize("M,N,K", [(512, 768, 1024), (1000, 256, 2048)])
def test_linear_dist_emulated_group(n, M, N, K):
    from rannc_b200.ops import _lib
    from rannc_b200.parallel.distop import DistGroup, linear_dist

    torch.manual_seed(0)
    dev = torch.device("cuda")
    W = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
    b = torch.randn(N, device=dev).bfloat16()
    x = torch.randn(M, K, device=dev).bfloat16().requires_grad_(True)
    ks = K // n
    shards = [W[:, r * ks:(r + 1) * ks].contiguous() for r in range(n)]
    grads = [torch.zeros(N, ks, device=dev, dtype=torch.float32) for _ in range(n)]
    grp = DistGroup(list(range(n)), N * K, torch.bfloat16, dev, local=True)
    for my in range(n):  # the view of each emulated rank: same result, different rotation
        grp.my_idx = my
        w = shards[my].clone().requires_grad_(True)
        y = linear_dist(x, w, b, grp, [s.data_ptr() for s in shards], [g.data_ptr() for g in grads])
        ref = x.float() @ W.float().t() + b.float()
        _close(y, ref)
        dy = torch.randn_like(y)
        for g in grads:
            g.zero_()
        x.grad = None
        y.backward(dy)
        torch.cuda.synchronize()
        assert _lib.read_error() == 0
        _close(x.grad, dy.float() @ W.float())
        dW = dy.float().t() @ x.detach().float()
        for r in range(n):
            _close(grads[r], dW[:, r * ks:(r + 1) * ks])


def test_peer_wait_gives_up_and_context_survives():
    """Failure detection on the device without a fault: a flag that nothing sets; the bounded wait runs
    out, the kernel records status 2 and returns, and the context keeps working."""
    import ctypes

    from rannc_b200.ops import _lib

    flag = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert _lib.read_error() == 0
    rc = _lib.lib().rb_wait_flag_probe(ctypes.c_void_p(flag.data_ptr()), ctypes.c_uint(1), ctypes.c_ulonglong(2000),
                                       _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert _lib.read_error() == 2      # peer wait ran out
    assert _lib.read_error() == 0      # cleared
    y = torch.ones(8, device="cuda") * 3
    assert float(y.sum()) == 24.0      # the context is intact
