"""Micro-benchmarks of the sm_100a kernels (CUDA-event timing, L2 flushed between iterations).

    python -m rannc_b200.ops.bench_kernels gemm --m 16384 --n 4096 --k 1024 [--layout nt|nn|tn] [--acc]
    python -m rannc_b200.ops.bench_kernels attn --batch 8 --heads 16 --seq 512 [--dropout 0.1]
    python -m rannc_b200.ops.bench_kernels ln --rows 32768 --hidden 1024
    python -m rannc_b200.ops.bench_kernels adam --numel 100000000
    python -m rannc_b200.ops.bench_kernels ag_gemm --m 8192 --n 4096 --k 4096 --ranks 4
    python -m rannc_b200.ops.bench_kernels gemm_rs --m 8192 --n 4096 --k 4096 --ranks 4
    python -m rannc_b200.ops.bench_kernels rs_adam --numel 100000000
    python -m rannc_b200.ops.bench_kernels bn --batch 64 --channels 2048 --hw 28      # also bn_bwd, im2col

``ag_gemm`` / ``gemm_rs`` run the all-gather -> GEMM and GEMM -> reduce-scatter kernels with the group's
``--ranks`` shards all placed on this GPU (the peers' buffers are local allocations), ``rs_adam`` runs the
reduce-scatter + Adam + all-gather kernel for a rank set of one: the same kernels as over NVLink, without
the link.

Each prints one JSON line with the time per call and the achieved fraction of the measured peaks
(``MEASURED_PEAKS.json`` at the repository root when present, else 6.65 TB/s and 1.59 PFLOP/s).
``--iters`` small and ``--no-flush`` make the run suitable for a profiler capture.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


def _time(fn, iters, warmup, flush):
    buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(iters):
        if buf is not None:
            buf.zero_()  # 256 MiB > the 126 MB L2
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters * 1e-3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "attn", "attn_bwd", "ln", "ln_bwd", "adam", "xent", "colsum",
                                      "ag_gemm", "gemm_rs", "rs_adam", "bn", "bn_bwd", "im2col"])
    ap.add_argument("--channels", type=int, default=2048)
    ap.add_argument("--hw", type=int, default=28)
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--layout", default="nt", help="nt: forward, nn: dgrad, tn: wgrad")
    ap.add_argument("--acc", action="store_true", help="fp32 output with accumulation (wgrad epilogue)")
    ap.add_argument("--gelu", action="store_true")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--dropout", type=float, default=0.0)
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--numel", type=int, default=100_000_000)
    ap.add_argument("--vocab", type=int, default=30522)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args()

    from . import _lib
    from . import kernels as K
    from .gemm import gemm

    hbm, flops_peak, src = _peaks()
    dt = torch.bfloat16
    out = {"kernel": a.kernel, "peaks": src}
    if a.kernel == "gemm":
        M, N, Kd = a.m, a.n, a.k
        ta, tb = {"nt": (False, True), "nn": (False, False), "tn": (True, False)}[a.layout]
        A = torch.randn((Kd, M) if ta else (M, Kd), device="cuda", dtype=dt)
        B = torch.randn((N, Kd) if tb else (Kd, N), device="cuda", dtype=dt)
        D = torch.zeros(M, N, device="cuda", dtype=torch.float32 if a.acc else dt)
        bias = torch.randn(N, device="cuda", dtype=dt) if a.gelu else None
        fn = lambda: gemm(A, B, trans_a=ta, trans_b=tb, out=D, accumulate=a.acc, bias=bias, gelu=a.gelu)  # noqa: E731
        t = _time(fn, a.iters, a.warmup, not a.no_flush)
        fl = 2.0 * M * N * Kd
        out.update(M=M, N=N, K=Kd, layout=a.layout, acc=a.acc, ms=t * 1e3, tflops=fl / t / 1e12,
                   frac_of_peak=fl / t / flops_peak)
    elif a.kernel in ("attn", "attn_bwd"):
        B, H, S, D = a.batch, a.heads, a.seq, 64
        qkv = torch.randn(B, S, 3, H, D, device="cuda", dtype=dt)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        if a.kernel == "attn":
            fn = lambda: K.attn_fwd(q, k, v, p_drop=a.dropout, seed=1, offset=1)  # noqa: E731
            fl = 4.0 * B * H * S * S * D
        else:
            o, lse = K.attn_fwd(q, k, v, p_drop=a.dropout, seed=1, offset=1)
            do = torch.randn_like(o)
            fn = lambda: K.attn_bwd(q, k, v, o, lse, do, p_drop=a.dropout, seed=1, offset=1)  # noqa: E731
            fl = 10.0 * B * H * S * S * D
        t = _time(fn, a.iters, a.warmup, not a.no_flush)
        out.update(B=B, H=H, S=S, D=D, dropout=a.dropout, ms=t * 1e3, tflops=fl / t / 1e12,
                   frac_of_peak=fl / t / flops_peak)
    elif a.kernel in ("ln", "ln_bwd"):
        R, Hd = a.rows, a.hidden
        x = torch.randn(R, Hd, device="cuda", dtype=dt)
        r = torch.randn(R, Hd, device="cuda", dtype=dt)
        g = torch.ones(Hd, device="cuda", dtype=dt)
        b = torch.zeros(Hd, device="cuda", dtype=dt)
        if a.kernel == "ln":
            fn = lambda: K.ln_fwd(x, r, g, b, 1e-5, a.dropout, 1, 1)  # noqa: E731
            nbytes = 4 * R * Hd * 2
        else:
            y, z, mean, rstd = K.ln_fwd(x, r, g, b, 1e-5, a.dropout, 1, 1)
            dy = torch.randn_like(x)
            fn = lambda: K.ln_bwd(dy, z, g, mean, rstd, a.dropout, 1, 1)  # noqa: E731
            nbytes = (3 + (1 if a.dropout > 0 else 0)) * R * Hd * 2
        t = _time(fn, a.iters, a.warmup, not a.no_flush)
        out.update(rows=R, hidden=Hd, dropout=a.dropout, ms=t * 1e3, gbs=nbytes / t / 1e9,
                   frac_of_peak=nbytes / t / hbm)
    elif a.kernel == "adam":
        n = a.numel
        p, gr, m, v = (torch.randn(n, device="cuda") for _ in range(4))
        p16 = torch.empty(n, device="cuda", dtype=dt)
        fn = lambda: K.adam_flat(p, gr, m, v, p16, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, False)  # noqa: E731
        t = _time(fn, a.iters, a.warmup, not a.no_flush)
        nbytes = n * (4 * 4 + 3 * 4 + 2)
        out.update(numel=n, ms=t * 1e3, gbs=nbytes / t / 1e9, frac_of_peak=nbytes / t / hbm)
    elif a.kernel == "xent":
        R, V = a.rows, a.vocab
        ld = (V + 63) // 64 * 64
        logits = torch.randn(R, ld, device="cuda", dtype=dt)
        labels = torch.randint(0, V, (R,), device="cuda")
        labels[torch.rand(R, device="cuda") > 0.15] = -100
        fn = lambda: K.xent_fwd(logits, labels, V)  # noqa: E731
        t = _time(fn, a.iters, a.warmup, not a.no_flush)
        nbytes = int(0.15 * R) * ld * 2
        out.update(rows=R, vocab=V, ms=t * 1e3, gbs=nbytes / t / 1e9, frac_of_peak=nbytes / t / hbm)
    elif a.kernel == "colsum":
        x = torch.randn(a.rows, a.hidden, device="cuda", dtype=dt)
        o = torch.zeros(a.hidden, device="cuda")
        fn = lambda: K.colsum(x, o)  # noqa: E731
        t = _time(fn, a.iters, a.warmup, not a.no_flush)
        nbytes = a.rows * a.hidden * 2
        out.update(rows=a.rows, hidden=a.hidden, ms=t * 1e3, gbs=nbytes / t / 1e9, frac_of_peak=nbytes / t / hbm)
    elif a.kernel in ("ag_gemm", "gemm_rs"):
        from ..parallel.distop import DistGroup, _gather_spec, _gemm_rs

        M, N, Kd, n = a.m, a.n, a.k, a.ranks
        ks = Kd // n
        grp = DistGroup(list(range(n)), N * Kd, dt, torch.device("cuda"), local=True)
        x = torch.randn(M, Kd, device="cuda", dtype=dt)
        if a.kernel == "ag_gemm":
            shards = [torch.randn(N, ks, device="cuda", dtype=dt) for _ in range(n)]
            wfull = grp.staging[: N * Kd].view(N, Kd)
            spec = _gather_spec(grp, [t.data_ptr() for t in shards], N, ks)
            fn = lambda: gemm(x, wfull, gather=spec)  # noqa: E731
        else:
            dy = torch.randn(M, N, device="cuda", dtype=dt)
            grads = [torch.zeros(N, ks, device="cuda") for _ in range(n)]
            ptrs = [t.data_ptr() for t in grads]
            fn = lambda: _gemm_rs(dy, x, N, Kd, ptrs, ks, 1.0)  # noqa: E731
        t = _time(fn, a.iters, a.warmup, not a.no_flush)
        fl = 2.0 * M * N * Kd
        # bytes that would cross NVLink with real peers: the other ranks' slices (in), or the other ranks'
        # gradient blocks (out, fp32)
        link = (n - 1) / n * N * Kd * (2 if a.kernel == "ag_gemm" else 4)
        t_roof = max(fl / flops_peak, link / 770e9)
        out.update(M=M, N=N, K=Kd, ranks=n, ms=t * 1e3, tflops=fl / t / 1e12, frac_of_peak=fl / t / flops_peak,
                   link_bytes=link, roofline_ms=t_roof * 1e3, frac_of_roofline=t_roof / t)
    elif a.kernel == "rs_adam":
        import ctypes

        from ..parallel.fused_reduce import MAX_PEERS, _Args

        n = a.numel // 64 * 64
        grad = torch.randn(n, device="cuda")
        p16 = torch.zeros(n, device="cuda", dtype=dt)
        master, m, v = (torch.randn(n, device="cuda") for _ in range(3))
        flags = torch.zeros(2 * MAX_PEERS, dtype=torch.int32, device="cuda")
        done = torch.zeros(1, dtype=torch.int32, device="cuda")
        state = {"epoch": 0}

        def fn():
            state["epoch"] += 1
            g = _Args()
            g.peer_grad[0], g.peer_param[0], g.peer_flags[0] = grad.data_ptr(), p16.data_ptr(), flags.data_ptr()
            g.master, g.m, g.v, g.done_counter = master.data_ptr(), m.data_ptr(), v.data_ptr(), done.data_ptr()
            g.lo, g.len, g.nranks, g.my_idx, g.epoch = 0, n, 1, 0, state["epoch"]
            g.grad_mul, g.lr, g.beta1, g.beta2, g.eps = 1.0, 1e-3, 0.9, 0.999, 1e-8
            g.weight_decay, g.bias_corr1, g.bias_corr2, g.adamw, g.dtype16 = 0.0, 0.1, 0.001, 0, 1
            _lib.check(_lib.lib().rb_rs_adam_ag(ctypes.byref(g), _lib.stream_ptr()), "rb_rs_adam_ag")

        t = _time(fn, a.iters, a.warmup, not a.no_flush)
        nbytes = n * (4 + 3 * 4 + 3 * 4 + 2)   # grad in; master, m, v in and out; 16-bit parameter out
        out.update(numel=n, ms=t * 1e3, gbs=nbytes / t / 1e9, frac_of_peak=nbytes / t / hbm)
    elif a.kernel in ("bn", "bn_bwd", "im2col"):
        N, C, HW = a.batch, a.channels, a.hw
        x4 = torch.randn(N, HW, HW, C, device="cuda", dtype=dt)
        R = N * HW * HW
        x2 = x4.view(R, C)
        if a.kernel == "im2col":
            fn = lambda: K.im2col(x4, 3, 1, 1)  # noqa: E731
            nbytes = R * C * 2 * 10          # the input once, nine shifted copies written
        else:
            g, b = torch.ones(C, device="cuda"), torch.zeros(C, device="cuda")
            rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
            res = torch.randn(R, C, device="cuda", dtype=dt)
            if a.kernel == "bn":
                fn = lambda: K.bn_fwd(x2, res, g, b, rm, rv, 1e-5, 0.1, True)  # noqa: E731
                nbytes = R * C * 2 * 4       # x twice (statistics, apply), residual, y
            else:
                y, mean, rstd = K.bn_fwd(x2, res, g, b, rm, rv, 1e-5, 0.1, True)
                dy = torch.randn_like(y)
                fn = lambda: K.bn_bwd(x2, dy, y, mean, rstd, g, True, True)  # noqa: E731
                nbytes = R * C * 2 * 8       # x, dy, y twice each (reduce, apply); dx, dres written
        t = _time(fn, a.iters, a.warmup, not a.no_flush)
        out.update(N=N, C=C, HW=HW, ms=t * 1e3, gbs=nbytes / t / 1e9, frac_of_peak=nbytes / t / hbm)
    out["device_error_word"] = _lib.read_error()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
