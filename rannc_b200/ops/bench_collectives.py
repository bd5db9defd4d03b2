"""Micro-benchmarks of the fused compute + collective kernels over REAL peers (one process per GPU).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m rannc_b200.ops.bench_collectives rs_adam --numel 336000000 [--multimem 0|1] [--ctas 0]
    ...                                          ag_gemm --m 8192 --n 4096 --k 4096
    ...                                          gemm_rs --m 8192 --n 4096 --k 4096
    ...                                          barrier

``rs_adam``: the reduce-scatter + Adam + all-gather kernel on a flat buffer of ``--numel`` elements sharded over
the N ranks (symmetric memory; ``multimem.ld_reduce`` / ``multimem.st`` when the fabric gives a multicast
address and ``--multimem 1``, plain peer loads / stores otherwise).  ``ag_gemm`` / ``gemm_rs``: the
all-gather -> GEMM and GEMM -> reduce-scatter kernels of the tensor-partitioned linear layer with every rank's
weight slice / gradient block in its own GPU's symmetric memory.  ``barrier``: the one-warp flag barrier.

Timing: CUDA events on the launching stream after warm-up, a process-group barrier before every timed
launch so that the ranks start together, L2 flushed between iterations, the MAXIMUM over ranks of the mean
time per launch.  Rank 0 prints one JSON line with the bytes that cross NVLink per GPU and direction, the
roofline time -- the slower of FLOPs / measured GEMM peak, local bytes / measured copy bandwidth and link
bytes / 770 GB/s (measured peer copy, per direction and GPU) -- and the achieved fraction of it.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os

import torch

LINK_BPS = 770e9


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["rs_adam", "ag_gemm", "gemm_rs", "barrier"])
    ap.add_argument("--numel", type=int, default=336_000_000)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--multimem", type=int, default=1)
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args()

    import torch.distributed._symmetric_memory as symm_mem

    from ..parallel import comm
    from ..parallel.fused_reduce import MAX_PEERS, RS_BEGIN, RS_END, RS_PULL, RS_UPDATE, _Args, symm_empty
    from . import _lib

    comm.start()
    rank, world = comm.get_rank(), comm.get_world_size()
    dev = comm.device()
    hbm, flops_peak, src = _peaks()
    dt = torch.bfloat16
    flush = None if a.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    pg = comm.group(list(range(world))) if world > 1 else None
    lib = _lib.lib()

    def timed(fn, after=None):
        """``after``: launched behind the timed kernel, outside the events (a barrier that keeps a rank from
        starting the next launch while peers still use its buffers)."""
        for _ in range(a.warmup):
            fn()
            if after is not None:
                after()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        tot = 0.0
        for _ in range(a.iters):
            if flush is not None:
                flush.zero_()
            torch.cuda.synchronize()
            comm.barrier()
            s.record()
            fn()
            e.record()
            if after is not None:
                after()
            torch.cuda.synchronize()
            tot += s.elapsed_time(e)
        t = torch.tensor([tot / a.iters], dtype=torch.float64, device=dev)
        comm.allreduce(t, "max")
        return float(t.item()) * 1e-3

    out = {"kernel": a.kernel, "ranks": world, "peaks": src}
    if a.kernel in ("rs_adam", "barrier"):
        n = a.numel // (64 * world) * (64 * world)
        shard = n // world
        grad = symm_empty(n, torch.float32, dev).normal_()
        p16 = symm_empty(n, dt, dev).zero_()
        flags = symm_empty(2 * MAX_PEERS, torch.int32, dev).zero_()
        torch.cuda.synchronize()
        if world > 1:
            gh, ph, fh = (symm_mem.rendezvous(t, pg) for t in (grad, p16, flags))
        master, m, v = (torch.randn(shard, device=dev) for _ in range(3))
        done = torch.zeros(1, dtype=torch.int32, device=dev)
        state = {"epoch": 0}
        mc = bool(a.multimem) and world > 1 and bool(getattr(gh, "multicast_ptr", 0)) and \
            bool(getattr(ph, "multicast_ptr", 0))
        fptrs = (ctypes.c_void_p * MAX_PEERS)()
        for r in range(world):
            fptrs[r] = fh.buffer_ptrs[r] if world > 1 else flags.data_ptr()

        def launch():
            state["epoch"] += 1
            g = _Args()
            for r in range(world):
                g.peer_grad[r] = gh.buffer_ptrs[r] if world > 1 else grad.data_ptr()
                g.peer_param[r] = ph.buffer_ptrs[r] if world > 1 else p16.data_ptr()
                g.peer_flags[r] = fptrs[r]
            if mc:
                g.mc_grad, g.mc_param = gh.multicast_ptr, ph.multicast_ptr
            g.master, g.m, g.v, g.done_counter = master.data_ptr(), m.data_ptr(), v.data_ptr(), done.data_ptr()
            g.lo, g.len, g.nranks, g.my_idx, g.epoch = rank * shard, shard, world, rank, state["epoch"]
            g.grad_mul, g.lr, g.beta1, g.beta2, g.eps = 1.0 / world, 1e-3, 0.9, 0.999, 1e-8
            g.weight_decay, g.bias_corr1, g.bias_corr2, g.adamw, g.dtype16 = 0.0, 0.1, 0.001, 0, 1
            g.num_ctas = a.ctas
            g.mode = RS_BEGIN | RS_END | RS_PULL | RS_UPDATE
            _lib.check(lib.rb_rs_adam_ag(ctypes.byref(g), _lib.stream_ptr()), "rb_rs_adam_ag")

        def barrier_only():
            state["epoch"] += 1
            _lib.check(lib.rb_peer_barrier(fptrs, ctypes.c_int(world), ctypes.c_int(rank), ctypes.c_int(0),
                                           ctypes.c_uint(state["epoch"]), ctypes.c_ulonglong(0), _lib.stream_ptr()),
                       "rb_peer_barrier")

        if a.kernel == "barrier":
            t = timed(barrier_only)
            out.update(ms=t * 1e3)
        else:
            t = timed(launch)
            local = shard * (4 + 3 * 4 + 3 * 4 + 2)          # own gradients, state in and out, own 16-bit copy
            link_in = (world - 1) * shard * 4                 # the peers' gradients of this rank's shard
            link_out = (world - 1) * shard * 4                # this rank's gradients of the peers' shards
            t_roof = max(local / hbm, max(link_in, link_out) / LINK_BPS)
            out.update(numel=n, shard=shard, multimem=mc, ctas=a.ctas or 148, ms=t * 1e3, local_bytes=local,
                       link_in_bytes=link_in, link_out_bytes=link_out + (world - 1) * shard * 2,
                       link_gbs_in=link_in / t / 1e9, roofline_ms=t_roof * 1e3, frac_of_roofline=t_roof / t)
    else:
        from ..parallel.distop import DistGroup, _gather_spec, _gemm_rs
        from .gemm import gemm

        M, N, Kd = a.m, a.n, a.k
        ks = Kd // world
        grp = DistGroup(list(range(world)), N * Kd, dt, dev, local=(world == 1))
        x = torch.randn(M, Kd, device=dev, dtype=dt)
        if a.kernel == "ag_gemm":
            sh = grp.alloc_shared(N * ks, dt)
            sh.t.normal_()
            torch.cuda.synchronize()
            comm.barrier()
            wfull = grp.staging[: N * Kd].view(N, Kd)
            spec = _gather_spec(grp, sh.ptrs, N, ks)

            def launch():
                gemm(x, wfull, gather=spec)

            link = (world - 1) * N * ks * 2
        else:
            sh = grp.alloc_shared(N * ks, torch.float32)
            dy = torch.randn(M, N, device=dev, dtype=dt)
            comm.barrier()

            def launch():
                _gemm_rs(dy, x, N, Kd, sh.ptrs, ks, 1.0)

            link = (world - 1) * N * ks * 4
        t = timed(launch, after=grp.barrier)
        fl = 2.0 * M * N * Kd
        t_roof = max(fl / flops_peak, link / LINK_BPS)
        out.update(M=M, N=N, K=Kd, ms=t * 1e3, tflops=fl / t / 1e12, frac_of_peak=fl / t / flops_peak,
                   link_bytes=link, roofline_ms=t_roof * 1e3, frac_of_roofline=t_roof / t)
    torch.cuda.synchronize()
    err = torch.tensor([float(_lib.read_error())], dtype=torch.float64, device=dev)
    comm.allreduce(err, "max")
    out["device_error_word"] = int(err.item())
    if rank == 0:
        print(json.dumps(out))
    comm.barrier()
    comm.clear()


if __name__ == "__main__":
    main()
