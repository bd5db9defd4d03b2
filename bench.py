#!/usr/bin/env python
"""Headline benchmark: BERT-Large masked-LM + NSP pre-training throughput (samples/s).

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Model and data follow the benchmark definition: 24 layers, hidden 1024, 16 heads,
FFN 4096, GELU, post-LN, vocabulary 30522, sequence length 512, bf16 mixed
precision (fp32 master weights and Adam moments), global batch 256 split evenly
over the GPUs (strong scaling), token ids uniform over the vocabulary, 15 % of the
positions used as MLM labels, NSP labels Bernoulli(0.5), random-init weights.
The model is wrapped in ``RaNNCModule`` (the public API); partitioning
(stages x replicas x micro-batches) is decided by the framework.

Two timed regions of K optimizer steps each, after W warm-up steps:
  * ``value``: inputs already on the device, CUDA events around the K steps;
  * ``e2e``:   every step copies its inputs from pinned host memory and reads the
               loss back to the host.
Both are the maximum over ranks.  Rank 0 prints one JSON line.

Arms (``--impl``):
  * ``ours``      (default) this library.  Before its own model is built it also runs the ``eager`` arm for
                  a few steps (outside every timed region of its own) and reports ``vs_baseline`` = its
                  samples/s over the eager arm's.
  * ``eager``     stock PyTorch only: the same ``nn.Module``, ``F.scaled_dot_product_attention``, bf16
                  autocast, ``torch.optim.Adam(fused=True)``, ``DistributedDataParallel`` when N > 1; none of
                  this library's kernels, planner or runtime is imported.
  * ``reference`` the reference implementation itself (prints why it is unavailable here).

Other models: ``--model bert13b`` (256 layers, hidden 2048; parameters declared under
``DistributeModelParams``, ZeRO, 8 micro-batches), ``--model bert26b`` (128 layers, hidden 4096;
tensor-partitioned linear layers + pipeline + data parallel, global batch 128), ``--model wide_resnet``.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


def reference_unavailable():
    print(json.dumps({
        "impl": "reference",
        "unavailable": "the reference cannot be installed offline here: its CMake configure step fails "
                       "(MPI not found; six empty git submodules; needs PyTorch 1.11 JIT internals, Boost, Apex)"}))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for nm, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def _plain_bert_module(fname: str = "bert.py"):
    """The model files are plain ``torch.nn`` code; load one by path so that the eager arm imports nothing
    else of this library."""
    spec = importlib.util.spec_from_file_location("_bench_plain_" + fname[:-3],
                                                  os.path.join(HERE, "rannc_b200", "models", fname))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def _dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def _max_over_ranks(x: float, dev) -> float:
    import torch
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return x


def _barrier():
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def run_eager(args, steps: int, warmup: int, want_e2e: bool):
    """Stock PyTorch arm.  Returns a dict with value / ms_per_step (/ e2e).  The global batch of one optimizer
    step is the same as in the other arm; when the activations of a rank's whole share do not fit, the share is
    processed in equal micro-batches with gradient accumulation (``no_sync`` under DDP until the last one)."""
    import contextlib

    import torch
    import torch.distributed as dist

    rank, world, local = _dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1234)
    lb = args.global_batch // world
    n_sets = 2
    host = []
    resnet = args.model == "wide_resnet"
    scaler = None
    if resnet:
        # the same wide ResNet-152 on stock PyTorch: channels-last, fp16 autocast with a GradScaler (or bf16),
        # SGD momentum
        rn = _plain_bert_module("resnet.py")
        half = (args.amp_dtype or "fp16") == "fp16"
        amp_dtype = torch.float16 if half else torch.bfloat16
        model = rn.ResNetWithLoss(rn.wide_resnet152(width_mult=args.width)).to(dev).to(
            memory_format=torch.channels_last)
        opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
        scaler = torch.amp.GradScaler("cuda") if half else None
        for s in range(n_sets):
            g = torch.Generator().manual_seed(100 + s)
            x = torch.randn(lb, 3, args.image, args.image, generator=g).to(amp_dtype).contiguous(
                memory_format=torch.channels_last).pin_memory()
            y = torch.randint(0, 1000, (lb,), generator=g).pin_memory()
            host.append((x, y))
        default_micro = 32
    else:
        bert = _plain_bert_module()
        amp_dtype = torch.bfloat16
        cfg = bert.BertConfig(hidden_size=args.hidden, num_hidden_layers=args.layers,
                              num_attention_heads=args.heads, intermediate_size=4 * args.hidden,
                              max_position_embeddings=max(512, args.seq))
        model = bert.BertForPreTraining(cfg).to(dev)
        opt = torch.optim.Adam(model.parameters(), lr=1e-4, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.0,
                               fused=True)
        for s in range(n_sets):
            full = bert.synthetic_batch(cfg, args.global_batch, args.seq, seed=100 + s)
            host.append(tuple(t[rank * lb:(rank + 1) * lb].contiguous().pin_memory() for t in full))
        default_micro = 64
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], gradient_as_bucket_view=True) \
        if world > 1 else model
    dev_sets = [tuple(t.to(dev) for t in hs) for hs in host]
    micro = [min(lb, args.eager_micro_batch if args.eager_micro_batch > 0 else default_micro)]

    def one_step(batch):
        nmb = (lb + micro[0] - 1) // micro[0]
        total = None
        for i in range(nmb):
            sl = tuple(t[i * micro[0]:(i + 1) * micro[0]] for t in batch)
            last = i == nmb - 1
            ctx = net.no_sync() if (world > 1 and not last) else contextlib.nullcontext()
            with ctx:
                with torch.autocast("cuda", dtype=amp_dtype):
                    loss = net(*sl)
                part = loss * (sl[0].shape[0] / lb)
                (scaler.scale(part) if scaler is not None else part).backward()
            total = loss.detach() if total is None else total + loss.detach()
        if scaler is not None:
            scaler.step(opt)
            scaler.update()
        else:
            opt.step()
        opt.zero_grad(set_to_none=True)
        return total / nmb

    # warm-up; a micro-batch that does not fit is halved (every rank takes the same decision)
    done = 0
    while done < warmup:
        try:
            one_step(dev_sets[done % n_sets])
            torch.cuda.synchronize()
            oom = 0
        except torch.OutOfMemoryError:
            oom = 1
        oom = int(_max_over_ranks(float(oom), dev))
        if oom:
            opt.zero_grad(set_to_none=True)
            torch.cuda.empty_cache()
            if micro[0] <= 1:
                raise RuntimeError("eager arm: out of memory at micro-batch 1")
            micro[0] //= 2
            done = 0
            continue
        done += 1

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    _barrier()
    torch.cuda.synchronize()
    e0.record()
    for i in range(steps):
        last = one_step(dev_sets[(warmup + i) % n_sets])
    e1.record()
    torch.cuda.synchronize()
    _barrier()
    ms = _max_over_ranks(e0.elapsed_time(e1), dev)
    out = {"value": args.global_batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "micro_batch": micro[0],
           "last_loss": float(last.item()), "params": sum(p.numel() for p in model.parameters())}
    if want_e2e:
        h2d = sum(t.numel() * t.element_size() for t in host[0])
        _barrier()
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        e0.record()
        for i in range(steps):
            batch = tuple(t.to(dev, non_blocking=True) for t in host[i % n_sets])
            lv = float(one_step(batch).item())
        e1.record()
        torch.cuda.synchronize()
        wall = (time.perf_counter() - w0) * 1e3
        _barrier()
        e2e_ms = _max_over_ranks(max(e0.elapsed_time(e1), wall), dev)
        out["e2e"] = {"value": args.global_batch * steps / (e2e_ms / 1e3), "unit": "samples/s",
                      "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / steps,
                      "last_loss": lv}
    del net, model, opt, dev_sets
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    return out


def eager_main(args):
    import torch

    rank, world, local = _dist_env()
    if world != args.gpus:
        if rank == 0:
            print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch one process per GPU", file=sys.stderr)
        return 2
    sampler = ClockSampler(local)
    sampler.start()
    r = run_eager(args, args.steps, args.warmup, not args.no_e2e)
    clocks = sampler.stop()
    if rank == 0 and args.model == "wide_resnet":
        print(json.dumps({
            "metric": "ResNet samples/s (max over ranks)", "value": r["value"], "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": args.amp_dtype or "fp16",
            "data": "synthetic (N(0,1) images, uniform labels), random-init weights", "impl": "eager",
            "config": {"model": f"wide ResNet-152 x{args.width:g}", "params": r["params"],
                       "global_batch": args.global_batch, "image": args.image,
                       "parallelism": (f"ddp{world}" if world > 1 else "single") + f"_microbatch{r['micro_batch']}",
                       "optimizer": "torch.optim.SGD(momentum=0.9), autocast + GradScaler, channels-last, cuDNN",
                       "l2": "per-step working set far exceeds the 126 MB L2; no flush needed"},
            "clocks": clocks, "e2e": r.get("e2e"), "gpu_launches": 0,
            "note": "stock PyTorch kernels only (context number, not this library)"}))
    elif rank == 0:
        print(json.dumps({
            "metric": "BERT samples/s (max over ranks)", "value": r["value"], "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (uniform token ids, 15% MLM labels, Bernoulli NSP), random-init weights",
            "impl": "eager",
            "config": {"model": f"BERT {args.layers}L/{args.hidden}H/{args.heads}heads MLM+NSP", "params": r["params"],
                       "global_batch": args.global_batch, "seq_len": args.seq,
                       "parallelism": (f"ddp{world}" if world > 1 else "single") + f"_microbatch{r['micro_batch']}",
                       "optimizer": "torch.optim.Adam(fused=True), bf16 autocast, SDPA",
                       "l2": "per-step working set far exceeds the 126 MB L2; no flush needed"},
            "clocks": clocks, "e2e": r.get("e2e"), "gpu_launches": 0,
            "note": "stock PyTorch kernels only (context number, not this library)"}))
    _barrier()
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "eager", "reference"])
    ap.add_argument("--global-batch", type=int, default=0, help="0: the model's benchmark definition")
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--hidden", type=int, default=0)
    ap.add_argument("--heads", type=int, default=0)
    ap.add_argument("--zero", type=int, default=-1, help="-1: on when more than one GPU")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-baseline", action="store_true", help="ours: do not run the eager arm for vs_baseline")
    ap.add_argument("--baseline-steps", type=int, default=3)
    ap.add_argument("--eager-micro-batch", type=int, default=0, help="eager arm: rows per micro-batch (0: 64)")
    ap.add_argument("--model", default="bert", choices=["bert", "bert13b", "bert26b", "wide_resnet"],
                    help="bert: the headline benchmark; bert13b / bert26b: the enlarged configurations; "
                         "wide_resnet: ResNet-152 with every width x --width")
    ap.add_argument("--width", type=float, default=8.0)
    ap.add_argument("--image", type=int, default=224)
    ap.add_argument("--amp-dtype", default="", choices=["", "fp16", "bf16"],
                    help="16-bit compute type (default: bf16 for bert, fp16 for wide_resnet)")
    ap.add_argument("--dist-params", type=int, default=-1, help="declare the model under DistributeModelParams "
                                                                "(-1: on for bert13b)")
    ap.add_argument("--pipeline", type=int, default=0, help="force this many micro-batches (0: planner's choice; "
                                                            "bert13b defaults to 8)")
    ap.add_argument("--stages", type=int, default=0, help="force this many pipeline stages (0: planner's choice)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_unavailable()
        return 0
    if args.warmup < 3:
        args.warmup = 3
    shape = {"bert": (24, 1024, 16, 256), "bert13b": (256, 2048, 32, 256), "bert26b": (128, 4096, 64, 128),
             "wide_resnet": (24, 1024, 16, 256)}[args.model]
    args.layers = args.layers or shape[0]
    args.hidden = args.hidden or shape[1]
    args.heads = args.heads or shape[2]
    args.global_batch = args.global_batch or shape[3]
    if args.impl == "eager":
        return eager_main(args)

    # ---- baseline context number first, while the device is still empty (stock PyTorch, outside every timed
    # region of this library's arm)
    baseline = None
    if args.model == "bert" and not args.no_baseline and int(os.environ.get("WORLD_SIZE", "1")) == args.gpus:
        try:
            baseline = run_eager(args, max(1, args.baseline_steps), 3, False)
        except Exception as e:  # noqa: BLE001
            baseline = {"error": f"{type(e).__name__}: {e}"[:200]}

    if args.model == "bert13b" and args.pipeline == 0:
        args.pipeline = 8
    if args.pipeline > 0:
        os.environ.setdefault("RANNC_PIPELINE_NUM", str(args.pipeline))
    if args.stages > 0:
        os.environ.setdefault("RANNC_PARTITION_NUM", str(args.stages))
    if args.model == "bert26b":
        os.environ.setdefault("RANNC_FORCE_DIST_MATMUL", "true")
    if args.model == "wide_resnet" and args.gpus == 1:
        # one stage, several micro-batches: each micro-batch's backward right after its forward, so that nothing
        # has to be recomputed (185.7 against 141.2 samples/s on one GPU).  Measured on one GPU only, hence not
        # switched on for more (set RANNC_INTERLEAVE_BACKWARD=true to try it there).
        os.environ.setdefault("RANNC_INTERLEAVE_BACKWARD", "true")

    import torch

    import rannc_b200 as pyrannc
    from rannc_b200.models.bert import BertConfig, BertForPreTraining, synthetic_batch
    from rannc_b200.ops import _lib

    rank, world = pyrannc.get_rank(), pyrannc.get_world_size()
    if world != args.gpus:
        if rank == 0:
            print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch one process per GPU", file=sys.stderr)
        return 2
    dev = pyrannc._comm.device()
    if dev.type != "cuda":
        print("bench.py needs a CUDA device", file=sys.stderr)
        return 2
    torch.manual_seed(1234)
    lb = args.global_batch // world
    n_sets = 4
    host = []
    half = False
    is_bert = args.model.startswith("bert")
    if is_bert:
        cfg = BertConfig(hidden_size=args.hidden, num_hidden_layers=args.layers, num_attention_heads=args.heads,
                         intermediate_size=4 * args.hidden, max_position_embeddings=max(512, args.seq))
        dist_params = (args.model == "bert13b") if args.dist_params < 0 else bool(args.dist_params)
        big = args.model in ("bert13b", "bert26b")
        if big:
            # tens of billions of parameters: they are created on the device, in the 16-bit compute type, with
            # the layers' own default initialisation (a host-side fp32 copy per rank would not fit the host)
            import contextlib

            os.environ.setdefault("RANNC_MEASURE_PROFILES", "false")
            prev_dtype = torch.get_default_dtype()
            torch.set_default_dtype(torch.bfloat16)
            ctx = pyrannc.DistributeModelParams() if dist_params else contextlib.nullcontext()
            try:
                with torch.device(dev), ctx:
                    # with dist_params every parameter is cut to this rank's 1/world shard as soon as its
                    # layer exists; full values are assembled on the owners at deployment
                    model = BertForPreTraining(cfg, init_weights=False)
            finally:
                torch.set_default_dtype(prev_dtype)
        elif dist_params:
            with pyrannc.DistributeModelParams():
                model = BertForPreTraining(cfg, init_weights=False)
        else:
            model = BertForPreTraining(cfg)
        optimizer = torch.optim.Adam(model.parameters(), lr=1e-4, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.0)
        if args.zero < 0:
            use_zero = world > 1 and args.model != "bert26b"   # tensor-partitioned layers exclude ZeRO
        else:
            use_zero = bool(args.zero)
        n_sets = 4 if args.model == "bert" else 2
        # a few distinct synthetic batches in pinned host memory
        for s in range(n_sets):
            full = synthetic_batch(cfg, args.global_batch, args.seq, seed=100 + s)
            host.append(tuple(t[rank * lb:(rank + 1) * lb].contiguous().pin_memory() for t in full))
    else:
        # wide ResNet-152: bottleneck blocks 3/8/36/3, every convolution x --width, BatchNorm, fp16 mixed
        # precision (every step checks the gradients for overflow; the loss scale stays 1 unless the caller installs a
        # dynamic scaler with amp.initialize), SGD momentum 0.9, images N(0, 1), labels uniform over 1000 classes
        from rannc_b200.models.resnet import ResNetWithLoss, wide_resnet152

        half = (args.amp_dtype or "fp16") == "fp16"
        pyrannc.amp.set_dtype(torch.float16 if half else torch.bfloat16)
        model = ResNetWithLoss(wide_resnet152(width_mult=args.width))
        optimizer = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
        use_zero = False if args.zero < 0 else bool(args.zero)
        n_sets = 2
        for s in range(n_sets):
            g = torch.Generator().manual_seed(100 + s)
            x = torch.randn(lb, 3, args.image, args.image, generator=g).to(
                torch.float16 if half else torch.bfloat16).pin_memory()
            y = torch.randint(0, 1000, (lb,), generator=g).pin_memory()
            host.append((x, y))
    nparams = sum(p.numel() for p in model.parameters())
    wrapped = pyrannc.RaNNCModule(model, optimizer, enable_apex_amp=True, enable_zero=use_zero)
    t_start = time.perf_counter()

    def progress(what):
        # large models spend minutes before the first step: say where (stderr, rank 0)
        if rank == 0 and args.model != "bert":
            print(f"[bench] +{time.perf_counter() - t_start:.1f}s {what}", file=sys.stderr, flush=True)

    progress(f"model built ({nparams / 1e9:.2f} B parameters)")

    h2d_bytes = sum(t.numel() * t.element_size() for t in host[0])
    dev_sets = [tuple(t.to(dev) for t in hs) for hs in host]

    def step_device(i):
        loss = wrapped(*dev_sets[i % n_sets])
        loss.backward()
        optimizer.step()
        optimizer.zero_grad()
        return loss

    def step_e2e(i):
        batch = tuple(t.to(dev, non_blocking=True) for t in host[i % n_sets])
        loss = wrapped(*batch)
        loss.backward()
        optimizer.step()
        optimizer.zero_grad()
        return float(loss.item())  # device -> host read of the step's result

    losses = []
    for i in range(args.warmup):
        losses.append(float(step_device(i).item()))
        progress(f"warm-up step {i} done (the first one traces, plans and deploys)")
    torch.cuda.synchronize()

    # value check of the fused gradient path under this very run: one step from the same state down the
    # fused kernel and down the NCCL collectives (outside the timed regions)
    fused_err = None
    red = getattr(wrapped, "_fused_reducer", None)
    if world > 1 and red is not None and args.model not in ("bert13b", "bert26b"):
        # (not for the enlarged models: the check clones the optimizer state, tens of GB there)
        try:
            from rannc_b200.parallel.fused_reduce import compare_with_collectives

            fused_err = compare_with_collectives(wrapped, optimizer, lambda: step_device(0))
        except Exception as e:  # noqa: BLE001
            fused_err = f"{type(e).__name__}: {e}"[:200]

    # host time to enqueue one step, with an idle device and an empty launch queue (no synchronisation inside).
    # A step of tens of thousands of launches fills the launch queue, after which the host advances at the
    # device's pace: for the enlarged models this figure is an upper bound of the host's own work, not a measure.
    enq = []
    for i in range(1 if args.model in ("bert13b", "bert26b") else 3):
        torch.cuda.synchronize()
        pyrannc.barrier()
        t0 = time.perf_counter()
        step_device(i)
        enq.append((time.perf_counter() - t0) * 1e3)
        progress("enqueue-time step done")
    torch.cuda.synchronize()
    host_enqueue_ms = _max_over_ranks(statistics.median(enq), dev)

    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    pyrannc.barrier()
    torch.cuda.synchronize()
    l0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        last = step_device(args.warmup + i)
    e1.record()
    torch.cuda.synchronize()
    pyrannc.barrier()
    launches = _lib.launch_count() - l0
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    pyrannc._comm.allreduce(t, "max")
    ms = float(t.item())
    losses.append(float(last.item()))

    e2e = None
    if not args.no_e2e:
        pyrannc.barrier()
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        e0.record()
        for i in range(args.steps):
            lv = step_e2e(i)
        e1.record()
        torch.cuda.synchronize()
        wall = (time.perf_counter() - w0) * 1e3
        pyrannc.barrier()
        t = torch.tensor([max(e0.elapsed_time(e1), wall)], dtype=torch.float64, device=dev)
        pyrannc._comm.allreduce(t, "max")
        e2e_ms = float(t.item())
        e2e = {"value": args.global_batch * args.steps / (e2e_ms / 1e3), "unit": "samples/s",
               "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / args.steps,
               "last_loss": lv}
    clocks = sampler.stop()
    err = _lib.read_error()
    peak_mem = torch.tensor([float(torch.cuda.max_memory_allocated(dev))], dtype=torch.float64, device=dev)
    pyrannc._comm.allreduce(peak_mem, "max")

    if rank == 0:
        dep = wrapped._dep
        stages = len(dep.fwd_graph_order)
        repl = [len(dep.allocation[s]) for s in dep.fwd_graph_order]
        par = (f"pp{stages}" if stages > 1 else "") + f"dp{repl[0]}" + (f"_mb{dep.pipeline_num}" if dep.pipeline_num > 1 else "") \
            + ("_zero" if use_zero else "") + ("_distop" if getattr(wrapped, "_dist_groups", None) else "")
        if is_bert:
            mname = (f"BERT-Large {args.layers}L/{args.hidden}H/{args.heads}heads MLM+NSP" if
                     (args.layers, args.hidden) == (24, 1024) else
                     f"BERT {args.layers}L/{args.hidden}H/{args.heads}heads MLM+NSP")
            data = "synthetic (uniform token ids, 15% MLM labels, Bernoulli NSP), random-init weights"
            optname, dtype = "Adam (fused, fp32 master)", "bf16"
        else:
            mname = f"Wide ResNet-152 (widths x{args.width:g}), {args.image}x{args.image} images"
            data = "synthetic (N(0,1) images, uniform labels over 1000 classes), random-init weights"
            optname = "SGD momentum 0.9 (fused, fp32 master" + (", fp16 overflow check at loss scale 1)" if half else ")")
            dtype = "fp16" if half else "bf16"
        value = args.global_batch * args.steps / (ms / 1e3)
        plan = getattr(wrapped, "_plan", None)
        planned_ms = None
        if plan is not None and getattr(plan, "estimates", None):
            try:
                from rannc_b200.graph.planner import planned_step_ms

                planned_ms = planned_step_ms(plan.estimates, dep.pipeline_num)
            except Exception:  # noqa: BLE001
                planned_ms = None
        out = {
            "metric": ("BERT" if is_bert else "ResNet") + " samples/s (max over ranks)",
            "value": value,
            "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (value / baseline["value"]) if baseline and "value" in baseline else None,
            "baseline_impl": "eager PyTorch in the same process before this arm (bf16 autocast, SDPA, fused Adam"
                             + (", DDP" if world > 1 else "") + "): see --impl eager" if baseline else None,
            "baseline": baseline,
            "dtype": dtype, "data": data,
            "impl": "ours",
            "config": {"model": mname,
                       "params": nparams, "global_batch": args.global_batch,
                       "seq_len": args.seq if is_bert else None,
                       "parallelism": par, "stages": stages, "replicas": repl, "micro_batches": dep.pipeline_num,
                       "checkpointing": bool(dep.checkpointing), "optimizer": optname,
                       "l2": "per-step working set (weights 0.67 GB + activations, tens of GB) far exceeds the "
                             "126 MB L2; no flush needed"},
            "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": launches,
            "launches_per_step": launches / max(1, args.steps),
            "host_enqueue_ms": host_enqueue_ms,
            "planned_step_ms": planned_ms,
            "fused_reduce": bool(red is not None),
            "multimem": bool(red is not None and red.multimem_active()),
            "overlap_buckets": int(red.num_buckets()) if red is not None else 0,
            "fused_vs_nccl_max_rel_err": fused_err,
            "peak_mem_bytes": int(peak_mem.item()),
            "device_error_word": err,
            "losses": [round(x, 4) for x in losses],
        }
        print(json.dumps(out))
    pyrannc.barrier()
    return 0


if __name__ == "__main__":
    sys.exit(main())
