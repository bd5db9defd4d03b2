"""Per-operator profiles for the partitioner's cost model.

Two modes:

* analytic (default, needs no GPU): a roofline estimate from shapes -- FLOPs
  over the sustained tensor-core rate and bytes over the copy bandwidth, both
  taken from the configuration (defaults are the rates measured on B200);
* measured (``measure_profiles``): every operator of the rewritten graph is
  timed on the device with CUDA events, forward and backward, on fake-shaped
  random inputs, and ``SubgraphProfiler`` runs whole candidate subgraphs --
  forward + backward at a given micro-batch size, with or without
  recomputation -- and reports device time (CUDA events), host enqueue time,
  the allocator peak, and the bytes kept for backward: the counterpart of the
  reference's GraphProfiler (src/comp/GraphProfiler.cpp:245-415), on the device
  clock instead of the host's.  The planner uses it in two ways: to calibrate
  the operator figures block by block (one measurement per block of the
  coarsened graph), and -- ``measure_subgraphs`` -- as the profile source of the
  stage search itself, one measurement per candidate stage like the reference.

Profiles are kept in the reference's ``ProfileDB`` file layout
(src/comp/GraphProfiler.h:54-57,133-160): ``save_graph_profile`` /
``load_graph_profile`` / ``graph_profile_file``.
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.fx as fx

from .. import _core
from ..utils.config import conf

_VIEW_OPS = {"aten::view", "aten::reshape", "aten::transpose", "aten::permute", "aten::unsqueeze", "aten::squeeze",
             "aten::slice", "aten::select", "aten::expand", "aten::t", "aten::sym_size", "aten::alias",
             "aten::detach", "prim::getitem", "aten::flatten", "aten::unflatten", "aten::contiguous"}


def _numel_bytes(val) -> int:
    if isinstance(val, torch.Tensor):
        n = 1
        for d in val.shape:
            n *= int(getattr(getattr(d, "node", None), "hint", d)) if not isinstance(d, int) else d
        return n * val.element_size()
    if isinstance(val, (list, tuple)):
        return sum(_numel_bytes(v) for v in val)
    return 0


def _shape(val):
    return [int(getattr(getattr(d, "node", None), "hint", d)) if not isinstance(d, int) else d for d in val.shape]


def _gemm_flops(x_val, w_val) -> float:
    xs, ws = _shape(x_val), _shape(w_val)
    m = 1
    for d in xs[:-1]:
        m *= d
    return 2.0 * m * ws[0] * ws[1]


def analytic_profiles(gm: fx.GraphModule) -> Dict[str, "_core.NodeProfile"]:
    tflops = float(conf("dev_tflops")) * 1e12
    hbm = float(conf("dev_hbm_gbs")) * 1e9
    overhead = 4.0
    out = {}
    for n in gm.graph.nodes:
        if n.op != "call_function":
            continue
        from .tracer import op_name

        name = op_name(n.target)
        val = n.meta.get("val")
        out_bytes = _numel_bytes(val)
        in_bytes = sum(_numel_bytes(a.meta.get("val")) for a in n.all_input_nodes)
        flops = 0.0
        act = out_bytes
        if name in _VIEW_OPS:
            out[n.name] = _core.NodeProfile(0.0, 0.0, 0, 0, False)
            continue
        args = n.args
        try:
            if name in ("rannc::linear", "aten::linear"):
                flops = _gemm_flops(args[0].meta["val"], args[1].meta["val"])
                if len(args) > 3 and args[3] == "gelu":
                    act = 2 * out_bytes
            elif name == "rannc::mlp":
                f1 = _gemm_flops(args[0].meta["val"], args[1].meta["val"])
                flops = 2 * f1
                xs, w1 = _shape(args[0].meta["val"]), _shape(args[1].meta["val"])
                m = 1
                for d in xs[:-1]:
                    m *= d
                act = out_bytes + 2 * m * w1[0] * args[0].meta["val"].element_size()
            elif name == "rannc::qkv_attention":
                xs, ws = _shape(args[0].meta["val"]), _shape(args[1].meta["val"])
                B, S = xs[0], xs[1]
                H = int(args[11])
                D = ws[0] // H
                flops = 3 * 2.0 * B * S * ws[0] * ws[1] + 4.0 * B * H * S * S * D
                act = 5 * B * S * ws[0] * args[0].meta["val"].element_size() + B * H * S * 4
            elif name in ("rannc::sdpa", "aten::scaled_dot_product_attention"):
                B, H, S, D = _shape(args[0].meta["val"])
                flops = 4.0 * B * H * S * S * D
                act = out_bytes + B * H * S * 4
                if name.startswith("aten"):
                    act += B * H * S * S * args[0].meta["val"].element_size()
            elif name in ("aten::matmul", "aten::bmm", "aten::mm", "aten::addmm"):
                a, b = args[-2].meta["val"], args[-1].meta["val"]
                sa, sb = _shape(a), _shape(b)
                m = 1
                for d in sa[:-1]:
                    m *= d
                flops = 2.0 * m * sa[-1] * sb[-1]
            elif name in ("aten::conv2d", "aten::convolution", "aten::_convolution", "rannc::conv2d"):
                w = _shape(args[1].meta["val"])
                o = _shape(val)
                flops = 2.0 * o[0] * o[1] * o[2] * o[3] * w[1] * w[2] * w[3]
        except Exception:  # noqa: BLE001 - estimates only
            flops = 0.0
        fwd = overhead + flops / tflops * 1e6 + (in_bytes + out_bytes) / hbm * 1e6
        bwd = overhead + 2.0 * flops / tflops * 1e6 + 2.0 * (in_bytes + out_bytes) / hbm * 1e6
        if name in ("rannc::sdpa", "aten::scaled_dot_product_attention"):
            bwd = overhead + 2.5 * flops / tflops * 1e6 + 2.0 * (in_bytes + out_bytes) / hbm * 1e6
        is_float = isinstance(val, torch.Tensor) and val.is_floating_point()
        out[n.name] = _core.NodeProfile(fwd, bwd if is_float or flops else 0.0, act if is_float else 0, 0, True)
    return out


def _with_main_grad(t: torch.Tensor) -> torch.Tensor:
    """A stand-in for a deployed 16-bit parameter: it carries the fp32 gradient buffer the fused operators
    accumulate into (and split K for), so that what is timed is what training runs."""
    if t.dtype in (torch.float16, torch.bfloat16):
        t.main_grad = torch.zeros(t.shape, dtype=torch.float32, device=t.device)
    return t


def measured_profiles(gm: fx.GraphModule, device, iters: int = 3, param_names=()) -> Dict[str, "_core.NodeProfile"]:
    """Times every call_function node on ``device`` with CUDA events (forward and backward).  ``param_names``:
    placeholders that are parameters (their stand-ins get an fp32 gradient buffer like deployed ones)."""
    base = analytic_profiles(gm)
    if not torch.cuda.is_available():
        return base
    from .tracer import op_name

    param_names = set(param_names)
    cur = [None]

    def real(v):
        if isinstance(v, torch.Tensor):
            shp = _shape(v)
            if v.is_floating_point():
                t = torch.randn(shp, dtype=v.dtype, device=device).requires_grad_(True)
                return _with_main_grad(t) if cur[0] in param_names else t
            return torch.zeros(shp, dtype=v.dtype, device=device)
        return v

    for n in gm.graph.nodes:
        if n.op != "call_function" or op_name(n.target) in _VIEW_OPS:
            continue
        try:
            def conv(a):
                if isinstance(a, fx.Node):
                    cur[0] = a.name
                    return real(a.meta.get("val"))
                if isinstance(a, (list, tuple)):
                    return type(a)(conv(x) for x in a)
                return a

            args = conv(n.args)
            kwargs = {k: conv(v) for k, v in n.kwargs.items()}
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ft = bt = 0.0
            for it in range(iters + 1):
                ev[0].record()
                y = n.target(*args, **kwargs)
                ev[1].record()
                did_bwd = False
                if isinstance(y, torch.Tensor) and y.requires_grad:
                    y.backward(torch.ones_like(y))
                    did_bwd = True
                ev[2].record()
                torch.cuda.synchronize()
                if it > 0:
                    ft += ev[0].elapsed_time(ev[1]) * 1e3
                    bt += ev[1].elapsed_time(ev[2]) * 1e3 if did_bwd else 0.0
            p = base[n.name]
            base[n.name] = _core.NodeProfile(ft / iters, bt / iters, p.activation_bytes, p.working_bytes, True)
        except Exception:  # noqa: BLE001 - keep the estimate for operators that cannot run standalone
            continue
    return base


_OP_ITER = 1          # ``iteration`` field of the ProfileDB key under which operator profiles are filed


def _key_graphs(ir_graph):
    """The traced graph under a fixed name (its own name carries the module's random id), as the ``ir_graphs``
    part of a ProfileDB key."""
    if ir_graph is None:
        return {}
    g = _core.IRGraph.loads(ir_graph.dumps())
    g.name = "model"
    return {"model": g}


def _as_graph_profile(name: str, p: "_core.NodeProfile") -> "_core.GraphProfile":
    gp = _core.GraphProfile()
    gp.name = name
    # microseconds, rounded up so that an operator that takes time never reads as free
    gp.fwd_time = int(-(-p.fwd_us // 1)) if p.fwd_us > 0 else 0
    gp.bwd_time = int(-(-p.bwd_us // 1)) if p.bwd_us > 0 else 0
    gp.fwd_cuda_time, gp.bwd_cuda_time = gp.fwd_time, gp.bwd_time
    gp.activation_size = int(p.activation_bytes)
    gp.working_mem = int(p.working_bytes)
    return gp


def save_profiles(path: str, profiles: Dict[str, "_core.NodeProfile"], batch: int, ir_graph=None,
                  db: "_core.ProfileDB" = None) -> None:
    """Writes the operator profiles in the reference's ``ProfileDB`` layout: one item whose key holds the traced
    graph and the batch size and whose result maps every operator id to a ``GraphProfile`` record
    (src/comp/GraphProfiler.h:54-57,133-160; config ``save_graph_profile``).  ``db``: a database that already
    holds subgraph measurements to be written along."""
    db = db if db is not None else _core.ProfileDB()
    graphs = _key_graphs(ir_graph)
    db.add(graphs, int(batch), _OP_ITER, False, {k: _as_graph_profile(k, p) for k, p in profiles.items()})
    with open(path, "wb") as f:
        f.write(db.dumps())


def load_profiles(path: str, node_ids, batch: int, ir_graph=None) -> Dict[str, "_core.NodeProfile"]:
    """Reads a file written by ``save_profiles``.  It must hold an item for this traced graph and batch size that
    covers exactly the graph's operators; anything else means it belongs to another model or configuration."""
    db = _core.ProfileDB()
    with open(path, "rb") as f:
        db.loads(f.read())
    graphs = _key_graphs(ir_graph)
    found = db.get(graphs, int(batch), _OP_ITER, False)
    if found is None:
        raise RuntimeError(f"profile file {path} has no entry for this graph at batch {batch}")
    want = set(node_ids)
    if set(found) != want:
        missing = sorted(want - set(found))[:5]
        raise RuntimeError(f"profile file {path} does not match the traced graph (e.g. missing {missing})")
    return {k: _core.NodeProfile(float(v.fwd_time), float(v.bwd_time), int(v.activation_size), int(v.working_mem),
                                 bool(v.fwd_time or v.bwd_time or v.activation_size))
            for k, v in found.items()}


class SubgraphProfiler:
    """Runs a set of operators of the traced graph as one graph on the device and measures it.

    ``measure(ids, batch, checkpointing)`` cuts the operators ``ids`` (plus the batch-independent operators
    they read from: views of parameters, constants, size arithmetic) out of the traced FX graph, feeds it
    random tensors of the right shapes with the batch dimension scaled to ``batch``, and runs forward +
    backward ``profiling_iter`` times after one warm-up.  Returns a ``GraphProfile``: forward / backward device
    time from CUDA events (``*_time`` and ``*_cuda_time``, microseconds), host time to enqueue them
    (``*_cpu_time``; with ``enable_kineto`` the split comes from ``torch.profiler`` instead), the allocator peak
    over the run, the bytes still held after the forward (kept for backward) and the transient remainder.
    Counterpart of GraphProfiler::computeGraph (src/comp/GraphProfiler.cpp:245-415) and of KinetoWrapper
    (src/comp/KinetoWrapper.cpp:9-40).  Measurements are kept in a ``ProfileDB`` (reference file layout)."""

    def __init__(self, tm, device, iters: int = 1, max_bytes: int = 0):
        self.tm = tm
        self.device = device
        self.iters = max(1, int(iters))
        self.db = _core.ProfileDB()
        self.by_name = {n.name: n for n in tm.gm.graph.nodes}
        self.owned = {n.id for n in tm.ir.nodes if n.is_batch or n.is_criterion}
        self.order = {n.name: i for i, n in enumerate(tm.gm.graph.nodes)}
        self.max_bytes = int(max_bytes)
        self.use_kineto = bool(conf("enable_kineto"))
        self.count = 0

    # ---------------------------------------------------------------- graph cutting
    def _cut(self, ids):
        inset = set(ids)
        stack = list(ids)
        while stack:
            n = self.by_name[stack.pop()]
            for a in n.all_input_nodes:
                if a.op == "call_function" and a.name not in inset and a.name not in self.owned:
                    inset.add(a.name)
                    stack.append(a.name)
        g = fx.Graph()
        env, inputs = {}, []

        def arg(a):
            if a.name not in env:
                ph = g.placeholder(a.name)
                ph.meta = dict(a.meta)
                env[a.name] = ph
                inputs.append(a)
            return env[a.name]

        outs = []
        for name in sorted(inset, key=lambda k: self.order[k]):
            src = self.by_name[name]
            for a in src.all_input_nodes:
                if a.name not in env and a.name not in inset:
                    arg(a)
            env[name] = g.node_copy(src, lambda x: env[x.name] if x.name in env else arg(x))
            val = src.meta.get("val")
            if name in self.owned and isinstance(val, torch.Tensor) and val.is_floating_point() and \
                    any(u.name not in inset for u in src.users):
                outs.append(env[name])
        if not outs:
            last = [env[n] for n in sorted(inset, key=lambda k: self.order[k]) if
                    isinstance(self.by_name[n].meta.get("val"), torch.Tensor) and
                    self.by_name[n].meta["val"].is_floating_point()]
            outs = last[-1:]
        g.output(tuple(outs))
        # placeholders first (fx requires it): node_copy appended them in order of first use, which is fine
        # because every placeholder was created before the node that uses it; reorder to the front
        gm = fx.GraphModule(self.tm.gm, _placeholders_first(g))
        return gm, inputs

    def _make_input(self, node, ratio: float):
        val = node.meta.get("val")
        name = node.name
        if isinstance(val, torch.Tensor):
            shp = _shape(val)
            is_param = name in self.tm.params or name in self.tm.buffers or name in self.tm.constants
            if not is_param and shp and self.tm.trace_batch > 0 and shp[0] % self.tm.trace_batch == 0 and \
                    self.tm.ir.has_value(name) and self.tm.ir.value(name).is_batch:
                shp = [max(1, int(round(shp[0] * ratio)))] + shp[1:]
            if val.is_floating_point():
                t = (torch.randn(shp, dtype=val.dtype, device=self.device) * 0.02).requires_grad_(True)
                return _with_main_grad(t) if (name in self.tm.params and self.device.type == "cuda") else t
            return torch.zeros(shp, dtype=val.dtype, device=self.device)
        if isinstance(val, (int, torch.SymInt)):
            h = int(getattr(getattr(val, "node", None), "hint", val)) if not isinstance(val, int) else val
            if self.tm.trace_batch > 0 and not isinstance(val, int) and h % self.tm.trace_batch == 0:
                return max(1, int(round(h * ratio)))
            return h
        return val

    # ---------------------------------------------------------------- measurement
    def measure(self, ids, batch: int, checkpointing: bool = False):
        ids = [i for i in ids if i in self.by_name]
        if not ids:
            return None
        ratio = float(batch) / max(1, self.tm.trace_batch)
        try:
            gm, inputs = self._cut(ids)
            est = sum(_numel_bytes(self.by_name[i].meta.get("val")) for i in ids) * ratio
            if self.max_bytes and est * 3 > self.max_bytes:
                return None
            args = [self._make_input(n, ratio) for n in inputs]
            return self._run(gm, args, checkpointing, "+".join(ids[:2]) + f"..({len(ids)})")
        except torch.OutOfMemoryError:
            torch.cuda.empty_cache()
            return None
        except Exception:  # noqa: BLE001 - a subgraph that cannot run standalone keeps its estimate
            return None

    def _run(self, gm, args, checkpointing: bool, name: str):
        if self.device.type != "cuda":
            return self._run_host(gm, args, checkpointing, name)
        import time

        dev = self.device
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ft = bt = fcpu = bcpu = float("inf")
        peak = kept = 0
        for it in range(max(2, self.iters) + 1):
            for a in args:
                if isinstance(a, torch.Tensor) and a.grad is not None:
                    a.grad = None
            torch.cuda.synchronize(dev)
            torch.cuda.reset_peak_memory_stats(dev)
            base = torch.cuda.memory_allocated(dev)
            t0 = time.perf_counter()
            ev[0].record()
            if checkpointing:
                with torch.no_grad():
                    outs = gm(*args)
                held = torch.cuda.memory_allocated(dev) - base
                outs = gm(*args)      # the recomputation, charged to the backward like the runtime does
                ev[1].record()
                t1 = time.perf_counter()
            else:
                outs = gm(*args)
                ev[1].record()
                t1 = time.perf_counter()
                held = torch.cuda.memory_allocated(dev) - base
            outs = [o for o in (outs if isinstance(outs, (tuple, list)) else (outs,))
                    if isinstance(o, torch.Tensor) and o.requires_grad]
            if outs:
                torch.autograd.backward(outs, [torch.ones_like(o) for o in outs])
            ev[2].record()
            t2 = time.perf_counter()
            torch.cuda.synchronize(dev)
            if it > 0:
                f, b = ev[0].elapsed_time(ev[1]) * 1e3, ev[1].elapsed_time(ev[2]) * 1e3
                if checkpointing:
                    # forward without grad + recomputation were timed together: half is the forward
                    f, b = f / 2, b + f / 2
                # the fastest of the timed runs: allocator warm-up and clock ramps only ever add time
                ft, bt = min(ft, f), min(bt, b)
                fcpu, bcpu = min(fcpu, (t1 - t0) * 1e6), min(bcpu, (t2 - t1) * 1e6)
                peak = max(peak, torch.cuda.max_memory_allocated(dev) - base)
                kept = max(kept, held)
            del outs
        n = 1
        out_bytes = 0
        gp = _core.GraphProfile()
        gp.name = name
        gp.fwd_time, gp.bwd_time = int(ft / n + 0.5), int(bt / n + 0.5)
        gp.fwd_cuda_time, gp.bwd_cuda_time = gp.fwd_time, gp.bwd_time
        gp.fwd_cpu_time, gp.bwd_cpu_time = int(fcpu / n + 0.5), int(bcpu / n + 0.5)
        if self.use_kineto:
            self._kineto_split(gm, args, gp)
        gp.max_allocated_mem = int(peak)
        gp.activation_size = int(max(0, kept - out_bytes))
        gp.working_mem = int(max(0, peak - kept))
        gp.checkpointing = bool(checkpointing)
        self.count += 1
        return gp

    def _run_host(self, gm, args, checkpointing: bool, name: str):
        """Without a CUDA device (CPU ranks): host clock, and the bytes of the tensors the forward returns and
        saves are approximated by the outputs'."""
        import time

        ft = bt = 0.0
        kept = 0
        for it in range(self.iters + 1):
            for a in args:
                if isinstance(a, torch.Tensor) and a.grad is not None:
                    a.grad = None
            t0 = time.perf_counter()
            if checkpointing:
                with torch.no_grad():
                    gm(*args)
            outs = gm(*args)
            t1 = time.perf_counter()
            outs = [o for o in (outs if isinstance(outs, (tuple, list)) else (outs,))
                    if isinstance(o, torch.Tensor) and o.requires_grad]
            kept = sum(o.numel() * o.element_size() for o in outs)
            if outs:
                torch.autograd.backward(outs, [torch.ones_like(o) for o in outs])
            t2 = time.perf_counter()
            if it > 0:
                f, b = (t1 - t0) * 1e6, (t2 - t1) * 1e6
                if checkpointing:
                    f, b = f / 2, b + f / 2
                ft, bt = ft + f, bt + b
        gp = _core.GraphProfile()
        gp.name = name
        gp.fwd_time, gp.bwd_time = max(1, int(ft / self.iters + 0.5)), max(1, int(bt / self.iters + 0.5))
        gp.fwd_cpu_time, gp.bwd_cpu_time = gp.fwd_time, gp.bwd_time
        gp.activation_size = int(kept)
        gp.max_allocated_mem = int(kept)
        gp.checkpointing = bool(checkpointing)
        self.count += 1
        return gp

    def _kineto_split(self, gm, args, gp) -> None:
        """``enable_kineto``: host and device time of one more forward + backward from ``torch.profiler``
        (reference: KinetoWrapper, src/comp/KinetoWrapper.cpp:9-40)."""
        try:
            from torch.profiler import ProfilerActivity, profile

            with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
                outs = gm(*args)
                outs = [o for o in (outs if isinstance(outs, (tuple, list)) else (outs,))
                        if isinstance(o, torch.Tensor) and o.requires_grad]
                if outs:
                    torch.autograd.backward(outs, [torch.ones_like(o) for o in outs])
                torch.cuda.synchronize(self.device)
            cpu = sum(e.self_cpu_time_total for e in prof.key_averages())
            cuda = sum(getattr(e, "self_device_time_total", 0) for e in prof.key_averages())
            total = max(1, gp.fwd_time + gp.bwd_time)
            gp.fwd_cpu_time = int(cpu * gp.fwd_time / total)
            gp.bwd_cpu_time = int(cpu * gp.bwd_time / total)
            gp.fwd_cuda_time = int(cuda * gp.fwd_time / total)
            gp.bwd_cuda_time = int(cuda * gp.bwd_time / total)
        except Exception:  # noqa: BLE001
            pass

    # ---------------------------------------------------------------- calibration of the operator profiles
    def calibrate(self, node_profiles, blocks, batch: int, additive):
        """``blocks``: (block name, operator ids, IRGraph) per block of the coarsened graph.  Each block is
        measured once at micro-batch ``batch``; the operator profiles inside it are scaled so that their sum
        matches the measurement (time forward, time backward, bytes kept for backward).  ``additive(name)``
        returns the (fwd, bwd, activation) sums the current profiles give for the block at that batch.
        Returns (new profiles, list of (block, measured / estimated) for the log)."""
        out = dict(node_profiles)
        report = []
        for name, ids, graph in blocks:
            cached = self.db.get({name: graph}, int(batch), self.iters, False)
            gp = cached.get(name) if cached else None
            if gp is None:
                gp = self.measure(ids, batch, False)
                if gp is None:
                    continue
                self.db.add({name: graph}, int(batch), self.iters, False, {name: gp})
            ef, eb, ea = additive(name)
            rf = gp.fwd_time / ef if ef > 0 and gp.fwd_time > 0 else 1.0
            rb = gp.bwd_time / eb if eb > 0 and gp.bwd_time > 0 else 1.0
            ra = gp.activation_size / ea if ea > 0 and gp.activation_size > 0 else 1.0
            # a single measurement can be off: keep the correction within a factor of four
            rf, rb, ra = (min(4.0, max(0.25, r)) for r in (rf, rb, ra))
            for i in ids:
                p = out.get(i)
                if p is None:
                    continue
                out[i] = _core.NodeProfile(p.fwd_us * rf, p.bwd_us * rb, int(p.activation_bytes * ra),
                                           p.working_bytes, p.scales_with_batch)
            report.append((name, len(ids), rf, rb, ra))
        return out, report


def _placeholders_first(g: fx.Graph) -> fx.Graph:
    """A copy of ``g`` with its placeholders moved in front of every other node."""
    out = fx.Graph()
    env = {}
    for n in g.nodes:
        if n.op == "placeholder":
            env[n] = out.placeholder(n.name)
            env[n].meta = dict(n.meta)
    for n in g.nodes:
        if n.op == "placeholder":
            continue
        if n.op == "output":
            out.output(torch.fx.node.map_arg(n.args[0], lambda x: env[x]))
        else:
            env[n] = out.node_copy(n, lambda x: env[x])
    out.lint()
    return out
