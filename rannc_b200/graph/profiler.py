"""Per-operator profiles for the partitioner's cost model.

Two modes:

* analytic (default, needs no GPU): a roofline estimate from shapes -- FLOPs
  over the sustained tensor-core rate and bytes over the copy bandwidth, both
  taken from the configuration (defaults are the rates measured on B200);
* measured (``measure_profiles``): every operator of the rewritten graph is
  timed on the device with CUDA events, forward and backward, on fake-shaped
  random inputs -- the counterpart of the reference's GraphProfiler
  (src/comp/GraphProfiler.cpp:245-415), but per operator instead of per
  candidate subgraph, and on the device clock instead of the host's.
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


def measured_profiles(gm: fx.GraphModule, device, iters: int = 3) -> Dict[str, "_core.NodeProfile"]:
    """Times every call_function node on ``device`` with CUDA events (forward and backward)."""
    base = analytic_profiles(gm)
    if not torch.cuda.is_available():
        return base
    from .tracer import op_name

    def real(v):
        if isinstance(v, torch.Tensor):
            shp = _shape(v)
            if v.is_floating_point():
                return torch.randn(shp, dtype=v.dtype, device=device).requires_grad_(True)
            return torch.zeros(shp, dtype=v.dtype, device=device)
        return v

    for n in gm.graph.nodes:
        if n.op != "call_function" or op_name(n.target) in _VIEW_OPS:
            continue
        try:
            def conv(a):
                if isinstance(a, fx.Node):
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


def save_profiles(path: str, profiles: Dict[str, "_core.NodeProfile"], batch: int) -> None:
    """Writes the operator profiles (msgpack: batch size, then per node id the five profile fields).  Counterpart
    of the reference's profile dump (src/comp/GraphProfiler.cpp, ``save_graph_profile``): a later run with
    ``load_graph_profile`` plans from the file instead of profiling again."""
    body = {k: [float(p.fwd_us), float(p.bwd_us), int(p.activation_bytes), int(p.working_bytes),
                bool(p.scales_with_batch)] for k, p in profiles.items()}
    with open(path, "wb") as f:
        f.write(_core.msgpack_pack({"batch": int(batch), "nodes": body}))


def load_profiles(path: str, node_ids, batch: int) -> Dict[str, "_core.NodeProfile"]:
    """Reads a file written by ``save_profiles``.  It must cover exactly the nodes of the traced graph and have
    been taken at the same batch size; anything else means it belongs to another model or configuration."""
    with open(path, "rb") as f:
        raw = _core.msgpack_unpack(f.read())
    if int(raw["batch"]) != int(batch):
        raise RuntimeError(f"profile file {path} was taken at batch {raw['batch']}, this run traces batch {batch}")
    nodes = raw["nodes"]
    want = set(node_ids)
    if set(nodes) != want:
        missing = sorted(want - set(nodes))[:5]
        raise RuntimeError(f"profile file {path} does not match the traced graph (e.g. missing {missing})")
    return {k: _core.NodeProfile(v[0], v[1], int(v[2]), int(v[3]), bool(v[4])) for k, v in nodes.items()}
