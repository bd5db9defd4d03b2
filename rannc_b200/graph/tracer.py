"""Model -> aten-level FX graph -> partitioner IR.

The reference re-implements ``torch.jit.trace`` so that parameters and buffers
become graph inputs after the real inputs, traces at batch size 2 and then runs
every operator once to learn shapes (src/bind/Tracer.cpp:276-463,
src/comp/GraphProfiler.cpp:792-920).  Here ``torch.export`` does all of that
with fake tensors: parameters and buffers are lifted to placeholders, shapes
come from ``node.meta['val']`` and the batch dimension is exported as a symbol,
so the same graph runs at every micro-batch size.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.fx as fx
from torch.export import Dim
from torch.export.graph_signature import InputKind, OutputKind

from .. import _core
from ..utils.config import conf

logger = logging.getLogger("rannc")

_ELEM = {
    torch.float32: _core.IRTensorElemType.FLOAT,
    torch.float64: _core.IRTensorElemType.DOUBLE,
    torch.float16: _core.IRTensorElemType.HALF,
    torch.bfloat16: _core.IRTensorElemType.BFLOAT16,
    torch.int32: _core.IRTensorElemType.INT,
    torch.int64: _core.IRTensorElemType.LONG,
    torch.bool: _core.IRTensorElemType.BOOL,
    torch.int8: _core.IRTensorElemType.INT,
    torch.uint8: _core.IRTensorElemType.INT,
    torch.int16: _core.IRTensorElemType.INT,
}


def _hint(d) -> int:
    if isinstance(d, int):
        return d
    node = getattr(d, "node", None)
    if node is not None:
        h = getattr(node, "hint", None)
        if h is not None:
            return int(h)
    return int(d)


def ir_type_of(val, requires_grad: bool = False):
    """IR type of a fake value found in ``node.meta['val']``."""
    if isinstance(val, torch.Tensor):
        elem = _ELEM.get(val.dtype, _core.IRTensorElemType.UNDEF)
        return _core.IRType.tensor(elem, [_hint(d) for d in val.shape], bool(requires_grad or val.requires_grad))
    if isinstance(val, (list, tuple)):
        return _core.IRType.tuple([ir_type_of(v) for v in val])
    if isinstance(val, bool):
        return _core.IRType.scalar(_core.IRScalarType.BOOL)
    if isinstance(val, (int, torch.SymInt)):
        return _core.IRType.scalar(_core.IRScalarType.INT)
    if isinstance(val, (float, torch.SymFloat)):
        return _core.IRType.scalar(_core.IRScalarType.FLOAT)
    return _core.IRType.none()


def op_name(target) -> str:
    """TorchScript-style operator name, e.g. ``aten::linear`` or ``rannc::mlp``."""
    if isinstance(target, torch._ops.OpOverload):
        ns, name = target._schema.name.split("::")
        return f"{ns}::{name}"
    mod = getattr(target, "__module__", "") or ""
    nm = getattr(target, "__name__", str(target))
    if mod.startswith("rannc_b200"):
        return f"rannc::{nm}"
    if mod in ("_operator", "operator"):
        return f"prim::{nm}"
    return f"{mod}::{nm}" if mod else nm


@dataclass
class TracedModel:
    gm: fx.GraphModule                      # aten-level graph; placeholders = params, buffers, user inputs
    ir: Any                                 # _core.IRGraph, batch size = the traced local batch
    user_inputs: List[str]                  # placeholder names in call order
    params: Dict[str, str]                  # placeholder name -> parameter fqn
    buffers: Dict[str, str]                 # placeholder name -> buffer fqn
    constants: Dict[str, torch.Tensor]      # placeholder name -> lifted constant tensor
    user_outputs: List[str]                 # names of output nodes the caller receives
    buffer_mutations: Dict[str, str]        # output node name -> buffer fqn to copy it into
    out_spec: Any = None                    # pytree spec of the model's return value
    dynamic_batch: bool = True
    rewrite_stats: Dict[str, int] = field(default_factory=dict)
    trace_batch: int = 0
    dim_names: Dict[str, List[str]] = field(default_factory=dict)   # use_named_tensors: value -> name per dim


def _flatten_args_keep_none(args) -> list:
    """Leaves of an output structure in order; constants appear as None."""
    out = []

    def rec(a):
        if isinstance(a, (list, tuple)):
            for x in a:
                rec(x)
        elif isinstance(a, dict):
            for x in a.values():
                rec(x)
        else:
            out.append(a if isinstance(a, fx.Node) else None)

    rec(args)
    return out


def _flatten_args(args) -> List[fx.Node]:
    out = []

    def rec(a):
        if isinstance(a, fx.Node):
            out.append(a)
        elif isinstance(a, (list, tuple)):
            for x in a:
                rec(x)
        elif isinstance(a, dict):
            for x in a.values():
                rec(x)

    rec(args)
    return out


def export_model(model: torch.nn.Module, args: Tuple[torch.Tensor, ...], dynamic_batch: bool = True):
    """``torch.export`` with dim 0 of every tensor input as one shared symbol (when it can be)."""
    if dynamic_batch:
        sizes = {a.shape[0] for a in args if isinstance(a, torch.Tensor) and a.dim() > 0}
        if len(sizes) == 1 and next(iter(sizes)) >= 2:
            b = Dim("batch", min=1, max=1 << 30)
            ds = tuple(({0: b} if isinstance(a, torch.Tensor) and a.dim() > 0 else None) for a in args)
            try:
                return torch.export.export(model, tuple(args), dynamic_shapes=ds, strict=False), True
            except Exception as e:  # noqa: BLE001
                logger.warning("export with a symbolic batch dimension failed (%s); exporting with static shapes",
                               str(e).splitlines()[0] if str(e) else type(e).__name__)
    return torch.export.export(model, tuple(args), strict=False), False


def _batch_hint(val, dynamic_batch: bool) -> int:
    """+1 if a dimension of the fake tensor is symbolic (derived from the batch symbol), -1 if none is and the
    tensor is not 0-dim (scalars are left to the loss rule), 0 when the trace has no symbolic batch."""
    if not dynamic_batch or not isinstance(val, torch.Tensor) or val.dim() == 0:
        return 0
    return 1 if any(not isinstance(d, int) for d in val.shape) else -1


def trace_dim_names(gm: fx.GraphModule) -> Dict[str, List[str]]:
    """Name of every dimension of every tensor value of a trace made with a symbolic batch: ``"N"`` where the
    extent derives from the batch symbol, ``<value>_D<i>`` otherwise.

    The reference learns the same thing by running every node once on named tensors and reading the names that
    come out (``use_named_tensors``; src/comp/GraphProfiler.cpp:135-243, names built as in ``createDimnames``
    :149-170); here the symbolic shapes ``torch.export`` attaches to each node already carry it, so nothing
    is executed."""
    import re

    out: Dict[str, List[str]] = {}
    for n in gm.graph.nodes:
        val = n.meta.get("val")
        if not isinstance(val, torch.Tensor):
            continue
        base = re.sub(r"_+", "_", re.sub(r"[_:\[\]\.]+", "_", n.name))
        out[n.name] = ["N" if not isinstance(d, int) else f"{base}_D{i}" for i, d in enumerate(val.shape)]
    return out


def fx_to_ir(gm: fx.GraphModule, name: str, param_placeholders, user_inputs, batch_size: int,
             dynamic_batch: bool = False):
    """Builds the IRGraph: real inputs first, then parameters / buffers / constants."""
    g = _core.IRGraph()
    g.name = name
    g.batch_size = int(batch_size)
    placeholders = {n.name: n for n in gm.graph.nodes if n.op == "placeholder"}
    order = list(user_inputs) + [p for p in placeholders if p not in set(user_inputs)]
    for pname in order:
        n = placeholders[pname]
        is_param = pname in param_placeholders
        val = n.meta.get("val")
        t = ir_type_of(val, requires_grad=is_param and isinstance(val, torch.Tensor) and val.is_floating_point())
        v = _core.IRValue(pname, t, is_param)
        g.add_input(v)
    for n in gm.graph.nodes:
        if n.op == "call_function":
            ins, seen = [], set()
            for a in _flatten_args((n.args, n.kwargs)):
                if a.name not in seen:
                    seen.add(a.name)
                    ins.append(a.name)
            v = _core.IRValue(n.name, ir_type_of(n.meta.get("val")), False)
            v.batch_hint = _batch_hint(n.meta.get("val"), dynamic_batch)
            g.add_value(v)
            g.add_node(_core.IRNode(op_name(n.target), ins, [n.name], n.name))
        elif n.op == "get_attr":
            g.add_input(_core.IRValue(n.name, ir_type_of(n.meta.get("val")), True))
        elif n.op == "output":
            for a in _flatten_args(n.args):
                if a.name not in g.output_names:
                    g.add_output(a.name)
    g.check()
    return _core.guess_value_types(g)


def _materialise_passthrough(gm: fx.GraphModule) -> None:
    """An output that IS a model input (``forward(x): return x``) has no producing operator, so no stage would
    own it and a model made only of such outputs would have an empty graph.  Each one gets an ``aten.alias``
    node: a view, free at run time, that the planner can place like any other operator.  (The reference's
    test zoo has such a model: test/models.py, IdentityModel.)"""
    out_node = next(n for n in gm.graph.nodes if n.op == "output")
    made = {}

    def rec(a):
        if isinstance(a, fx.Node) and a.op == "placeholder":
            if a not in made:
                with gm.graph.inserting_before(out_node):
                    al = gm.graph.call_function(torch.ops.aten.alias.default, (a,))
                al.meta = dict(a.meta)
                made[a] = al
            return made[a]
        if isinstance(a, (tuple, list)):
            return type(a)(rec(x) for x in a)
        if isinstance(a, dict):
            return {k: rec(v) for k, v in a.items()}
        return a

    new_args = rec(out_node.args)
    if made:
        out_node.args = new_args
        gm.recompile()


def trace(model: torch.nn.Module, args: Tuple[torch.Tensor, ...], use_kernels: bool = False,
          name: str = "model") -> TracedModel:
    ep, dyn = export_model(model, args)
    gm = ep.graph_module
    sig = ep.graph_signature
    params, buffers, constants, user_inputs = {}, {}, {}, []
    for spec in sig.input_specs:
        nm = getattr(spec.arg, "name", None)
        if nm is None:
            continue
        if spec.kind == InputKind.PARAMETER:
            params[nm] = spec.target
        elif spec.kind == InputKind.BUFFER:
            buffers[nm] = spec.target
        elif spec.kind == InputKind.USER_INPUT:
            user_inputs.append(nm)
        elif spec.kind in (InputKind.CONSTANT_TENSOR, InputKind.CUSTOM_OBJ):
            constants[nm] = ep.constants[spec.target]
    user_outputs, buffer_mutations = [], {}
    for spec in sig.output_specs:
        nm = getattr(spec.arg, "name", None)
        if spec.kind == OutputKind.USER_OUTPUT:
            user_outputs.append(nm)
        elif spec.kind == OutputKind.BUFFER_MUTATION:
            buffer_mutations[nm] = spec.target
    stats = {}
    if use_kernels:
        from . import rewrite

        # linear layers that will run tensor-partitioned stay nodes of their own: all of them under
        # force_dist_matmul, and under keep_dist_params_sharded when the model was declared in shards
        keep = bool(conf("force_dist_matmul"))
        if not keep and bool(conf("keep_dist_params_sharded")):
            from .. import dist_param as _dp

            keep = any(_dp.dist_param_registered(id(p)) for p in model.parameters())
        stats = rewrite.fuse(gm, training=model.training, keep_linear=keep)
    else:
        from . import rewrite

        rewrite.drop_asserts(gm)
        rewrite.anchor_mutations(gm)
        gm.graph.eliminate_dead_code()
        gm.recompile()
    _materialise_passthrough(gm)
    # the rewrites may have replaced the nodes that produce the outputs: take the names from the graph
    out_node = next(n for n in gm.graph.nodes if n.op == "output")
    flat_out = _flatten_args_keep_none(out_node.args)
    if len(flat_out) == len(sig.output_specs):
        user_outputs, buffer_mutations = [], {}
        for spec, node in zip(sig.output_specs, flat_out):
            if node is None:
                continue
            if spec.kind == OutputKind.USER_OUTPUT:
                user_outputs.append(node.name)
            elif spec.kind == OutputKind.BUFFER_MUTATION:
                buffer_mutations[node.name] = spec.target
    batch = 0
    for a in args:
        if isinstance(a, torch.Tensor) and a.dim() > 0:
            batch = int(a.shape[0])
            break
    param_like = set(params) | set(buffers) | set(constants)
    ir = fx_to_ir(gm, name, param_like, user_inputs, batch, dynamic_batch=bool(dyn))
    out_spec = getattr(ep.module_call_graph[0].signature, "out_spec", None) if ep.module_call_graph else None
    names: Dict[str, List[str]] = {}
    if dyn and bool(conf("use_named_tensors")):
        names = trace_dim_names(gm)
        off0 = [v for v, dn in names.items() if "N" in dn[1:] and v not in param_like]
        if off0:
            # micro-batches and replicas split dimension 0; a value that carries the batch elsewhere still
            # works (it is produced and consumed inside one stage or moved whole) but is worth knowing about
            logger.info("values whose batch dimension is not the first one: %s", ", ".join(off0[:8]))
    return TracedModel(gm=gm, ir=ir, user_inputs=user_inputs, params=params, buffers=buffers, constants=constants,
                       user_outputs=user_outputs, buffer_mutations=buffer_mutations, out_spec=out_spec,
                       dynamic_batch=dyn, rewrite_stats=stats, trace_batch=batch, dim_names=names)
