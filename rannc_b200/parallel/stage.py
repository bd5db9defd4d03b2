"""Stage executor: runs one pipeline stage's graph forward and backward.

Counterpart of the reference's TorchDriver (src/torch/TorchDriver.cpp:378-847):
a stage is the sub-graph of the exported model that the partitioner assigned to
a set of ranks, materialised as an ``fx.GraphModule`` whose placeholders are the
stage's batch inputs followed by its parameters.  Forward keeps what backward
needs per micro-batch; with activation checkpointing it keeps only the stage
inputs and the dropout counter and recomputes in backward
(reference: src/comp/GraphConnector.cpp:395-457,518-599).  Values stay on the
device between micro-batches; nothing is staged through host memory.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.fx as fx

from .. import _core
from ..ops import functional as RF
from ..utils.config import conf

aten = torch.ops.aten


def build_stage_module(traced_gm: fx.GraphModule, sub_ir) -> fx.GraphModule:
    g = fx.Graph()
    env: Dict[str, fx.Node] = {}
    by_name = {n.name: n for n in traced_gm.graph.nodes}
    for name in sub_ir.input_names:
        ph = g.placeholder(name)
        src = by_name.get(name)
        if src is not None:
            ph.meta = dict(src.meta)
        env[name] = ph
    for irn in sub_ir.nodes:
        src = by_name[irn.id]
        env[src.name] = g.node_copy(src, lambda x: env[x.name])
    g.output(tuple(env[o] for o in sub_ir.output_names))
    g.lint()
    return fx.GraphModule(traced_gm, g)


def set_dropout(gm: fx.GraphModule, enabled: bool) -> None:
    """Flips every dropout site of a stage graph (reference: ConvertGraph.cpp:469-484)."""
    for n in gm.graph.nodes:
        if n.op != "call_function":
            continue
        if n.target is aten.dropout.default or n.target is RF.dropout:
            a = list(n.args)
            a[2] = bool(enabled)
            n.args = tuple(a)
        elif n.target is RF.dropout_add_layer_norm:
            a = list(n.args)
            a[6] = bool(enabled)
            n.args = tuple(a)
        elif n.target is RF.qkv_attention:
            a = list(n.args)
            if "orig_p" not in n.meta:
                n.meta["orig_p"] = a[8]
            a[8] = n.meta["orig_p"] if enabled else 0.0
            n.args = tuple(a)
        elif n.target is RF.sdpa or n.target is aten.scaled_dot_product_attention.default:
            a = list(n.args)
            if "orig_p" not in n.meta:
                n.meta["orig_p"] = a[4] if len(a) > 4 else n.kwargs.get("dropout_p", 0.0)
            if len(a) > 4:
                a[4] = n.meta["orig_p"] if enabled else 0.0
                n.args = tuple(a)
            else:
                kw = dict(n.kwargs)
                kw["dropout_p"] = n.meta["orig_p"] if enabled else 0.0
                n.kwargs = kw
    gm.recompile()


class _Saved:
    __slots__ = ("inputs", "outputs", "rng", "check")

    def __init__(self, inputs, outputs, rng):
        self.inputs, self.outputs, self.rng = inputs, outputs, rng
        self.check = None


class StageExec:
    def __init__(self, name: str, gm: fx.GraphModule, sub_ir, params: Dict[str, torch.Tensor]):
        self.name = name
        self.gm = gm
        self.input_names: List[str] = list(sub_ir.input_names)
        self.output_names: List[str] = list(sub_ir.output_names)
        self.param_names = [n for n in self.input_names if sub_ir.value(n).is_param]
        self.batch_input_names = [n for n in self.input_names if not sub_ir.value(n).is_param]
        self.params = params  # placeholder name -> tensor (parameter, buffer or constant)
        self.saved: Dict[int, _Saved] = {}
        self.keep_graph = False

    # ---------------------------------------------------------------- forward
    def _args(self, inputs: Dict[str, torch.Tensor], with_grad: bool):
        args, leaf = [], {}
        for n in self.input_names:
            if n in self.params:
                args.append(self.params[n])
                continue
            t = inputs[n]
            if isinstance(t, torch.Tensor):
                t = t.detach()
                if with_grad and t.is_floating_point():
                    t.requires_grad_(True)
                leaf[n] = t
            args.append(t)
        return args, leaf

    def forward(self, split: int, inputs: Dict[str, torch.Tensor], checkpointing: bool,
                grad_enabled: bool = True) -> Dict[str, torch.Tensor]:
        rng_state = RF.rng.get_state()
        torch_rng = None
        if checkpointing and grad_enabled:
            torch_rng = (torch.get_rng_state(), torch.cuda.get_rng_state() if torch.cuda.is_available() else None)
            args, leaf = self._args(inputs, False)
            with torch.no_grad():
                outs = self.gm(*args)
            self.saved[split] = _Saved(leaf, None, (rng_state, torch_rng))
            if bool(conf("verify_recomp")):
                # self check: the recomputation in backward must reproduce these values
                # (reference: GraphConnector.cpp:446-451,577-594)
                self.saved[split].check = [o.detach().clone() if isinstance(o, torch.Tensor) else None for o in outs]
        elif grad_enabled:
            args, leaf = self._args(inputs, True)
            outs = self.gm(*args)
            self.saved[split] = _Saved(leaf, dict(zip(self.output_names, outs)), None)
        else:
            args, _ = self._args(inputs, False)
            with torch.no_grad():
                outs = self.gm(*args)
        return {n: (o.detach() if isinstance(o, torch.Tensor) else o) for n, o in zip(self.output_names, outs)}

    # ---------------------------------------------------------------- backward
    def backward(self, split: int, out_grads: Dict[str, Optional[torch.Tensor]]) -> Dict[str, torch.Tensor]:
        sv = self.saved.pop(split) if not self.keep_graph else self.saved[split]
        if sv.outputs is None:
            # recompute with the dropout counters the original forward saw
            rf_state, torch_state = sv.rng
            cur_rf = RF.rng.get_state()
            cur_cpu = torch.get_rng_state()
            cur_cuda = torch.cuda.get_rng_state() if torch.cuda.is_available() else None
            RF.rng.set_state(rf_state)
            torch.set_rng_state(torch_state[0])
            if torch_state[1] is not None:
                torch.cuda.set_rng_state(torch_state[1])
            # backward of an autograd Function runs with grad mode off
            with torch.enable_grad():
                args, leaf = self._args(sv.inputs, True)
                outs = dict(zip(self.output_names, self.gm(*args)))
            chk = getattr(sv, "check", None)
            if chk is not None:
                for n, want in zip(self.output_names, chk):
                    got = outs[n]
                    if want is not None and not torch.allclose(got.detach().float(), want.float(), rtol=1e-3,
                                                                atol=1e-3 * float(want.float().abs().max() + 1e-6)):
                        raise RuntimeError(f"verify_recomp: recomputed value {n} of stage {self.name} differs from "
                                           f"the one computed in the forward pass")
            RF.rng.set_state(cur_rf)
            torch.set_rng_state(cur_cpu)
            if cur_cuda is not None:
                torch.cuda.set_rng_state(cur_cuda)
        else:
            leaf, outs = sv.inputs, sv.outputs
        tensors, grads = [], []
        for n in self.output_names:
            o, g = outs[n], out_grads.get(n)
            if g is None or not isinstance(o, torch.Tensor) or not o.requires_grad:
                continue
            tensors.append(o)
            grads.append(g.to(o.dtype) if g.dtype != o.dtype else g)
        if tensors:
            torch.autograd.backward(tensors, grads, retain_graph=self.keep_graph)
        res = {}
        for n, t in leaf.items():
            if isinstance(t, torch.Tensor) and t.grad is not None:
                res[n] = t.grad
                t.grad = None
        return res

    def clear(self):
        self.saved.clear()
