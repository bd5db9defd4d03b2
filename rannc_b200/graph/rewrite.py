"""Graph pass that swaps ATen nodes of an exported model for the fused sm_100a operators.

Runs on the aten-level FX graph produced by ``torch.export`` before it is turned
into the partitioner's IR, so the cost model and the stages see fused operators.
Patterns (all guarded; an unmatched node simply stays an ATen call):

* ``linear`` -> tcgen05 GEMM; ``gelu(linear)`` -> GEMM with GELU epilogue;
  ``linear(gelu(linear))`` -> one MLP operator whose backward folds the GELU
  derivative into the dgrad GEMM epilogue;
* ``layer_norm(add(dropout(y), r))`` (any operand order, dropout/add optional)
  -> one fused dropout + residual + LayerNorm kernel;
* ``scaled_dot_product_attention`` -> fused flash attention;
* ``cross_entropy_loss(float(reshape(slice(logits))))`` -> fused softmax
  cross-entropy reading the 16-bit logits once;
* stand-alone ``dropout`` / ``gelu`` / ``embedding``.

The reference has no such pass: it runs the traced TorchScript graph node by
node (src/torch/TorchDriver.cpp:566).
"""
from __future__ import annotations

import operator

import torch
import torch.fx as fx

from ..ops import functional as RF

aten = torch.ops.aten

_DROP_TARGETS = set()
for _name in ("_assert_tensor_metadata", "_assert_scalar", "sym_constrain_range_for_size", "sym_constrain_range",
              "_assert_async"):
    _op = getattr(aten, _name, None)
    if _op is not None:
        for _ov in _op.overloads():
            _DROP_TARGETS.add(getattr(_op, _ov))


def _users(n: fx.Node):
    return list(n.users.keys())


def _single_user(n: fx.Node):
    u = _users(n)
    return u[0] if len(u) == 1 else None


def _is(n, *targets) -> bool:
    return isinstance(n, fx.Node) and n.op == "call_function" and n.target in targets


def _val(n):
    return n.meta.get("val") if isinstance(n, fx.Node) else None


def _arg(n: fx.Node, i: int, name: str, default=None):
    if len(n.args) > i:
        return n.args[i]
    return n.kwargs.get(name, default)


def drop_asserts(gm: fx.GraphModule) -> int:
    k = 0
    for n in list(gm.graph.nodes):
        if n.op == "call_function" and n.target in _DROP_TARGETS and not n.users:
            gm.graph.erase_node(n)
            k += 1
    return k


def after_effects(effects, value):
    """Identity on ``value``; ``effects`` are the results of in-place updates that must run with it."""
    return value


def anchor_mutations(gm: fx.GraphModule) -> int:
    """An in-place update whose result nothing reads (``num_batches_tracked.add_(1)`` of BatchNorm) would
    belong to no stage, because stages are cut along data dependencies.  Each such node is tied to the next
    node that produces a used tensor from the same module call: that node's result is routed through
    ``after_effects(update, result)``, so the update travels with its consumer's stage."""
    pending, k = [], 0
    for n in list(gm.graph.nodes):
        if n.op != "call_function":
            continue
        tgt = n.target
        inplace = isinstance(tgt, torch._ops.OpOverload) and tgt._schema.name.endswith("_") and tgt._schema.is_mutable
        if inplace and not n.users:
            pending.append(n)
            continue
        val = n.meta.get("val")
        if pending and n.users and isinstance(val, torch.Tensor) and val.is_floating_point():
            users = list(n.users)
            with gm.graph.inserting_after(n):
                tie = gm.graph.call_function(after_effects, (tuple(pending), n))
            tie.meta = dict(n.meta)
            for u in users:
                u.replace_input_with(n, tie)
            k += len(pending)
            pending = []
    return k


def _replace(gm, old: fx.Node, fn, args, kwargs=None):
    with gm.graph.inserting_before(old):
        new = gm.graph.call_function(fn, tuple(args), kwargs or {})
    new.meta = dict(old.meta)
    old.replace_all_uses_with(new)
    gm.graph.erase_node(old)
    return new


def _erase_if_dead(gm, *nodes):
    for n in nodes:
        if isinstance(n, fx.Node) and not n.users and n.op == "call_function":
            gm.graph.erase_node(n)


def fuse(gm: fx.GraphModule, training: bool = True, keep_linear: bool = False) -> dict:
    """Rewrites ``gm`` in place; returns a count of each rewrite applied.  With ``keep_linear`` every
    ``linear`` stays a node of its own (no q/k/v or MLP fusion), so that it can be turned into a
    tensor-partitioned linear once the replica sets are known."""
    stats = {}

    def bump(k):
        stats[k] = stats.get(k, 0) + 1

    drop_asserts(gm)
    g = gm.graph

    # ---- q/k/v projections of one input + attention -> one operator
    def _proj(node):
        """transpose(view(linear(x, w, b), [B, S, H, D]), 1, 2) -> (linear node, H) or None"""
        if not _is(node, aten.transpose.int) or sorted(node.args[1:3]) != [1, 2] or len(_users(node)) != 1:
            return None
        v = node.args[0]
        if not _is(v, aten.view.default, aten.reshape.default) or len(_users(v)) != 1 or len(v.args[1]) != 4:
            return None
        lin = v.args[0]
        if not _is(lin, aten.linear.default) or len(_users(lin)) != 1:
            return None
        heads = v.args[1][2]
        return (lin, v, int(heads)) if isinstance(heads, int) else None

    for n in list(g.nodes):
        if keep_linear or not _is(n, aten.scaled_dot_product_attention.default):
            continue
        pq, pk, pv = (_proj(a) for a in n.args[:3])
        if pq is None or pk is None or pv is None:
            continue
        x = pq[0].args[0]
        if pk[0].args[0] is not x or pv[0].args[0] is not x or not (pq[2] == pk[2] == pv[2]):
            continue
        xv = _val(x)
        if xv is None or xv.dim() != 3:
            continue
        u = _single_user(n)
        if u is None or not _is(u, aten.transpose.int) or sorted(u.args[1:3]) != [1, 2]:
            continue
        u2 = _single_user(u)
        if u2 is None or not _is(u2, aten.reshape.default, aten.view.default, aten._unsafe_view.default) or \
                len(u2.args[1]) != 3:
            continue
        mask = _arg(n, 3, "attn_mask")
        pdrop = _arg(n, 4, "dropout_p", 0.0)
        causal = _arg(n, 5, "is_causal", False)
        scale = n.kwargs.get("scale")
        args = (x, pq[0].args[1], _arg(pq[0], 2, "bias"), pk[0].args[1], _arg(pk[0], 2, "bias"),
                pv[0].args[1], _arg(pv[0], 2, "bias"), mask, pdrop, causal, scale, pq[2])
        _replace(gm, u2, RF.qkv_attention, args)
        _erase_if_dead(gm, u, n)
        bump("qkv_attention")
    g.eliminate_dead_code()

    # ---- linear -> gelu -> linear  /  linear -> gelu
    for n in list(g.nodes):
        if keep_linear or not _is(n, aten.linear.default) or n not in g.nodes:
            continue
        u = _single_user(n)
        if u is not None and _is(u, aten.gelu.default) and u.kwargs.get("approximate", "none") == "none":
            u2 = _single_user(u)
            if u2 is not None and _is(u2, aten.linear.default) and u2.args[0] is u:
                x, w1, b1 = n.args[0], n.args[1], _arg(n, 2, "bias")
                w2, b2 = u2.args[1], _arg(u2, 2, "bias")
                _replace(gm, u2, RF.mlp, (x, w1, b1, w2, b2))
                _erase_if_dead(gm, u, n)
                bump("mlp")
                continue
            x, w, b = n.args[0], n.args[1], _arg(n, 2, "bias")
            _replace(gm, u, RF.linear, (x, w, b, "gelu"))
            _erase_if_dead(gm, n)
            bump("linear_gelu")
    for n in list(g.nodes):
        if _is(n, aten.linear.default):
            _replace(gm, n, RF.linear, (n.args[0], n.args[1], _arg(n, 2, "bias")))
            bump("linear")

    # ---- layer_norm(add(dropout(y), r))
    for n in list(g.nodes):
        if not _is(n, aten.layer_norm.default):
            continue
        x, shape, gamma, beta = n.args[0], n.args[1], _arg(n, 2, "weight"), _arg(n, 3, "bias")
        eps = _arg(n, 4, "eps", 1e-5)
        if gamma is None or beta is None or len(shape) != 1:
            continue
        y, res, p = x, None, 0.0
        dead = []
        if _is(x, aten.add.Tensor) and len(_users(x)) == 1 and isinstance(x.args[1], fx.Node) and \
                _arg(x, 2, "alpha", 1) == 1:
            a, b = x.args[0], x.args[1]
            va, vb = _val(a), _val(b)
            if va is not None and vb is not None and tuple(va.shape) == tuple(vb.shape):
                if _is(b, aten.dropout.default) and len(_users(b)) == 1 and not _is(a, aten.dropout.default):
                    a, b = b, a
                y, res = a, b
                dead.append(x)
        if _is(y, aten.dropout.default) and len(_users(y)) == 1:
            if y.args[2]:
                p = float(y.args[1])
            dead.append(y)
            y = y.args[0]
        _replace(gm, n, RF.dropout_add_layer_norm, (y, res, gamma, beta, p, eps, training))
        _erase_if_dead(gm, *dead)
        bump("dropout_add_ln" if res is not None or p > 0 else "layer_norm")

    # ---- attention
    for n in list(g.nodes):
        if _is(n, aten.scaled_dot_product_attention.default):
            q, k, v = n.args[:3]
            mask = _arg(n, 3, "attn_mask")
            p = _arg(n, 4, "dropout_p", 0.0)
            causal = _arg(n, 5, "is_causal", False)
            scale = n.kwargs.get("scale")
            _replace(gm, n, RF.sdpa, (q, k, v, mask, p, causal, scale))
            bump("sdpa")

    # ---- cross entropy over (possibly sliced / reshaped / up-cast) logits
    for n in list(g.nodes):
        if not _is(n, aten.cross_entropy_loss.default):
            continue
        logits, labels = n.args[0], n.args[1]
        weight = _arg(n, 2, "weight")
        reduction = _arg(n, 3, "reduction", 1)
        ignore_index = _arg(n, 4, "ignore_index", -100)
        smoothing = _arg(n, 5, "label_smoothing", 0.0)
        if weight is not None or reduction != 1 or smoothing != 0.0:
            continue
        base, chain = logits, []
        num_classes = None
        while isinstance(base, fx.Node) and base.op == "call_function" and len(_users(base)) == 1:
            if base.target in (aten.to.dtype, aten._to_copy.default, aten.reshape.default, aten.view.default,
                               aten.contiguous.default, aten.clone.default):
                chain.append(base)
                base = base.args[0]
            elif base.target is aten.slice.Tensor:
                bv = _val(base.args[0])
                dim = _arg(base, 1, "dim", 0)
                start = _arg(base, 2, "start", 0) or 0
                step = _arg(base, 4, "step", 1)
                if bv is None or dim not in (-1, bv.dim() - 1) or start != 0 or step != 1:
                    break
                num_classes = int(_val(base).shape[-1])
                chain.append(base)
                base = base.args[0]
            else:
                break
        bv = _val(base)
        lv = _val(logits)
        if bv is None or lv is None or bv.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            continue
        if num_classes is None:
            num_classes = int(lv.shape[-1])
        if int(lv.shape[-1]) != num_classes:
            continue
        _replace(gm, n, RF.cross_entropy, (base, labels, num_classes, ignore_index))
        for c in chain:
            _erase_if_dead(gm, c)
        bump("cross_entropy")

    # ---- convolution, batch norm (+ residual add) (+ relu)
    for n in list(g.nodes):
        if _is(n, aten.conv2d.default):
            a = list(n.args) + [None] * (7 - len(n.args))
            x, w, b = a[0], a[1], a[2] if a[2] is not None else n.kwargs.get("bias")
            stride = a[3] if a[3] is not None else n.kwargs.get("stride", 1)
            padding = a[4] if a[4] is not None else n.kwargs.get("padding", 0)
            dilation = a[5] if a[5] is not None else n.kwargs.get("dilation", 1)
            groups = a[6] if a[6] is not None else n.kwargs.get("groups", 1)
            if isinstance(padding, str):
                continue
            _replace(gm, n, RF.conv2d, (x, w, b, stride, padding, dilation, groups))
            bump("conv2d")
    for n in list(g.nodes):
        if not _is(n, aten.batch_norm.default) or n not in g.nodes:
            continue
        x, w, b, rm, rv, train, momentum, eps = n.args[:8]
        xv = _val(x)
        if xv is None or xv.dim() != 4 or w is None or b is None or not train:
            continue
        relu, residual, chain = False, None, []
        u = _single_user(n)
        if u is not None and _is(u, aten.add.Tensor) and len(u.args) == 2 and not u.kwargs and \
                all(isinstance(t, fx.Node) for t in u.args):
            other = u.args[1] if u.args[0] is n else u.args[0]
            ov = _val(other)
            u2 = _single_user(u)
            if ov is not None and ov.shape == xv.shape and u2 is not None and _is(u2, aten.relu.default, aten.relu_.default):
                relu, residual, chain = True, other, [u, u2]
        elif u is not None and _is(u, aten.relu.default, aten.relu_.default):
            relu, chain = True, [u]
        args = (x, w, b, rm, rv, bool(train), float(momentum), float(eps), relu, residual)
        if not chain:
            _replace(gm, n, RF.batch_norm_act, args)
        else:
            # the fused node takes the place of the last node of the chain (every operand is defined by then)
            last = chain[-1]
            with g.inserting_before(last):
                new = g.call_function(RF.batch_norm_act, args)
            new.meta = dict(last.meta)
            last.replace_all_uses_with(new)
            for m in reversed(chain):
                g.erase_node(m)
            g.erase_node(n)
        bump("batch_norm_act")

    # ---- stand-alone element-wise ops
    for n in list(g.nodes):
        if _is(n, aten.dropout.default):
            _replace(gm, n, RF.dropout, (n.args[0], float(n.args[1]), bool(n.args[2])))
            bump("dropout")
        elif _is(n, aten.gelu.default) and n.kwargs.get("approximate", "none") == "none":
            _replace(gm, n, RF.gelu, (n.args[0],))
            bump("gelu")
        elif _is(n, aten.embedding.default):
            pad = _arg(n, 2, "padding_idx", -1)
            _replace(gm, n, RF.embedding, (n.args[0], n.args[1], pad))
            bump("embedding")

    # after the fusions, so that a batch norm and the activation behind it are still adjacent above
    anchor_mutations(gm)
    g.eliminate_dead_code()
    g.lint()
    gm.recompile()
    return stats
