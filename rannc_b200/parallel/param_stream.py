"""Parameters streamed from host memory: a stage whose 16-bit parameters do not stay on the device.

``offload_params`` keeps the fp32 master weights and optimizer moments in pinned host memory.  With
``offload_param_window_mb > 0`` the 16-bit parameters and their fp32 gradients live there too, and a stage runs
as a chain of *segments* -- consecutive operators whose parameters fit half the window:

* forward: the segment's parameters are copied to the device (the next segment's copy is already in flight on a
  copy stream), the segment runs without an autograd graph, its inputs are kept, the parameters are dropped;
* backward, last segment first: parameters in again, a zeroed (first micro-batch) or re-loaded (later ones) fp32
  gradient window, the segment is recomputed from its kept inputs with a graph, differentiated, the window goes
  back to the host and everything of the segment leaves the device.

So the device holds two segments' parameters, one segment's gradients, one segment's activations and the kept
inputs at the segment boundaries -- whatever the size of the model.

The reference moves each parameter to the device in a hook in front of its first use and back to the host in a
hook behind its last use, and the other way round in backward (``rannc::offloadingPreHook`` /
``offloadingPostHook``, src/torch/TorchDriver.cpp:318-374, src/torch/CustomOps.h:15-87); its optimizer step
brings all parameters back to the device at once (pyrannc/opt.py:304-312), which this design never needs.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.fx as fx

from ..ops import functional as RF
from ..utils.log import get_logger
from .stage import StageExec

logger = get_logger("ParamStream")


class _Window:
    __slots__ = ("params", "views", "bufs", "ready", "nbytes")

    def __init__(self, params, views, bufs, ready, nbytes):
        self.params, self.views, self.bufs, self.ready, self.nbytes = params, views, bufs, ready, nbytes


def _runs(params):
    """Groups parameters that lie back to back in a host flat buffer: [(group, lo, hi, [(param, offset, numel)])].
    One run is one device allocation and one copy; parameters the storage laid out adjacently (the three
    projection weights of a QKV block) stay adjacent on the device, so the single-GEMM paths keep working."""
    by_group = {}
    for p in params:
        g, o, n = p._rannc_flat
        by_group.setdefault(id(g), (g, []))[1].append((o, n, p))
    out = []
    for g, items in by_group.values():
        items.sort(key=lambda t: t[0])
        cur = None
        for o, n, p in items:
            if cur is not None and 0 <= o - cur[2] < 64:
                cur[2] = o + n
                cur[3].append((p, o, n))
            else:
                cur = [g, o, o + n, [(p, o, n)]]
                out.append(cur)
    return out


class ParamStreamer:
    """Moves streamed parameters and their gradient windows between the host and the device."""

    def __init__(self, device: torch.device):
        self.device = device
        self.cuda = device.type == "cuda"
        self.stream = torch.cuda.Stream(device) if self.cuda else None
        self.last_flush = None
        self.resident = 0          # parameter bytes on the device right now
        self.peak_resident = 0
        self.fetched_bytes = 0     # total host -> device parameter traffic (statistics)

    # ------------------------------------------------------------------ parameters
    def prefetch(self, params: Sequence[torch.nn.Parameter]) -> _Window:
        """Starts the host -> device copies of ``params`` on the copy stream."""
        bufs, views, plist = [], [], []
        nbytes = 0
        if self.cuda:
            # the device blocks come from the compute stream's pool: the copy stream may write them only after
            # everything the compute stream has been given so far (their previous user is among it)
            self.stream.wait_stream(torch.cuda.current_stream())
        for g, lo, hi, items in _runs(params):
            h = g.flat_param[lo:hi]
            d = torch.empty(hi - lo, dtype=h.dtype, device=self.device)
            if self.cuda:
                with torch.cuda.stream(self.stream):
                    d.copy_(h, non_blocking=True)
                d.record_stream(self.stream)
            else:
                d.copy_(h)
            bufs.append(d)
            nbytes += h.numel() * h.element_size()
            for p, o, n in items:
                plist.append(p)
                views.append(d[o - lo:o - lo + n].view(p._rannc_shape))
        ready = None
        if self.cuda:
            ready = torch.cuda.Event()
            ready.record(self.stream)
        self.resident += nbytes
        self.fetched_bytes += nbytes
        self.peak_resident = max(self.peak_resident, self.resident)
        return _Window(plist, views, bufs, ready, nbytes)

    def attach(self, w: _Window) -> None:
        """The parameters of the window become usable on the current stream."""
        if w.ready is not None:
            torch.cuda.current_stream().wait_event(w.ready)
        for p, v in zip(w.params, w.views):
            p.data = v

    def release(self, w: _Window) -> None:
        for p, v in zip(w.params, w.views):
            if p.data.data_ptr() == v.data_ptr():
                p.data = torch.empty(0, dtype=v.dtype, device=self.device)
            p.main_grad = None
            p.grad = None
        self.resident -= w.nbytes
        w.nbytes = 0
        w.bufs, w.views = [], []

    # ------------------------------------------------------------------ gradients
    def open_grads(self, params: Sequence[torch.nn.Parameter]):
        """fp32 gradient windows on the device, laid out like the host buffer; a parameter that already has
        gradients from an earlier micro-batch (or an earlier segment: tied weights) starts from them."""
        self.wait()
        runs = []
        for g, lo, hi, items in _runs(params):
            valid = [p._rannc_grad_valid for p, _, _ in items]
            if all(valid):
                d = g.flat_grad[lo:hi].to(self.device, non_blocking=True)
            else:
                d = torch.zeros(hi - lo, dtype=g.flat_grad.dtype, device=self.device)
                for (p, o, n), ok in zip(items, valid):
                    if ok:
                        d[o - lo:o - lo + n].copy_(g.flat_grad[o:o + n], non_blocking=True)
            for p, o, n in items:
                v = d[o - lo:o - lo + n].view(p._rannc_shape)
                v._rannc_window = True
                p.main_grad = v
                p.grad = None
            runs.append((g, lo, hi, items, d))
        return runs

    def flush_grads(self, runs) -> None:
        """Gradients autograd left in ``p.grad`` join the window, the window goes to the host."""
        from ..ops import kernels as K

        for g, lo, hi, items, d in runs:
            for p, o, n in items:
                mg = p.main_grad
                if p.grad is not None and mg is not None and p.grad.data_ptr() != mg.data_ptr():
                    if p.grad.is_cuda and p.grad.dtype in (torch.float16, torch.bfloat16):
                        K.accum_f32(mg, p.grad.contiguous())
                    else:
                        mg.add_(p.grad.float())
                p.grad = None
                p.main_grad = None
        if self.cuda:
            self.stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.stream):
                for g, lo, hi, items, d in runs:
                    # the padding between two parameters of a run is zero on both sides
                    g.flat_grad[lo:hi].copy_(d, non_blocking=True)
                    d.record_stream(self.stream)
                ev = torch.cuda.Event()
                ev.record(self.stream)
            self.last_flush = ev
        else:
            for g, lo, hi, items, d in runs:
                g.flat_grad[lo:hi].copy_(d)
        for g, lo, hi, items, d in runs:
            for p, _, _ in items:
                p._rannc_grad_valid = True

    def wait(self, host: bool = False) -> None:
        if self.last_flush is None:
            return
        if host:
            self.last_flush.synchronize()
        else:
            torch.cuda.current_stream().wait_event(self.last_flush)


class _Segment:
    __slots__ = ("gm", "inputs", "outputs", "params", "streamed", "nbytes")

    def __init__(self, gm, inputs, outputs, params, streamed, nbytes):
        self.gm = gm                  # fx.GraphModule: placeholders = ``inputs``, output = tuple of ``outputs``
        self.inputs = inputs          # value names, in placeholder order (stage inputs, parameters, earlier values)
        self.outputs = outputs        # value names later segments or the stage's caller need
        self.params = params          # placeholder name -> tensor, for the parameter-like inputs
        self.streamed = streamed      # the streamed Parameters among them (deduplicated)
        self.nbytes = nbytes


def _pbytes(t) -> int:
    h = getattr(t, "_rannc_host", None)
    if h is not None:
        return h.numel() * h.element_size()
    return t.numel() * t.element_size()


def split_into_segments(gm: fx.GraphModule, params: Dict[str, torch.Tensor], max_bytes: int,
                        resident: bool = False) -> List[_Segment]:
    """Cuts a stage graph into consecutive runs of operators whose streamed parameters take at most ``max_bytes``
    (one operator's parameters may exceed it: it then forms a segment of its own).  ``resident``: every
    parameter counts, streamed or not (segments for recomputation only)."""
    nodes = [n for n in gm.graph.nodes if n.op == "call_function"]
    out_node = next(n for n in gm.graph.nodes if n.op == "output")
    stage_outs = [a.name for a in out_node.all_input_nodes]

    def streamed_of(n):
        res = []
        for a in n.all_input_nodes:
            t = params.get(a.name) if a.op == "placeholder" else None
            if t is not None and (hasattr(t, "_rannc_host") or
                                  (resident and isinstance(t, torch.nn.Parameter))):
                res.append((a.name, t))
        return res

    groups: List[List[fx.Node]] = [[]]
    seen: set = set()
    size = 0
    for n in nodes:
        mine = [(nm, t) for nm, t in streamed_of(n) if nm not in seen]
        add = sum(_pbytes(t) for _, t in mine)
        if groups[-1] and size > 0 and size + add > max_bytes:
            groups.append([])
            seen, size = set(), 0
            mine = streamed_of(n)
            add = sum(_pbytes(t) for _, t in mine)
        groups[-1].append(n)
        seen.update(nm for nm, _ in mine)
        size += add
    groups = [g for g in groups if g]
    segs: List[_Segment] = []
    seg_of = {n.name: i for i, g in enumerate(groups) for n in g}
    for i, grp in enumerate(groups):
        inside = {n.name for n in grp}
        g = fx.Graph()
        env: Dict[str, fx.Node] = {}
        inputs: List[str] = []
        ext: List[fx.Node] = []
        for n in grp:
            for a in n.all_input_nodes:
                if a.name not in inside and a.name not in env:
                    ext.append(a)
                    env[a.name] = None
        for a in ext:
            ph = g.placeholder(a.name)
            ph.meta = dict(a.meta)
            env[a.name] = ph
            inputs.append(a.name)
        for n in grp:
            env[n.name] = g.node_copy(n, lambda x: env[x.name])
        outs = [n.name for n in grp
                if n.name in stage_outs or any(seg_of.get(u.name, i) != i for u in n.users if u.op == "call_function")]
        g.output(tuple(env[o] for o in outs))
        g.lint()
        sub = fx.GraphModule(gm, g)
        ptens = {nm: params[nm] for nm in inputs if nm in params}
        streamed, ids = [], set()
        for t in ptens.values():
            if hasattr(t, "_rannc_host") and id(t) not in ids:
                ids.add(id(t))
                streamed.append(t)
        nbytes = sum(_pbytes(t) for t in (ptens.values() if resident else streamed)
                     if isinstance(t, torch.Tensor))
        segs.append(_Segment(sub, inputs, outs, ptens, streamed, nbytes))
    return segs


class _SegSaved:
    __slots__ = ("inputs", "rng")

    def __init__(self, inputs, rng):
        self.inputs, self.rng = inputs, rng


class StreamedStage(StageExec):
    """A stage that runs segment by segment.  Same interface as :class:`StageExec`.

    With a ``streamer`` the parameters of a segment are on the device only while the segment runs and activation
    recomputation is built in, whatever the ``checkpointing`` argument of ``forward`` says.  Without one
    (``checkpoint_segments``) the parameters are resident and the class only refines recomputation: where the
    plain stage recomputes its whole forward in backward and so holds a whole stage's activations of one
    micro-batch, this one keeps the values at the segment boundaries and recomputes one segment at a time, so
    the peak is one SEGMENT's activations -- same arithmetic, a fraction of the memory, which buys larger
    micro-batches for deep stages (the reference recomputes stage by stage, GraphConnector.cpp:395-457)."""

    def __init__(self, name: str, gm: fx.GraphModule, sub_ir, params: Dict[str, torch.Tensor],
                 streamer: Optional[ParamStreamer], window_bytes: int, segments: int = 0):
        super().__init__(name, gm, sub_ir, params)
        self.streamer = streamer
        if streamer is not None:
            self.segments = split_into_segments(gm, params, max(1, window_bytes // 2))
        else:
            total = sum(_pbytes(t) for t in {id(t): t for t in params.values()
                                             if isinstance(t, torch.nn.Parameter)}.values())
            self.segments = split_into_segments(gm, params, max(1, total // max(1, segments)), resident=True)
        self.mode: Dict[int, bool] = {}     # micro-batch -> ran segment by segment
        self._last_use: Dict[str, int] = {}
        for i, s in enumerate(self.segments):
            for nm in s.inputs:
                self._last_use[nm] = i
        self.seg_saved: Dict[int, List[_SegSaved]] = {}
        logger.info("stage %s: %d segments, largest %.1f MiB of parameters", name, len(self.segments),
                    max((s.nbytes for s in self.segments), default=0) / (1 << 20))

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _rng_state():
        return (RF.rng.get_state(), torch.get_rng_state(),
                torch.cuda.get_rng_state() if torch.cuda.is_available() else None)

    @staticmethod
    def _set_rng_state(st):
        RF.rng.set_state(st[0])
        torch.set_rng_state(st[1])
        if st[2] is not None:
            torch.cuda.set_rng_state(st[2])

    def _seg_args(self, seg: _Segment, env: Dict[str, object], with_grad: bool):
        args, leaf = [], {}
        for nm in seg.inputs:
            if nm in seg.params:
                args.append(seg.params[nm])
                continue
            t = env[nm]
            if isinstance(t, torch.Tensor):
                t = t.detach()
                if with_grad and t.is_floating_point():
                    t.requires_grad_(True)
                    leaf[nm] = t
            args.append(t)
        return args, leaf

    # ------------------------------------------------------------------ forward
    def forward(self, split: int, inputs: Dict[str, torch.Tensor], checkpointing: bool,
                grad_enabled: bool = True) -> Dict[str, torch.Tensor]:
        st = self.streamer
        if st is None and not (checkpointing and grad_enabled):
            # resident parameters and nothing to recompute: the plain stage
            self.mode[split] = False
            return super().forward(split, inputs, checkpointing, grad_enabled)
        self.mode[split] = True
        env: Dict[str, object] = {n: inputs[n] for n in self.batch_input_names}
        saved: List[_SegSaved] = []
        nxt = st.prefetch(self.segments[0].streamed) if (st is not None and self.segments) else None
        keep = set(self.output_names)
        for i, seg in enumerate(self.segments):
            win = nxt
            if st is not None:
                st.attach(win)
                nxt = st.prefetch(self.segments[i + 1].streamed) if i + 1 < len(self.segments) else None
            rng = self._rng_state() if grad_enabled else None
            args, _ = self._seg_args(seg, env, False)
            with torch.no_grad():
                outs = seg.gm(*args)
            if grad_enabled:
                saved.append(_SegSaved({nm: env[nm] for nm in seg.inputs if nm not in seg.params}, rng))
            if st is not None:
                st.release(win)
            for nm, o in zip(seg.outputs, outs):
                env[nm] = o
            for nm in seg.inputs:
                if self._last_use.get(nm) == i and nm not in keep and nm not in seg.params:
                    env.pop(nm, None)
        if grad_enabled:
            self.seg_saved[split] = saved
        res = {}
        for n in self.output_names:
            o = env[n]
            res[n] = o.detach() if isinstance(o, torch.Tensor) else o
        return res

    # ------------------------------------------------------------------ backward
    def backward(self, split: int, out_grads: Dict[str, Optional[torch.Tensor]]) -> Dict[str, torch.Tensor]:
        st = self.streamer
        if not (self.mode.get(split, True) if self.keep_graph else self.mode.pop(split, True)):
            return super().backward(split, out_grads)
        saved = self.seg_saved[split] if self.keep_graph else self.seg_saved.pop(split)
        grads: Dict[str, torch.Tensor] = {n: g for n, g in out_grads.items() if g is not None}
        cur = self._rng_state()
        last = len(self.segments) - 1
        nxt = st.prefetch(self.segments[last].streamed) if (st is not None and self.segments) else None
        for i in range(last, -1, -1):
            seg, sv = self.segments[i], saved[i]
            win = nxt
            if st is not None:
                st.attach(win)
                nxt = st.prefetch(self.segments[i - 1].streamed) if i > 0 else None
            wanted = [nm for nm in seg.outputs if nm in grads]
            if not wanted:
                if st is not None:
                    st.release(win)
                continue
            gruns = st.open_grads([p for p in seg.streamed if p.requires_grad]) if st is not None else None
            self._set_rng_state(sv.rng)
            with torch.enable_grad():
                args, leaf = self._seg_args(seg, sv.inputs, True)
                outs = dict(zip(seg.outputs, seg.gm(*args)))
            tensors, gs = [], []
            for nm in wanted:
                o = outs[nm]
                if isinstance(o, torch.Tensor) and o.requires_grad:
                    g = grads.pop(nm)
                    tensors.append(o)
                    gs.append(g.to(o.dtype) if g.dtype != o.dtype else g)
            if tensors:
                torch.autograd.backward(tensors, gs)
            for nm, t in leaf.items():
                if t.grad is None:
                    continue
                if nm in grads:
                    grads[nm] = grads[nm] + t.grad
                else:
                    grads[nm] = t.grad
                t.grad = None
            if st is not None:
                st.flush_grads(gruns)
            del outs, tensors, gs, leaf, args
            if st is not None:
                st.release(win)
        self._set_rng_state(cur)
        return {n: grads[n] for n in self.batch_input_names if n in grads}

    def clear(self):
        super().clear()
        self.seg_saved.clear()
        self.mode.clear()
