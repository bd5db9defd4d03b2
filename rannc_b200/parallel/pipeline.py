"""Whole-iteration driver: micro-batching, routes between stages, distributed backward.

Counterpart of the reference's GraphLauncher + GraphConnector + RaNNCTensorBackward
(src/comp/GraphLauncher.cpp:133-496, src/comp/GraphConnector.cpp:291-641,
src/comp/Backward.cpp:87-129).  Schedule: synchronous pipeline -- for every
micro-batch, every local stage in order: receive its inputs, run it, send its
outputs -- then the same in reverse for the backward pass, which autograd
triggers through the returned tensor.  Routes between rank sets use the
contiguous-row all-to-all-v of ``comm.redist``; a route whose source and
destination rank sets coincide is a local slice.  The scalar loss is combined
with batch-share weights (reference: src/comm/SComm.cpp:526-578).

Differences from the reference, all made possible by 180 GB of HBM: stage
inputs / outputs never round-trip through host memory between micro-batches,
and recomputation (activation checkpointing) is used only when the planner
found that the activations do not fit.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import _core
from ..utils.config import conf
from ..utils.log import get_logger
from . import comm
from .stage import StageExec

logger = get_logger("GraphLauncher")
MASTER = "MASTER"


class _RouteTable:
    def __init__(self, dep):
        self.into: Dict[str, list] = {}      # stage -> stage-to-stage routes arriving
        self.outof: Dict[str, list] = {}     # stage -> stage-to-stage routes leaving
        self.master_in: Dict[str, list] = {}  # stage -> MASTER->stage routes
        self.master_out: Dict[str, list] = {}  # stage -> stage->MASTER routes
        for r in dep.fwd_routes:
            self.into.setdefault(r.dest_graph, []).append(r)
            self.outof.setdefault(r.source_graph, []).append(r)
        for r in dep.fwd_in_routes:
            self.master_in.setdefault(r.dest_graph, []).append(r)
        for r in dep.fwd_out_routes:
            self.master_out.setdefault(r.source_graph, []).append(r)


class PipelineRuntime:
    def __init__(self, dep, stages: Dict[str, StageExec], user_inputs: List[str], user_outputs: List[str],
                 global_batch: int, gather_inputs: bool = True):
        self.dep = dep
        self.stages = stages  # local stages only
        self.user_inputs = user_inputs
        self.user_outputs = user_outputs
        self.B = int(global_batch)
        self.P = int(dep.pipeline_num)
        self.rank = comm.get_rank()
        self.world = comm.get_world_size()
        self.routes = _RouteTable(dep)
        self.order = list(dep.fwd_graph_order)
        self.alloc = {k: sorted(v) for k, v in dep.allocation.items()}
        self.all_ranks = list(range(self.world))
        self.calc = _core.BatchSizeCalculator(self.P, self.B)
        self.checkpointing = bool(dep.checkpointing)
        # checkpointing_no_last: the last stage keeps its activations (same rule as the stage search)
        self.no_ckpt_stage = self.order[-1] if (bool(conf("checkpointing_no_last")) and len(self.order) > 1) else None
        self.pending = comm.PendingOps()
        self.gather_inputs = gather_inputs
        # the ranks that hand inputs in and take outputs back: every rank with its slice of the batch, or
        # (gather_inputs=False) rank 0 with the whole batch, the outputs then being broadcast
        # (reference: GraphLauncher.cpp:41-57,110-118,412-413)
        self.master = self.all_ranks if gather_inputs else [0]
        self._fwd_state = None
        self._in_grads: Dict = {}
        self.split_hook = None      # called as split_hook(i, P) before the backward of micro-batch i starts
        sets = [self.all_ranks] + list(self.alloc.values())
        for r in list(dep.fwd_routes):
            sets.append(sorted(set(r.sources) | set(r.dests)))
        comm.create_groups(sets)
        self.out_is_loss = {o: bool(dep.graph.value(o).is_loss) for o in user_outputs}
        # debugging aids of the reference (config items display_comm_value / display_act_value,
        # src/comp/GraphLauncher.cpp, src/comm/SComm.cpp): log a digest of every value that crosses a stage
        # boundary / that a stage produces; `profiling` accumulates host-side time per stage and direction
        self.show_comm = bool(conf("display_comm_value"))
        self.show_act = bool(conf("display_act_value"))
        self.timers = _core.TimeCounter(bool(conf("profiling")))

    # ---------------------------------------------------------------- helpers
    def _show(self, what: str, name: str, split: int, t) -> None:
        if isinstance(t, torch.Tensor) and t.numel() > 0:
            f = t.detach().float()
            logger.info("%s %s [micro-batch %d] shape=%s sum=%.6g absmean=%.6g", what, name, split,
                        tuple(t.shape), float(f.sum()), float(f.abs().mean()))

    def _rows(self, ranks: Sequence[int], rank: int, split: int, mult: int = 1) -> int:
        ranks = sorted(ranks)
        if rank not in ranks:
            return 0
        return self.calc.local_split_size(ranks.index(rank), len(ranks), split) * mult

    def _mult(self, ir_value, split_rows_global: int) -> int:
        """First dimension may be a multiple of the batch (reference: BatchSizeCalculator.cpp:169-172)."""
        dims = ir_value.type.tensor_dim
        if not dims or self.B <= 0:
            return 1
        d0 = dims[0]
        return max(1, d0 // self.B) if d0 % self.B == 0 else 1

    def _move(self, value, t: Optional[torch.Tensor], src: Sequence[int], dst: Sequence[int], split: int):
        """Moves the rows of one micro-batch of a batch value from rank set ``src`` to rank set ``dst``."""
        src, dst = sorted(src), sorted(dst)
        mult = self._mult(value, 0)
        if src == dst:
            return t
        total = self.calc.split_size(split) * mult
        args = _core.get_redist_args(self.rank, self.world, total, src, dst, split, self.P, self.B)
        recv_rows = sum(args.recvcounts)
        dims = list(value.type.tensor_dim)
        row_shape = dims[1:]
        dtype = _TORCH_DTYPE[value.type.tensor_elem_type]
        return comm.redist(t, args, recv_rows, None, row_shape, dtype, self.pending)

    # ---------------------------------------------------------------- forward
    def forward(self, inputs: Sequence[torch.Tensor], grad_enabled: bool = True,
                interleave_scale: Optional[float] = None):
        """``interleave_scale``: the caller promises that every output is a loss whose backward() will arrive with
        this upstream gradient (1, or the loss scale).  With a single stage each micro-batch's backward then runs
        right after its forward, so only one micro-batch's activations are ever alive; ``backward`` later only
        checks the promise."""
        comm.check_peers()
        P = self.P
        if getattr(self, "_interleaved", None) is not None:
            logger.warning("interleave_backward: the previous forward call was not followed by backward(); the "
                           "gradients it produced are still in the gradient buffers (evaluate under torch.no_grad())")
        inter = interleave_scale is not None and grad_enabled and P > 1 and len(self.order) == 1 and \
            self.order[0] in self.stages
        self._interleaved = float(interleave_scale) if inter else None
        self.interleaved_steps = getattr(self, "interleaved_steps", 0) + (1 if inter else 0)
        by_name = dict(zip(self.user_inputs, inputs))
        # cumulative local row offsets of this rank's share of each micro-batch
        local_rows = [self.calc.local_split_size(self.master.index(self.rank), len(self.master), i)
                      if self.rank in self.master else 0 for i in range(P)]
        offs = [0]
        for r in local_rows:
            offs.append(offs[-1] + r)
        stage_vals: Dict[Tuple[int, str], Dict[str, torch.Tensor]] = {}
        loss_acc: Dict[str, torch.Tensor] = {}
        tensor_out: Dict[str, List[Optional[torch.Tensor]]] = {o: [None] * P for o in self.user_outputs}
        dev = comm.device()

        for i in range(P):
            for sname in self.order:
                ranks = self.alloc[sname]
                mine = sname in self.stages
                ins: Dict[str, torch.Tensor] = {}
                # caller -> stage
                for r in self.routes.master_in.get(sname, []):
                    v = r.ir_value
                    x = by_name.get(r.value_name)
                    if not v.is_batch or x is None or not isinstance(x, torch.Tensor) or x.dim() == 0:
                        if mine:
                            ins[r.value_name] = x
                        continue
                    mult = self._mult(v, 0)
                    piece = x[offs[i] * mult: offs[i + 1] * mult]
                    got = self._move(v, piece, self.master, ranks, i)
                    if mine:
                        ins[r.value_name] = got
                # stage -> stage
                for r in self.routes.into.get(sname, []):
                    src_ranks = self.alloc[r.source_graph]
                    held = stage_vals.get((i, r.source_graph), {}).get(r.value_name)
                    if r.ir_value.is_batch:
                        got = self._move(r.ir_value, held, src_ranks, ranks, i)
                    else:
                        got = self._bcast_value(r.ir_value, held, src_ranks, ranks)
                    if mine:
                        ins[r.value_name] = got
                        if self.show_comm:
                            self._show("recv", r.value_name, i, got)
                if not mine:
                    continue
                st = self.stages[sname]
                _core.trace_begin(_core.func_key("forward", sname, i, False))
                self.timers.start("forward " + sname)
                outs = st.forward(i, ins, self.checkpointing and sname != self.no_ckpt_stage, grad_enabled)
                self.timers.stop("forward " + sname)
                _core.trace_end(_core.func_key("forward", sname, i, False))
                stage_vals[(i, sname)] = outs
                if inter:
                    # this micro-batch's backward, now: d(global loss)/d(local loss) x world x upstream gradient
                    if self.split_hook is not None:
                        self.split_hook(i, P)
                    og = {}
                    for r in self.routes.master_out.get(sname, []):
                        w = self._loss_weight(ranks, i) * self.world * self._interleaved
                        og[r.value_name] = torch.full((), w, dtype=torch.float32, device=dev)
                    _core.trace_begin(_core.func_key("backward", sname, i, True))
                    self.timers.start("backward " + sname)
                    st.backward(i, og)
                    self.timers.stop("backward " + sname)
                    _core.trace_end(_core.func_key("backward", sname, i, True))
                if self.show_act:
                    for oname, o in outs.items():
                        self._show("out", oname, i, o)
                # stage -> caller
                for r in self.routes.master_out.get(sname, []):
                    o = outs[r.value_name]
                    if r.ir_value.is_loss or o.dim() == 0:
                        w = self._loss_weight(ranks, i)
                        contrib = o.float() * w
                        loss_acc[r.value_name] = contrib if r.value_name not in loss_acc else \
                            loss_acc[r.value_name] + contrib
        # gather caller-visible outputs
        results = []
        for oname in self.user_outputs:
            v = self.dep.graph.value(oname)
            producer = self._producer_of(oname)
            pr = self.alloc[producer]
            if v.is_loss or not v.type.tensor_dim:
                t = loss_acc.get(oname)
                if t is None:
                    t = torch.zeros((), dtype=torch.float32, device=dev)
                if self.world > 1:
                    t = t.clone()
                    comm.allreduce(t, "sum")
                results.append(t)
            else:
                pieces = []
                for i in range(P):
                    held = stage_vals.get((i, producer), {}).get(oname)
                    got = self._move(v, held, pr, self.master, i)
                    pieces.append(got)
                pieces = [p for p in pieces if p is not None]
                full = _cat_rows(pieces) if pieces else None
                if not self.gather_inputs and self.world > 1:
                    if full is None:
                        full = torch.empty(list(v.type.tensor_dim), dtype=_TORCH_DTYPE[v.type.tensor_elem_type],
                                           device=dev)
                    comm.bcast(full, self.master[0])
                results.append(full)
        self.pending.wait()
        self._fwd_state = (offs, local_rows)
        return results

    def _producer_of(self, oname: str) -> str:
        for r in self.dep.fwd_out_routes:
            if r.value_name == oname:
                return r.source_graph
        raise RuntimeError(f"no stage produces output {oname}")

    def _loss_weight(self, ranks: Sequence[int], split: int) -> float:
        """Share of the global batch this replica's micro-batch slice covers."""
        return self._rows(ranks, self.rank, split) / float(self.B)

    def _bcast_value(self, value, t, src: Sequence[int], dst: Sequence[int]):
        """Non-batch value produced on ``src`` and needed on ``dst`` (same on every source rank)."""
        src, dst = sorted(src), sorted(dst)
        if self.rank in src and t is not None and self.rank in dst:
            return t
        union = sorted(set(src) | set(dst))
        if self.rank not in union:
            return None
        dims = list(value.type.tensor_dim)
        buf = t if (self.rank == src[0] and t is not None) else \
            torch.empty(dims, dtype=_TORCH_DTYPE[value.type.tensor_elem_type], device=comm.device())
        comm.bcast(buf, src[0], union)
        return buf if self.rank in dst else None

    # ---------------------------------------------------------------- backward
    def backward(self, out_grads: Sequence[Optional[torch.Tensor]], want_input_grads: Sequence[str] = ()):
        """Runs the backward pass; returns the gradients of the user inputs named in ``want_input_grads``
        (this rank's rows; the same names must be asked for on every rank)."""
        comm.check_peers()
        P = self.P
        if getattr(self, "_interleaved", None) is not None:
            # the backward passes ran inside forward(); what is left is to see that the upstream gradient is the
            # one they were run with
            want = self._interleaved
            self._interleaved = None
            for g in out_grads:
                if g is not None and abs(float(g) - want) > 1e-6 * max(1.0, abs(want)):
                    raise RuntimeError(
                        f"interleave_backward: the loss was differentiated with an upstream gradient of {float(g)} "
                        f"where {want} was expected (call loss.backward() on the returned loss itself, or through "
                        f"amp.scale_loss); set interleave_backward=false for anything else")
            return {}
        input_grads: Dict[str, List[Optional[torch.Tensor]]] = {n: [None] * P for n in want_input_grads}
        offs, _ = self._fwd_state
        gmap = dict(zip(self.user_outputs, out_grads))
        dev = comm.device()
        recv_grads: Dict[Tuple[int, str], Dict[str, torch.Tensor]] = {}
        for i in range(P):
            if self.split_hook is not None:
                self.split_hook(i, P)
            for sname in reversed(self.order):
                ranks = self.alloc[sname]
                mine = sname in self.stages
                og: Dict[str, torch.Tensor] = dict(recv_grads.pop((i, sname), {})) if mine else {}
                # caller -> stage (gradients of the model outputs)
                for r in self.routes.master_out.get(sname, []):
                    g = gmap.get(r.value_name)
                    if g is None:
                        continue
                    v = r.ir_value
                    if v.is_loss or not v.type.tensor_dim:
                        if mine:
                            # d(global loss)/d(local loss) x world: the gradient reduction averages over the
                            # world size (see ParamStorage)
                            w = self._loss_weight(ranks, i) * self.world
                            gg = g.to(dev).float() * w
                            og[r.value_name] = gg if r.value_name not in og else og[r.value_name] + gg
                    else:
                        mult = self._mult(v, 0)
                        piece = g[offs[i] * mult: offs[i + 1] * mult]
                        got = self._move(v, piece, self.master, ranks, i)
                        if mine and got is not None:
                            og[r.value_name] = got if r.value_name not in og else og[r.value_name] + got
                # later stages -> this stage: gradients of values this stage sent
                for r in self.routes.outof.get(sname, []):
                    if not r.ir_value.type.holds_gradient():
                        continue
                    dst_ranks = self.alloc[r.dest_graph]
                    held = None
                    key = (i, r.dest_graph, r.value_name)
                    if key in self._in_grads:
                        held = self._in_grads.pop(key)
                    elif self.rank in dst_ranks and r.ir_value.is_batch:
                        # the consumer produced no gradient for this value: the producer still expects rows
                        rows = self._rows(dst_ranks, self.rank, i, self._mult(r.ir_value, 0))
                        held = torch.zeros([rows] + list(r.ir_value.type.tensor_dim)[1:],
                                           dtype=_TORCH_DTYPE[r.ir_value.type.tensor_elem_type], device=dev)
                    if r.ir_value.is_batch:
                        got = self._move(r.ir_value, held, dst_ranks, ranks, i)
                    else:
                        got = self._reduce_value(r.ir_value, held, dst_ranks, ranks)
                    if mine and got is not None:
                        og[r.value_name] = got if r.value_name not in og else og[r.value_name] + got
                in_grads: Dict[str, torch.Tensor] = {}
                if mine:
                    st = self.stages[sname]
                    _core.trace_begin(_core.func_key("backward", sname, i, True))
                    self.timers.start("backward " + sname)
                    in_grads = st.backward(i, og)
                    self.timers.stop("backward " + sname)
                    _core.trace_end(_core.func_key("backward", sname, i, True))
                    for r in self.routes.into.get(sname, []):
                        if r.value_name in in_grads:
                            self._in_grads[(i, sname, r.value_name)] = in_grads[r.value_name]
                # stage -> caller: gradients of the model inputs the caller asked for (every rank takes part in
                # the move, like for the inputs themselves)
                for r in self.routes.master_in.get(sname, []):
                    if r.value_name not in input_grads or not r.ir_value.is_batch:
                        continue
                    piece = in_grads.get(r.value_name) if mine else None
                    if mine and piece is None:
                        rows = self._rows(ranks, self.rank, i, self._mult(r.ir_value, 0))
                        piece = torch.zeros([rows] + list(r.ir_value.type.tensor_dim)[1:],
                                            dtype=_TORCH_DTYPE[r.ir_value.type.tensor_elem_type], device=dev)
                    got = self._move(r.ir_value, piece, ranks, self.master, i)
                    if got is not None:
                        cur = input_grads[r.value_name][i]
                        input_grads[r.value_name][i] = got if cur is None else cur + got
        self.pending.wait()
        self._in_grads.clear()
        out = {}
        for name, pieces in input_grads.items():
            pieces = [x for x in pieces if x is not None]
            out[name] = _cat_rows(pieces) if pieces else None
        return out

    def _reduce_value(self, value, t, src: Sequence[int], dst: Sequence[int]):
        """Gradient of a non-batch value: summed over the consumers, delivered to the producers."""
        src, dst = sorted(src), sorted(dst)
        union = sorted(set(src) | set(dst))
        if self.rank not in union:
            return None
        if len(union) == 1:
            return t
        dims = list(value.type.tensor_dim)
        buf = t.clone() if t is not None and self.rank in src else \
            torch.zeros(dims, dtype=_TORCH_DTYPE[value.type.tensor_elem_type], device=comm.device())
        comm.allreduce(buf, "sum", union)
        if len(dst) > 1:
            buf = buf / len(dst)
        return buf if self.rank in dst else None

    def clear(self):
        if bool(conf("profiling")):
            # host-side time: launches are asynchronous, so set sync_allreduce / CUDA_LAUNCH_BLOCKING for
            # device-accurate figures, or use trace_events
            logger.info("time per stage (host side)\n%s", self.timers.summary())
        for st in self.stages.values():
            st.clear()


def _cat_rows(pieces: List[torch.Tensor]) -> torch.Tensor:
    """Micro-batch outputs back into one batch: row blocks copied into one preallocated tensor by the
    row-copy kernel (16-byte vectors) on the device, ``torch.cat`` elsewhere
    (reference: TorchUtil.cpp:976-1006, cat of the per-split outputs)."""
    if len(pieces) == 1:
        return pieces[0]
    p0 = pieces[0]
    row_bytes = p0[0].numel() * p0.element_size() if p0.dim() > 0 and p0.shape[0] > 0 else 0
    if not (p0.is_cuda and row_bytes > 0 and row_bytes % 16 == 0 and all(p.is_contiguous() for p in pieces)):
        return torch.cat(pieces, 0)
    from ..ops import kernels as K

    rows = sum(p.shape[0] for p in pieces)
    out = torch.empty((rows,) + tuple(p0.shape[1:]), dtype=p0.dtype, device=p0.device)
    off = 0
    for p in pieces:
        if p.shape[0]:
            K.rowcopy(p, out[off:], p.shape[0], row_bytes, row_bytes, row_bytes)
        off += p.shape[0]
    return out


_TORCH_DTYPE = {
    _core.IRTensorElemType.FLOAT: torch.float32,
    _core.IRTensorElemType.DOUBLE: torch.float64,
    _core.IRTensorElemType.HALF: torch.float16,
    _core.IRTensorElemType.BFLOAT16: torch.bfloat16,
    _core.IRTensorElemType.INT: torch.int32,
    _core.IRTensorElemType.LONG: torch.int64,
    _core.IRTensorElemType.BOOL: torch.bool,
}
