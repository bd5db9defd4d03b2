"""``RaNNCModule``: wrap an unmodified ``nn.Module`` (+ optimizer) and train it partitioned.

Public behaviour follows the reference's Python class and the C++ class behind it
(pyrannc/__init__.py:206-593, src/comp/RaNNCModule.cpp:95-660): lazy
initialisation on the first call (trace -> profile -> partition -> deploy),
``__call__`` rejecting keyword arguments, parameter views restricted to this
rank, ``clip_grad_norm``, collective ``state_dict`` / ``get_param`` /
``get_param_grad``, ``save_deployment``, ``undeploy``, ``enable_dropout`` and the
process-wide switches ``delay_grad_allreduce`` / ``keep_graph`` /
``sync_params_on_init``.
"""
from __future__ import annotations

import os
import random
import weakref
from collections import OrderedDict
from typing import Dict, List, Optional

import torch

from . import _core
from . import amp as _amp
from .graph import planner, profiler, tracer
from .parallel import comm
from .parallel.param_storage import ParamStorage
from .parallel.pipeline import PipelineRuntime
from .parallel.stage import StageExec, build_stage_module, set_dropout
from .utils.config import conf
from .utils.log import get_logger

logger = get_logger("RaNNCModule")

_delay_grad_allreduce = False
_keep_graph = False
_sync_params_on_init = True
_live_modules: "weakref.WeakSet[RaNNCModule]" = weakref.WeakSet()


def delay_grad_allreduce(flag: bool) -> None:
    """Skip the gradient reduction at the end of backward (gradient accumulation); call
    ``model.allreduce_grads()`` before the optimizer step (reference: src/comp/Backward.cpp:100-107)."""
    global _delay_grad_allreduce
    _delay_grad_allreduce = bool(flag)


def keep_graph(flag: bool) -> None:
    global _keep_graph
    _keep_graph = bool(flag)


def sync_params_on_init(flag: bool) -> None:
    global _sync_params_on_init
    _sync_params_on_init = bool(flag)


class _DistBackward(torch.autograd.Function):
    """Autograd node that turns ``out.backward()`` into the distributed backward pass
    (reference: RaNNCTensorBackward, src/comp/Backward.cpp:87-129)."""

    @staticmethod
    def forward(ctx, mod_ref, anchor, n_out, in_names, *tensors):
        # tensors = the model outputs followed by the user inputs that require gradients
        ctx.mod_ref = mod_ref
        ctx.n = n_out
        ctx.in_names = in_names
        outs = tensors[:n_out]
        return tuple(o.clone() if o.is_floating_point() else o for o in outs)

    @staticmethod
    def backward(ctx, *grads):
        mod = ctx.mod_ref()
        if mod is None:
            raise RuntimeError("the RaNNCModule of this output no longer exists")
        in_grads = mod._run_backward(grads, ctx.in_names) or {}
        return (None, None, None, None) + (None,) * ctx.n + tuple(in_grads.get(n) for n in ctx.in_names)


class RaNNCModule:
    def __init__(self, model: torch.nn.Module, optimizer=None, gather_inputs: bool = True,
                 load_deployment: Optional[str] = None, enable_apex_amp: bool = False,
                 allreduce_amp_master_params: bool = False, enable_zero: bool = False,
                 check_unused_values: bool = True, offload_params: bool = False):
        comm.start()
        if enable_zero and not enable_apex_amp:
            # same restriction as the reference (pyrannc/__init__.py:224-225)
            raise RuntimeError("enable_zero requires enable_apex_amp")
        self.model = model
        self.optimizer = optimizer
        self.gather_inputs = gather_inputs
        self.load_deployment = load_deployment
        self.use_amp_master_params = enable_apex_amp
        self.allreduce_amp_master_params = allreduce_amp_master_params
        self.enable_zero = enable_zero
        self.check_unused_values = check_unused_values
        self.offload_params = offload_params
        self.ready = False
        self.amp_dtype = _amp.get_dtype() if enable_apex_amp else None
        self.max_grad_norm = 0.0  # > 0: clip inside the fused optimizer step
        ident = [f"mod_{random.getrandbits(64):016x}"]
        self.id = comm.bcast_obj(ident[0], 0)
        self._storage: Optional[ParamStorage] = None
        self._runtime: Optional[PipelineRuntime] = None
        self._traced = None
        self._interleave = False
        self._plan = None
        self._anchor = None
        self._used_param_names: List[str] = []
        self._dropout = True
        self._fused_reducer = None
        _live_modules.add(self)

    # ------------------------------------------------------------------ call
    def __call__(self, *args, **kwargs):
        if kwargs:
            args = self._bind_keywords(args, kwargs)
        dev = comm.device()
        if dev.type == "cuda":
            for a in args:
                if isinstance(a, torch.Tensor) and not a.is_cuda:
                    raise RuntimeError("All inputs to RaNNCModule must be on a CUDA device")
        if self.use_amp_master_params:
            # floating-point inputs follow the 16-bit compute type (Apex O2 casts them in the patched forward)
            args = tuple(a.to(self.amp_dtype) if isinstance(a, torch.Tensor) and a.is_floating_point() and
                         a.dtype != self.amp_dtype else a for a in args)
        if not self.ready:
            self._init(args)
        # A batch smaller than the one the deployment was made for (the last batch of an epoch) is padded by
        # repeating rows, and the outputs are trimmed back (reference: GraphLauncher.cpp:377-404,
        # TorchUtil.cpp:785-811).  Each rank pads its own share, so no collective is needed.
        local_bs, want = self._batch_rows(args), self._local_batch
        trim = 0
        if 0 < local_bs < want:
            idx = torch.arange(want, device=next(a.device for a in args if isinstance(a, torch.Tensor))) % local_bs
            args = tuple(a.index_select(0, idx) if isinstance(a, torch.Tensor) and a.dim() > 0 and
                         a.shape[0] == local_bs else a for a in args)
            trim = local_bs
        elif local_bs > want:
            raise RuntimeError(f"this rank's batch ({local_bs}) is larger than the one the model was deployed "
                               f"with ({want})")
        self._dist_barrier()
        # user inputs that require gradients get them back through the same autograd node
        names = tuple(n for n, a in zip(self._traced.user_inputs, args)
                      if isinstance(a, torch.Tensor) and a.requires_grad and a.is_floating_point())
        extra = tuple(a for a in args if isinstance(a, torch.Tensor) and a.requires_grad and a.is_floating_point())
        # A model without trainable parameters, fed inputs that need no gradient, has nothing to differentiate:
        # its outputs stay plain tensors, nothing is saved for a backward pass, and none is expected on any rank.
        need_grad = torch.is_grad_enabled() and (self._trainable or bool(extra))
        inter = None
        if need_grad and self._interleave and not extra and not _keep_graph:
            # the gradient that will arrive at the outputs: 1, or the loss scale under amp.scale_loss
            inter = float(_amp.get_scaler().loss_scale()) if self.use_amp_master_params else 1.0
            self._set_split_hook()
        outs = self._runtime.forward(args, grad_enabled=need_grad, interleave_scale=inter)
        if need_grad:
            outs = list(_DistBackward.apply(weakref.ref(self), self._anchor, len(outs), names, *outs, *extra))
        if trim:
            outs = [o[: trim * (o.shape[0] // want)] if isinstance(o, torch.Tensor) and o.dim() > 0 and
                    o.shape[0] % want == 0 else o for o in outs]
        return self._pack_outputs(outs)

    def _bind_keywords(self, args, kwargs):
        """Keyword arguments are placed by the signature of the wrapped model's ``forward`` (the graph only has
        positional inputs); parameters skipped in between take their defaults.  The reference refuses keyword
        arguments (pyrannc/__init__.py, ``RaNNCModule.__call__``)."""
        import inspect

        sig = inspect.signature(self.model.forward)
        try:
            bound = sig.bind(*args, **kwargs)
        except TypeError as e:
            raise RuntimeError(f"arguments do not fit the model's forward{sig}: {e}") from None
        out, last = [], -1
        params = list(sig.parameters.values())
        for i, prm in enumerate(params):
            if prm.kind in (prm.VAR_POSITIONAL, prm.VAR_KEYWORD, prm.KEYWORD_ONLY):
                if prm.name in bound.arguments and bound.arguments[prm.name]:
                    raise RuntimeError(f"forward{sig}: only plain positional-or-keyword parameters can be bound")
                continue
            if prm.name in bound.arguments:
                last = i
        for i, prm in enumerate(params[:last + 1]):
            if prm.name in bound.arguments:
                out.append(bound.arguments[prm.name])
            elif prm.default is not prm.empty:
                out.append(prm.default)
        return tuple(out)

    @staticmethod
    def _batch_rows(args) -> int:
        for a in args:
            if isinstance(a, torch.Tensor) and a.dim() > 0:
                return int(a.shape[0])
        return 0

    def _pack_outputs(self, outs):
        spec = self._traced.out_spec
        if spec is not None:
            try:
                import torch.utils._pytree as pytree

                return pytree.tree_unflatten(list(outs), spec)
            except Exception:  # noqa: BLE001
                pass
        return outs[0] if len(outs) == 1 else tuple(outs)

    # ------------------------------------------------------------------ init
    def _init(self, args):
        _core.trace_enable(False)  # not during initialisation (reference: RaNNCModule.cpp:164-166)
        rank, world = comm.get_rank(), comm.get_world_size()
        dev = comm.device()
        model = self.model
        from . import dist_param as _dp

        if self.use_amp_master_params:
            # batch-norm scale / shift and running statistics stay in fp32 (as Apex O2 keeps them, which is
            # what the reference trains with); everything else goes to the 16-bit compute type
            keep32 = set()
            for mod in model.modules():
                if isinstance(mod, torch.nn.modules.batchnorm._BatchNorm):
                    keep32.update(id(t) for t in list(mod.parameters(recurse=False)) + list(mod.buffers(recurse=False)))
            for p in model.parameters():
                if not p.is_floating_point() or id(p) in keep32:
                    continue
                if _dp.dist_param_registered(id(p)):
                    _dp.set_dist_param_dtype(id(p), self.amp_dtype)
                    p.data = torch.zeros(1, dtype=self.amp_dtype, device=p.device).expand(p.shape)
                else:
                    p.data = p.data.to(self.amp_dtype)
            for b in model.buffers():
                if b.is_floating_point() and id(b) not in keep32:
                    b.data = b.data.to(self.amp_dtype)

        # global batch = sum of the local batches (reference: RaNNCModule.cpp:173-177)
        local_bs = 0
        for a in args:
            if isinstance(a, torch.Tensor) and a.dim() > 0:
                local_bs = int(a.shape[0])
                break
        self._local_batch = local_bs
        sizes = comm.allgather_obj(local_bs)
        if not self.gather_inputs:
            global_bs = sizes[0]     # rank 0 hands in the whole batch
        else:
            if len(set(sizes)) != 1:
                raise RuntimeError(f"every rank must pass the same local batch size, got {sizes}")
            global_bs = sum(sizes)

        logger.info("Tracing model ...")
        pdev = next((p.device for p in model.parameters()), torch.device("cpu"))
        targs = tuple(a.to(pdev) if isinstance(a, torch.Tensor) else a for a in args)
        use_kernels = dev.type == "cuda" and bool(conf("fused_kernels"))
        with torch.random.fork_rng(devices=[dev] if dev.type == "cuda" else []):
            self._traced = tracer.trace(model, targs, use_kernels=use_kernels, name=self.id)
        tm = self._traced
        if tm.rewrite_stats:
            logger.info("Fused operators: %s", str(tm.rewrite_stats))
        if self.check_unused_values:
            # (an input that is None or a plain Python value is a constant of the trace, not an unused tensor)
            tensor_inputs = {n for n, a in zip(tm.user_inputs, args) if isinstance(a, torch.Tensor)}
            unused = [v for v in _core.find_unused_values(tm.ir)
                      if v in tm.params or v in tensor_inputs]
            if unused:
                raise RuntimeError(f"values never used by the model: {unused}; pass check_unused_values=False to "
                                   f"ignore")
        ir = _core.scale_graph(tm.ir, global_bs)

        logger.info("Running profiler ...")
        prof_file = str(conf("graph_profile_file"))
        measuring = bool(conf("measure_profiles")) and dev.type == "cuda" and use_kernels and \
            not any(p.is_meta for p in model.parameters())
        sub_prof = None
        if bool(conf("load_graph_profile")) and os.path.exists(prof_file):
            node_profiles = profiler.load_profiles(prof_file, [n.id for n in tm.ir.nodes], tm.trace_batch, tm.ir)
            logger.info("Loaded operator profiles from %s", prof_file)
        elif measuring and rank == 0:
            node_profiles = profiler.measured_profiles(tm.gm, dev, iters=max(1, int(conf("profiling_iter"))),
                                                       param_names=tm.params.keys())
        else:
            node_profiles = profiler.analytic_profiles(tm.gm)
        if (measuring or bool(conf("measure_subgraphs"))) and rank == 0:
            sub_prof = profiler.SubgraphProfiler(tm, dev, iters=max(1, int(conf("profiling_iter"))))
        if bool(conf("save_graph_profile")) and rank == 0:
            profiler.save_profiles(prof_file, node_profiles, tm.trace_batch, tm.ir)
            logger.info("Saved operator profiles to %s", prof_file)
        # node times were taken at the traced (local) batch: express them at the global batch
        if global_bs != tm.trace_batch and tm.trace_batch > 0:
            r = global_bs / tm.trace_batch
            for k, p in node_profiles.items():
                if p.scales_with_batch:
                    node_profiles[k] = _core.NodeProfile(p.fwd_us * r, p.bwd_us * r, int(p.activation_bytes * r),
                                                         int(p.working_bytes * r), True)

        total_mem = 0
        if dev.type == "cuda":
            total_mem = torch.cuda.get_device_properties(dev).total_memory
        dep_bytes = None
        # interleave_backward: with ONE stage, a micro-batch's backward can run right after its forward, so that
        # only one micro-batch's activations are alive (the synchronous schedule of the reference keeps or
        # recomputes all of them).  Needs the upstream gradient before the caller's backward(): possible when every
        # output is a loss (it is 1, or the loss scale) and no input wants a gradient.
        self._interleave = bool(conf("interleave_backward")) and not _keep_graph and \
            all(tm.ir.value(o).is_loss for o in tm.user_outputs) and \
            not any(isinstance(a, torch.Tensor) and a.requires_grad for a in args)
        if rank == 0:
            logger.info("Partitioning the model for %d device(s), global batch %d ...", world, global_bs)
            self._plan = planner.plan(ir, node_profiles, world, global_bs, total_mem, self.use_amp_master_params,
                                      self.enable_zero, self.offload_params, self.id, self.load_deployment,
                                      subgraph_profiler=sub_prof, interleave=self._interleave)
            if sub_prof is not None:
                if bool(conf("save_graph_profile")) and sub_prof.count:
                    # the measured blocks / stages go into the same file as the operator profiles
                    profiler.save_profiles(prof_file, node_profiles, tm.trace_batch, tm.ir, db=sub_prof.db)
                del sub_prof
                if dev.type == "cuda":
                    torch.cuda.empty_cache()
            dep_bytes = bytes(_core.save_deployment(self._plan.deployment, world, self._plan.dev_mem))
        dry = int(conf("partitioning_dry_run_np"))
        if dry > 0:
            # plan for `dry` devices on fewer, then stop (reference: RaNNCModule.cpp:416-421)
            comm.barrier()
            raise SystemExit(0)
        dep_bytes = comm.bcast_bytes(dep_bytes, 0)
        dep, _, dev_mem = _core.load_deployment(dep_bytes)
        self._dep = dep
        self._dev_mem = dev_mem

        # ---- deploy
        name_to_param = OrderedDict(model.named_parameters(remove_duplicate=True))
        name_to_buffer = OrderedDict(model.named_buffers(remove_duplicate=True))
        self._all_param_names = list(name_to_param.keys())
        self._param_order_by_name = {n: i for i, n in enumerate(self._all_param_names)}
        self._global_param_order = {id(p): self._param_order_by_name[n] for n, p in name_to_param.items()}
        self._param_meta = {n: (tuple(p.shape), p.dtype) for n, p in name_to_param.items()}
        self._trainable = any(p.requires_grad for p in name_to_param.values())
        owner: Dict[str, set] = {n: set() for n in name_to_param}
        buf_owner: Dict[str, set] = {n: set() for n in name_to_buffer}
        local_stage_names = []
        for sname in dep.fwd_graph_order:
            sg = dep.subgraphs[sname]
            ranks = dep.allocation[sname]
            for pin in sg.param_input_names():
                if pin in tm.params:
                    owner[tm.params[pin]].update(ranks)
                elif pin in tm.buffers:
                    buf_owner[tm.buffers[pin]].update(ranks)
            if rank in ranks:
                local_stage_names.append(sname)
        # a parameter shared by two stages of the same rank cannot be told apart by the gradient
        # reduction (reference: ParamStorage.cpp:893-902)
        seen: Dict[str, str] = {}
        for sname in local_stage_names:
            for pin in dep.subgraphs[sname].param_input_names():
                if pin in tm.params:
                    fq = tm.params[pin]
                    if fq in seen and seen[fq] != sname and name_to_param[fq].requires_grad and world > 1:
                        raise RuntimeError(f"parameter {fq} is shared by stages {seen[fq]} and {sname} on rank {rank}")
                    seen[fq] = sname
        if bool(conf("verify_partitioning")) and rank == 0:
            self._verify_partitioning(tm, dep, args, name_to_param, name_to_buffer)
        # tensor-partitioned linear layers: which nodes, which weights, over which ranks
        dist_kernels = dev.type == "cuda" and bool(conf("fused_kernels")) and self.use_amp_master_params
        # force_dist_matmul: every eligible linear layer.  keep_dist_params_sharded: the linear layers whose weight
        # was declared in shards (DistributeModelParams) -- such a weight is never kept whole: each replica of
        # its stage stores one column slice, and the layer's GEMM gathers the slices from the peers in its
        # prologue (forward and input gradient) and scatters the weight gradient in its epilogue.
        force = bool(conf("force_dist_matmul"))
        keep_sharded = bool(conf("keep_dist_params_sharded")) and not force
        if force or keep_sharded:
            only = {id(p) for p in name_to_param.values() if _dp.dist_param_registered(id(p))} if keep_sharded \
                else None
            dist_nodes, sliced = self._select_dist_linears(tm, dep, name_to_param, owner,
                                                           256 if dist_kernels else 1, only_params=only)
        else:
            dist_nodes, sliced = {}, {}
        for fq, ranks in sliced.items():
            p = name_to_param[fq]
            was_dist = _dp.dist_param_registered(id(p))
            if was_dist:
                # assembled once (collective over the world, every rank in the same order), cut into the column
                # slice this rank keeps, and dropped again: the peak is one parameter, not the model
                full = _dp.load_dist_param(id(p), dev)
                _dp.remove_dist_param(id(p))
            if _sync_params_on_init and not was_dist:
                comm.create_groups([ranks])
            if rank in ranks:
                if not was_dist:
                    full = p.data.to(dev)
                    if _sync_params_on_init:
                        comm.bcast(full, ranks[0], ranks)
                ks = full.shape[1] // len(ranks)
                i = ranks.index(rank)
                p.data = full[:, i * ks:(i + 1) * ks].contiguous()
            elif was_dist:
                p.data = torch.empty(0, dtype=p.dtype, device=p.device)
            full = None
        unused_params = [n for n, r in owner.items() if not r]
        for n in unused_params:
            owner[n] = {0}
        self._used_param_names = [n for n in name_to_param if rank in owner[n]]
        self._used_buffer_names = [n for n in name_to_buffer if rank in buf_owner[n] or not buf_owner[n]]
        self._buffer_root = {n: (min(r) if r else 0) for n, r in buf_owner.items()}

        # a model that was built on the device: what this rank does not use would otherwise stay in its memory
        # for good (a model built on the host, as the reference requires, leaves those values on the host)
        released = 0
        for n, p in name_to_param.items():
            if rank not in owner[n] and p.device.type == "cuda" and p.numel() > 0 and \
                    not _dp.dist_param_registered(id(p)):
                released += p.numel() * p.element_size()
                p.data = torch.empty(0, dtype=p.dtype, device=p.device)
        if released:
            logger.info("released %.1f GB of device-resident parameters that other ranks own", released / 1e9)
        # parameters sharded at construction are assembled on their owners only (collective, global order)
        for n, p in name_to_param.items():
            if _dp.dist_param_registered(id(p)):
                _dp.materialize(p, rank in owner[n], dev)

        opt_group_of = {}
        if self.optimizer is not None:
            for gi, g in enumerate(self.optimizer.param_groups):
                for p in g["params"]:
                    opt_group_of[id(p)] = gi
        self._storage = ParamStorage(self.use_amp_master_params, self.enable_zero, self.allreduce_amp_master_params)
        self._storage.sync_on_init = _sync_params_on_init
        self._storage.offload = bool(self.offload_params) and dev.type == "cuda" and self.use_amp_master_params
        # offload_param_window_mb > 0: the 16-bit parameters and their gradients leave the device too and are
        # streamed through a window of that size, segment by segment (parallel/param_stream.py)
        window_mb = int(conf("offload_param_window_mb"))
        self._storage.stream16 = bool(self.offload_params) and self.use_amp_master_params and window_mb > 0
        if self._storage.stream16 and (bool(conf("force_dist_matmul")) or bool(conf("keep_dist_params_sharded"))):
            raise RuntimeError("offload_param_window_mb does not combine with tensor-partitioned linear layers")
        if self.offload_params and not self._storage.offload and not self._storage.stream16:
            logger.warning("offload_params needs a CUDA device and mixed precision (fp32 master weights); ignored")
        local_params = {n: name_to_param[n] for n in self._used_param_names}
        # the three projection weights (and biases) of a fused QKV block are laid out back to back so that one
        # GEMM (forward, dgrad, wgrad) and one column sum serve all three
        adjacent = []
        if use_kernels:
            from .ops import functional as _RF

            for node in tm.gm.graph.nodes:
                if node.op == "call_function" and node.target is _RF.qkv_attention:
                    fq = [tm.params.get(a.name) if isinstance(a, torch.fx.Node) else None for a in node.args[1:7]]
                    if all(f is not None for f in (fq[0], fq[2], fq[4])):
                        adjacent.append([fq[0], fq[2], fq[4]])
                    if all(f is not None for f in (fq[1], fq[3], fq[5])):
                        adjacent.append([fq[1], fq[3], fq[5]])
        if self._storage.stream16:
            from .parallel.param_stream import ParamStreamer

            self._storage.streamer = ParamStreamer(dev)
        want_fused = (self.use_amp_master_params and self.enable_zero and dev.type == "cuda" and world > 1 and
                      not self.offload_params and
                      bool(conf("fused_kernels")) and bool(conf("fused_grad_allreduce")) and
                      type(self.optimizer) in (torch.optim.Adam, torch.optim.AdamW, torch.optim.SGD))
        self._storage.deploy(local_params, {n: sorted(r) for n, r in owner.items()}, opt_group_of, dev,
                             self._param_order_by_name, symmetric=want_fused, sliced=sliced,
                             symmetric_slices=dist_kernels, adjacent=adjacent)
        for n in self._used_buffer_names:
            b = name_to_buffer[n]
            b.data = b.data.to(dev)
            ranks = sorted(buf_owner[n]) if buf_owner[n] else None
            if _sync_params_on_init and ranks and len(ranks) > 1:
                comm.create_groups([ranks])
                comm.bcast(b.data, ranks[0], ranks)
        if self.use_amp_master_params:
            self._storage.setup_master()

        stages: Dict[str, StageExec] = {}
        for sname in local_stage_names:
            sg = dep.subgraphs[sname]
            gm = build_stage_module(tm.gm, sg)
            tensors = {}
            for pin in sg.param_input_names():
                if pin in tm.params:
                    tensors[pin] = name_to_param[tm.params[pin]]
                elif pin in tm.buffers:
                    tensors[pin] = name_to_buffer[tm.buffers[pin]]
                elif pin in tm.constants:
                    tensors[pin] = tm.constants[pin].to(dev)
            if sname in dist_nodes:
                self._install_dist_linears(gm, sname, dist_nodes[sname], tuple(dep.allocation[sname]), name_to_param,
                                           dist_kernels, dev)
            nseg = int(conf("checkpoint_segments"))
            if self._storage.stream16 and any(hasattr(t, "_rannc_host") for t in tensors.values()):
                from .parallel.param_stream import StreamedStage

                st = StreamedStage(sname, gm, sg, tensors, self._storage.streamer, window_mb << 20)
            elif nseg > 1:
                # activation recomputation segment by segment instead of stage by stage
                from .parallel.param_stream import StreamedStage

                st = StreamedStage(sname, gm, sg, tensors, None, 0, segments=nseg)
            else:
                st = StageExec(sname, gm, sg, tensors)
            st.keep_graph = _keep_graph
            stages[sname] = st
        self._stages = stages
        self._runtime = PipelineRuntime(dep, stages, tm.user_inputs, tm.user_outputs, global_bs, self.gather_inputs)
        self._buffer_mutations = tm.buffer_mutations
        self._anchor = torch.zeros((), device=dev, requires_grad=True)

        if self.optimizer is not None:
            from .opt import patch_optimizer

            patch_optimizer(self, self.optimizer)
        if want_fused:
            self._setup_fused_reducer()
        self.ready = True
        comm.barrier()
        _core.trace_enable(bool(conf("trace_events")))
        logger.info("RaNNCModule is ready. (rank %d: stages %s)", rank, str(local_stage_names))

    # ------------------------------------------------------------------ validation
    def _verify_partitioning(self, tm, dep, args, name_to_param, name_to_buffer):
        """Runs the traced graph as a whole and as the chain of its stage graphs (dropout off) on the same
        inputs and compares every user output (reference: Validator::validate, src/comp/Validator.cpp:109-226).
        Runs on rank 0, on whatever device the parameters are on at this point; buffers that the graphs update
        in place (BatchNorm statistics) are copied first."""
        import copy as _copy

        from .parallel.stage import build_stage_module, set_dropout

        ph = {n.name: n for n in tm.gm.graph.nodes if n.op == "placeholder"}
        env: Dict[str, torch.Tensor] = {}
        pdev = next((p.device for p in name_to_param.values()), torch.device("cpu"))
        for nm, a in zip(tm.user_inputs, args):
            env[nm] = a.to(pdev) if isinstance(a, torch.Tensor) else a
        for nm in ph:
            if nm in tm.params:
                env[nm] = name_to_param[tm.params[nm]].detach()
            elif nm in tm.buffers:
                env[nm] = name_to_buffer[tm.buffers[nm]].detach()
            elif nm in tm.constants:
                env[nm] = tm.constants[nm].to(pdev)

        def run(gm, names, values):
            gm = _copy.deepcopy(gm)
            set_dropout(gm, False)
            gm.recompile()
            vals = [values[n].clone() if n in tm.buffers else values[n] for n in names]
            with torch.no_grad():
                return gm(*vals)

        whole_names = [n.name for n in tm.gm.graph.nodes if n.op == "placeholder"]
        whole = run(tm.gm, whole_names, env)
        whole = whole if isinstance(whole, (tuple, list)) else (whole,)
        out_nodes = []
        for n in tm.gm.graph.nodes:
            if n.op == "output":
                import torch.utils._pytree as pytree

                out_nodes = [a.name for a in pytree.tree_leaves(n.args) if isinstance(a, torch.fx.Node)]
        expected = dict(zip(out_nodes, whole))
        chained = dict(env)
        for sname in dep.fwd_graph_order:
            sg = dep.subgraphs[sname]
            outs = run(build_stage_module(tm.gm, sg), list(sg.input_names), chained)
            outs = outs if isinstance(outs, (tuple, list)) else (outs,)
            chained.update(zip(sg.output_names, outs))
        bad = []
        for o in tm.user_outputs:
            a, b = expected[o].float(), chained[o].float()
            tol = 1e-4 if expected[o].dtype == torch.float32 else 2e-2
            if a.shape != b.shape or not torch.allclose(a, b, rtol=tol, atol=tol * max(1.0, float(a.abs().max()))):
                bad.append(o)
        if bad:
            raise RuntimeError(f"verify_partitioning: outputs {bad} of the partitioned graphs differ from the "
                               f"original graph")
        logger.info("verify_partitioning: %d stage graph(s) reproduce the original graph", len(dep.fwd_graph_order))

    # ------------------------------------------------------------------ tensor-partitioned linear layers
    @staticmethod
    def _select_dist_linears(tm, dep, name_to_param, owner, col_unit: int = 1, only_params=None):
        """Every ``linear`` whose stage has more than one replica and whose weight is a plain 2-D parameter
        used by that node alone is partitioned along its input dimension over the replicas
        (reference: src/distop/PartitionTensor.cpp:230-298, config force_dist_matmul).  Deterministic: every
        rank derives the same selection from the deployment."""
        from .ops import functional as RF

        by_name = {n.name: n for n in tm.gm.graph.nodes}
        use_count: Dict[str, int] = {}
        for n in tm.gm.graph.nodes:
            if n.op == "placeholder":
                use_count[n.name] = len(n.users)
        dist_nodes: Dict[str, Dict[str, str]] = {}
        sliced: Dict[str, tuple] = {}
        for sname in dep.fwd_graph_order:
            ranks = tuple(sorted(dep.allocation[sname]))
            n = len(ranks)
            if n < 2:
                continue
            for irn in dep.subgraphs[sname].nodes:
                fxn = by_name.get(irn.id)
                if fxn is None or fxn.op != "call_function":
                    continue
                if fxn.target is torch.ops.aten.linear.default:
                    pass
                elif fxn.target is RF.linear and (len(fxn.args) < 4 or fxn.args[3] is None):
                    pass
                else:
                    continue
                w = fxn.args[1]
                if not isinstance(w, torch.fx.Node) or w.op != "placeholder" or w.name not in tm.params:
                    continue
                fq = tm.params[w.name]
                p = name_to_param.get(fq)
                if p is None or p.dim() != 2 or use_count.get(w.name, 0) != 1 or set(owner[fq]) != set(ranks):
                    continue
                if only_params is not None and id(p) not in only_params:
                    continue
                if p.shape[1] % (col_unit * n):   # the kernels move slices in 256-column tiles
                    continue
                dist_nodes.setdefault(sname, {})[fxn.name] = fq
                sliced[fq] = ranks
        return dist_nodes, sliced

    def _install_dist_linears(self, gm, sname, nodes, ranks, name_to_param, kernels, dev):
        """Turns the selected ``linear`` nodes of a stage graph into ``linear_dist_op`` calls.  With the
        kernels, peers read each other's weight slices and add into each other's gradient slices directly:
        both live in this rank's symmetric flat buffers, whose peer addresses are resolved here."""
        from .parallel import distop

        if not hasattr(self, "_dist_groups"):
            self._dist_groups = {}
        sizes = [name_to_param[fq].numel() * len(ranks) for fq in nodes.values()]
        dtype = next(iter(name_to_param[fq].dtype for fq in nodes.values()))
        grp = distop.DistGroup(ranks, max(sizes), dtype, dev, kernels=kernels)
        self._dist_groups[sname] = grp
        ptrs = {}
        if kernels:
            import torch.distributed._symmetric_memory as symm_mem

            seen = {}
            for fq in nodes.values():
                g, i = self._storage.by_name[fq]
                if id(g) not in seen:
                    pg = comm.group(ranks)
                    seen[id(g)] = (symm_mem.rendezvous(g.flat_param, pg), symm_mem.rendezvous(g.flat_grad, pg))
                ph, gh = seen[id(g)]
                off = g.offsets[i]
                ptrs[fq] = ([int(b) + off * g.flat_param.element_size() for b in ph.buffer_ptrs],
                            [int(b) + off * g.flat_grad.element_size() for b in gh.buffer_ptrs])
            self._dist_keep = getattr(self, "_dist_keep", []) + list(seen.values())
        for n in gm.graph.nodes:
            if n.name in nodes:
                fq = nodes[n.name]
                sp, gp = ptrs.get(fq, ([], []))
                key = distop.register_site(distop.LinearDistSite(grp, sp, gp))
                bias = n.args[2] if len(n.args) > 2 else n.kwargs.get("bias")
                n.target = distop.linear_dist_op
                n.args = (n.args[0], n.args[1], bias, key)
                n.kwargs = {}
        gm.graph.lint()
        gm.recompile()

    def _dist_barrier(self):
        """Peers read this rank's weight slices and write into its gradient slices from their own streams:
        a stream-ordered barrier over each replica set separates those accesses from this rank's optimizer
        step and zero_grad (before the first forward of a step and after the last backward)."""
        for grp in getattr(self, "_dist_groups", {}).values():
            grp.barrier()

    def _setup_fused_reducer(self):
        try:
            from .parallel.fused_reduce import FusedGradReducer

            self._fused_reducer = FusedGradReducer.create(self._storage, self.optimizer)
        except Exception as e:  # noqa: BLE001
            logger.warning("fused gradient reduction unavailable (%s); using NCCL collectives", str(e))
            self._fused_reducer = None
            return
        red = self._fused_reducer
        self._storage.reducer = red
        from .ops import functional as RF
        from .ops import kernels as K

        RF.set_grad_listener(red.on_grads)

        # a parameter whose gradient reaches it through autograd (an operator without a fused wgrad) is folded
        # into the fp32 buffer as soon as it is accumulated, and reported like the others
        def fold(p):
            mg = getattr(p, "main_grad", None)
            if mg is None or p.grad is None or p.grad.data_ptr() == mg.data_ptr():
                return
            if p.grad.is_cuda and p.grad.dtype in (torch.float16, torch.bfloat16):
                K.accum_f32(mg, p.grad.contiguous())
            else:
                mg.add_(p.grad.float())
            p.grad = None
            red.on_grads([p])

        self._grad_hooks = []
        for g in self._storage.groups:
            if g.flat_master is None:
                continue
            for p in g.params:
                if p.requires_grad:
                    self._grad_hooks.append(p.register_post_accumulate_grad_hook(fold))

    # ------------------------------------------------------------------ backward
    def _set_split_hook(self):
        red = self._fused_reducer
        if red is not None and red.handles_reduce:
            # the reducer is told which micro-batch's backward is the last one before the optimizer step: during
            # that one it launches each bucket's reduction as soon as the bucket's gradients are complete
            final = not _delay_grad_allreduce
            self._runtime.split_hook = lambda i, n: red.begin_backward(final and i == n - 1)
        else:
            self._runtime.split_hook = None

    def _run_backward(self, grads, want_input_grads=()):
        red = self._fused_reducer
        self._set_split_hook()
        try:
            in_grads = self._runtime.backward(grads, want_input_grads)
        finally:
            if red is not None and red.handles_reduce:
                red.end_backward()
        self._dist_barrier()
        if not _delay_grad_allreduce:
            if self.enable_zero:
                self.allreduce_grads_zero()
            else:
                self.allreduce_grads()
        return in_grads

    def allreduce_grads(self):
        if self._fused_reducer is not None and self._fused_reducer.handles_reduce:
            self._storage.fold_model_grads()
            self._fused_reducer.mark_ready()
            return
        self._storage.allreduce_grads()

    def allreduce_grads_zero(self):
        if self._fused_reducer is not None and self._fused_reducer.handles_reduce:
            self._storage.fold_model_grads()
            self._fused_reducer.mark_ready()
            return
        self._storage.allreduce_grads_zero()

    def _needs_grad_norm(self) -> bool:
        scaler = _amp.get_scaler()
        return (self.use_amp_master_params and (self.amp_dtype == torch.float16 or scaler.loss_scale() != 1.0)) or \
            self.max_grad_norm > 0.0

    def _amp_prepare_step(self):
        """Called by the patched optimizer step.  Returns None (nothing to do), False (overflow: skip the step)
        or a device tensor [gradient multiplier, skip flag] for the fused optimizer kernel."""
        scaler = _amp.get_scaler()
        scale = scaler.loss_scale() if self.use_amp_master_params else 1.0
        need_check = self.use_amp_master_params and self.amp_dtype == torch.float16
        if not need_check and scale == 1.0 and self.max_grad_norm <= 0.0:
            return None
        ss = self._storage.grad_sumsq()
        ctrl = self._storage._ctrl
        if ss.is_cuda:
            from .ops import kernels as K

            K.finalize_ctrl(ss, 1.0 / scale, float(self.max_grad_norm), ctrl, self._storage._norm)
        else:
            norm = float(ss.sqrt()) / scale
            bad = not torch.isfinite(ss).all()
            mul = 1.0 / scale
            if self.max_grad_norm > 0 and not bad:
                mul *= min(1.0, self.max_grad_norm / (norm + 1e-6))
            ctrl[0], ctrl[1] = mul, 1.0 if bad else 0.0
        if need_check:
            overflow = bool(ctrl[1].item() != 0)
            if scaler.update_scale(overflow):
                return False
        return ctrl

    # ------------------------------------------------------------------ parameters
    def parameters(self, recurse: bool = True):
        for _, p in self.named_parameters():
            yield p

    def named_parameters(self, prefix: str = "", recurse: bool = True):
        if not self.ready:
            yield from self.model.named_parameters(prefix, recurse)
            return
        used = set(self._used_param_names)
        for n, p in self.model.named_parameters(prefix, recurse):
            base = n[len(prefix) + 1:] if prefix else n
            if base in used:
                yield n, p

    def buffers(self, recurse: bool = True):
        for _, b in self.named_buffers():
            yield b

    def named_buffers(self, prefix: str = "", recurse: bool = True):
        if not self.ready:
            yield from self.model.named_buffers(prefix, recurse)
            return
        used = set(self._used_buffer_names)
        for n, b in self.model.named_buffers(prefix, recurse):
            base = n[len(prefix) + 1:] if prefix else n
            if base in used:
                yield n, b

    def to(self, *args, **kwargs):
        logger.warning("to() was ignored. RaNNC places the parameters itself.")
        return self

    def cuda(self, *args, **kwargs):
        logger.warning("cuda() was ignored. RaNNC places the parameters itself.")
        return self

    def train(self, mode: bool = True):
        if self.ready:
            logger.warning("train() after the first forward only toggles dropout; use enable_dropout().")
            self.enable_dropout(mode)
        self.model.train(mode)
        return self

    def eval(self):
        return self.train(False)

    def zero_grad(self):
        if self._storage is not None:
            self._storage.zero_grad()
        else:
            self.model.zero_grad()

    def clip_grad_norm(self, max_norm: float) -> float:
        """Global L2 norm over every rank's gradients, then scale (reference: ParamStorage.cpp:721-819)."""
        return self._storage.clip_grad_norm(float(max_norm))

    def _calc_grad_norm(self) -> float:
        return self._storage.calc_grad_norm()

    def get_param(self, name: str, amp_master_param: bool = False) -> torch.Tensor:
        shape, dtype = self._param_meta[name]
        return self._storage.get_param(name, shape, dtype, amp_master_param)

    def get_param_grad(self, name: str, amp_master_param: bool = False) -> torch.Tensor:
        shape, dtype = self._param_meta[name]
        return self._storage.get_param_grad(name, shape, dtype, amp_master_param)

    # ---- the reference's lower-level accessors (src/main.cpp:271-402, src/comp/RaNNCModule.cpp:595-664) --------
    def sync_param(self, name: str) -> torch.Tensor:
        """Collective: the current value of parameter ``name`` (the 16-bit / working copy) on every rank, on the
        CPU.  The reference addresses parameters by id; here the name is the key."""
        return self.get_param(name, False)

    def sync_param_grad(self, name: str) -> torch.Tensor:
        """Collective: the reduced gradient of parameter ``name`` on every rank, on the CPU."""
        return self.get_param_grad(name, False)

    def sync_param_zero(self, grad: bool = False) -> None:
        """Under ZeRO every rank updates slices of the parameters; the reference re-broadcasts the slices here
        before parameters are read.  The fused and the collective update paths of this runtime both leave every
        owner with the full 16-bit parameters after each step (the all-gather is part of the step), so there is
        nothing left to do; gradients are assembled on demand by :meth:`get_param_grad`."""
        if self.ready:
            self._storage._ensure_reduced(sticky=False)

    def align_params(self) -> None:
        """The reference re-aligns its ZeRO buffers after the optimizer was patched; the flat buffers here are
        laid out aligned at deployment and never move."""

    def get_local_param_range(self, name: str):
        """(begin, end) in elements, relative to the start of parameter ``name``, of the part whose fp32 master
        copy and optimizer state this rank keeps (the whole parameter without ZeRO; (0, 0) when this rank holds
        none of it).  Reference: ParamStorage::getLocalParamRange."""
        if not self.ready or name not in self._storage.by_name:
            return (0, 0)
        g, i = self._storage.by_name[name]
        lo, _ = g.param_range(i)
        a, b = g.local_range(i)
        return (a - lo, b - lo) if b > a else (0, 0)

    def get_local_param_segment(self, name: str) -> Optional[torch.Tensor]:
        """This rank's part of parameter ``name`` as a flat tensor: the fp32 master values under mixed precision,
        the parameter's own values otherwise (None when this rank holds none of it)."""
        if not self.ready or name not in self._storage.by_name:
            return None
        g, i = self._storage.by_name[name]
        a, b = g.local_range(i)
        if b <= a:
            return None
        if g.flat_master is not None:
            la = g.to_local(a)
            return g.flat_master[la:la + (b - a)]
        return g.flat_param[a:b]

    def _sync_orig_params(self, sync_all_ranks: bool = False, sync_grad: bool = False, name_pattern=None) -> None:
        """Collective: writes the trained values (and, with ``sync_grad``, the reduced gradients) back into the
        parameters of the wrapped model on rank 0, or on every rank (reference: pyrannc/__init__.py:539-572).  A
        parameter this rank holds keeps its place in the flat buffer and is already current; one it does not hold
        gets a tensor of its own."""
        if not self.ready:
            return
        rank = comm.get_rank()
        held = set(self._used_param_names)
        for name, p in self.model.named_parameters():
            if name_pattern is not None and name_pattern not in name:
                continue
            v = self.get_param(name, False)
            gv = self.get_param_grad(name, False) if (sync_grad and p.requires_grad) else None
            if rank != 0 and not sync_all_ranks:
                continue
            with torch.no_grad():
                if name not in held or p.data.numel() != v.numel():
                    dev = p.device if p.data.numel() else v.device
                    p.data = v.to(device=dev, dtype=p.dtype)
                if gv is not None:
                    p.grad = gv.to(device=p.device, dtype=p.dtype).view(p.shape)
        comm.barrier()

    def state_dict(self, *args, no_hook: bool = False, sync_all_ranks: bool = True, amp_master_params: bool = True,
                   rank0_only: bool = True, **kwargs):
        """Collective: every rank must call it.  Full CPU tensors under the original names (tied parameters
        under every alias); fp32 master values under mixed precision (reference: pyrannc/__init__.py:401-436)."""
        if not self.ready:
            return self.model.state_dict(*args, **kwargs)
        self._check_device_error()
        keep = comm.get_rank() == 0 or not rank0_only
        out = OrderedDict()
        by_id = {}
        for n, p in self.model.named_parameters(remove_duplicate=False):
            canon = by_id.setdefault(id(p), n)
            if canon == n:
                v = self.get_param(n, amp_master_params and self.use_amp_master_params)
                if keep:
                    out[n] = v
            elif keep:
                out[n] = out[canon]
        sd_keys = self.model.state_dict().keys()
        for n, b in self.model.named_buffers(remove_duplicate=False):
            if n not in sd_keys:
                continue
            v = b.detach().to(comm.device()).clone()
            if comm.get_world_size() > 1:
                # the stage that holds a buffer updates it (BatchNorm statistics); its first rank is the source
                comm.bcast(v, self._buffer_root.get(n, 0))
            if keep:
                out[n] = v.cpu()
        return out if keep else None

    def load_state_dict(self, state_dict, strict: bool = True):
        """Before the first forward call the values go into the wrapped model.  Afterwards they are written into
        the deployed storage on every rank that holds the parameter (working copy and fp32 master copy; shards
        and column slices are cut out locally), so the partitioning is kept; every rank passes the same
        ``state_dict``.  (The reference takes the model down and partitions it again:
        pyrannc/__init__.py:438-451.)  Optimizer state is not touched: load it with
        ``optimizer.load_state_dict(sd, from_global=True)``."""
        if not self.ready:
            return self.model.load_state_dict(state_dict, strict)
        params = dict(self.model.named_parameters(remove_duplicate=False))
        canon = {}
        for n, p in self.model.named_parameters(remove_duplicate=True):
            canon[id(p)] = n
        bufs = dict(self.model.named_buffers(remove_duplicate=False))
        expected = list(self.model.state_dict().keys())
        unexpected, done = [], set()
        with torch.no_grad():
            for k, v in state_dict.items():
                if k in params:
                    c = canon[id(params[k])]
                    if tuple(v.shape) != self._param_meta[c][0]:
                        raise RuntimeError(f"{k}: shape {tuple(v.shape)} does not match {self._param_meta[c][0]}")
                    if c not in done:
                        self._storage.load_param(c, v)
                        done.add(c)
                elif k in bufs:
                    b = bufs[k]
                    b.data.copy_(v.to(device=b.device, dtype=b.dtype))
                else:
                    unexpected.append(k)
        missing = [k for k in expected if k not in state_dict]
        if strict and (missing or unexpected):
            raise RuntimeError(f"load_state_dict: missing keys {missing[:8]}, unexpected keys {unexpected[:8]}")
        from torch.nn.modules.module import _IncompatibleKeys

        return _IncompatibleKeys(missing, unexpected)

    def dim_names(self) -> Dict[str, List[str]]:
        """With ``use_named_tensors``: traced value -> a name per dimension, ``"N"`` for the batch
        (reference: the names its profiler puts on tensors, src/comp/GraphProfiler.cpp:149-170).  Empty before
        the first call of the module or when the switch is off."""
        return dict(self._traced.dim_names) if self._traced is not None else {}

    def save_deployment(self, path: str) -> None:
        if comm.get_rank() == 0:
            with open(path, "wb") as f:
                f.write(_core.save_deployment(self._dep, comm.get_world_size(), self._dev_mem))

    def _check_device_error(self) -> None:
        """Every bounded wait inside a kernel of this library records, in a device word, that it gave up (an
        mbarrier that never completed, a peer flag that was never set).  Reading the word synchronises the
        device, so the runtime does it where it waits anyway: before parameters are collected for a checkpoint
        and when the module is taken down.  ``rannc_b200.ops._lib.read_error()`` reads it at any other time."""
        if self._kernels_on():
            from .ops import _lib

            err = _lib.read_error()
            if err > 0:
                what = {1: "an on-chip barrier wait", 2: "a wait for a peer GPU"}.get(err, f"code {err}")
                raise RuntimeError(f"a kernel gave up on {what} since the last check (rank {comm.get_rank()}); "
                                   f"results computed since then are not valid")

    def _after_step(self) -> None:
        """Called by the patched optimizer step.  Looks at the device error word as it was one step ago (an
        asynchronous copy, no synchronisation) and raises ``CommError`` when a kernel of this library gave up
        on a wait since then."""
        if not self._kernels_on() or not bool(conf("check_device_error_every_step")):
            return
        from .ops import _lib

        peek = getattr(self, "_err_peek", None)
        if peek is None:
            peek = self._err_peek = _lib.ErrorPeek()
        err = peek.poll()
        if err > 0:
            what = {1: "an on-chip barrier wait", 2: "a wait for a peer GPU", 3: "a bounds check"}.get(
                err, f"code {err}")
            _lib.read_error()  # clear
            raise comm.CommError(f"a kernel gave up on {what} during an earlier step (rank {comm.get_rank()}, "
                                 f"device error word {err}); results computed since then are not valid")

    def _kernels_on(self) -> bool:
        return bool(self.ready and comm.is_cuda() and bool(conf("fused_kernels")))

    def undeploy(self) -> None:
        if self._runtime is not None:
            try:
                self._check_device_error()
            except Exception as e:  # taking the module down must not fail (it also runs at interpreter exit)
                logger.error("%s", e)
            self._runtime.clear()
        self._runtime = None
        self._stages = {}
        self.ready = False

    def enable_dropout(self, enable: bool) -> None:
        self._dropout = bool(enable)
        for st in getattr(self, "_stages", {}).values():
            set_dropout(st.gm, enable)

    def is_checkpointing_enabled(self) -> bool:
        return bool(self._dep.checkpointing) if self.ready else False

    def __getattr__(self, name):
        model = self.__dict__.get("model")
        if model is not None and hasattr(model, name):
            return getattr(model, name)
        raise AttributeError(name)

    def __del__(self):
        try:
            self.undeploy()
        except Exception:  # noqa: BLE001
            pass
