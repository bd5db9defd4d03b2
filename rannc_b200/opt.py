"""Optimizer patching and optimizer checkpoints.

Same contract as the reference's ``pyrannc/opt.py``:

* ``patch_optimizer`` rewrites ``param_groups`` so the optimizer only sees the
  parameters placed on this rank (under mixed precision: their fp32 master
  copies; under ZeRO: the local fp32 segments, empty segments dropped --
  pyrannc/opt.py:205-246), and patches ``step``, ``zero_grad``, ``state_dict``
  and ``load_state_dict``;
* ``optimizer.state_dict(from_global=True)`` gathers the state of every
  parameter to rank 0 in the format
  ``{'state': {global_param_order: {...}}, 'param_groups': <original groups>}``
  (pyrannc/opt.py:98-157) and ``load_state_dict(sd, from_global=True)``
  re-shards it (pyrannc/opt.py:186-202,276-289).

What differs: for Adam / AdamW / SGD the patched ``step`` runs ONE fused kernel
per (flat buffer, param group) over the flat master / gradient / moment buffers
-- un-scaling, clipping, overflow skip, update and the 16-bit write-back in one
pass -- instead of stepping per parameter (``ops/kernels.py: adam_flat``).  Any
other optimizer class still works through its own ``step`` on the master views.
"""
from __future__ import annotations

import copy
import types
from typing import Dict, List, Optional

import torch

from .ops import functional as RF
from .parallel import comm
from .utils.config import conf
from .utils.log import get_logger

logger = get_logger("Optimizer")


def _fusable(opt) -> Optional[str]:
    if not bool(conf("fused_kernels")):
        return None
    if type(opt) in (torch.optim.Adam, torch.optim.AdamW):
        for g in opt.param_groups:
            if g.get("amsgrad") or g.get("maximize") or g.get("capturable"):
                return None
        return "adam"
    if type(opt) is torch.optim.SGD:
        for g in opt.param_groups:
            if g.get("maximize"):
                return None
        return "sgd"
    return None


def _state_on_host(g) -> bool:
    """fp32 master weights and moments of the group are kept in host memory and streamed through the device by
    the update (``offload_params``; with streamed 16-bit parameters the gradients are host-resident too)."""
    return g.flat_master is not None and not g.flat_master.is_cuda and \
        (g.flat_grad.is_cuda or (getattr(g, "streamed", False) and g.device.type == "cuda"))


class _FlatState:
    """Moment buffers of one flat group, indexed like its master buffer (the shard under ZeRO)."""

    def __init__(self, n: int, device, kind: str, host: bool = False):
        if host:
            # offload_params: the moments stay in pinned host memory and stream through the device
            self.m = torch.zeros(n, dtype=torch.float32).pin_memory()
            self.v = torch.zeros(n, dtype=torch.float32).pin_memory() if kind == "adam" else None
        else:
            self.m = torch.zeros(n, dtype=torch.float32, device=device)
            self.v = torch.zeros(n, dtype=torch.float32, device=device) if kind == "adam" else None
        self.step = 0


class _OffloadWindow:
    """Two sets of device staging buffers and a copy stream: while the update kernel works on one chunk of
    (master, m, v), the next chunk is on its way in and the previous one on its way out
    (reference: offload_params moves parameters per operator with H2D / D2H hooks, TorchDriver.cpp:318-374;
    here the 16-bit parameters stay resident and the 12 bytes / parameter of fp32 state are what leaves
    the device)."""

    def __init__(self, device, chunk: int, n_state: int):
        self.chunk = chunk
        self.stream = torch.cuda.Stream(device)
        self.bufs = [[torch.empty(chunk, dtype=torch.float32, device=device) for _ in range(n_state)]
                     for _ in range(2)]
        self.free = [None, None]
        self.extra = {}

    def _extra(self, k: int, j: int, dtype, device):
        key = (k, j, dtype)
        buf = self.extra.get(key)
        if buf is None:
            buf = self.extra[key] = torch.empty(self.chunk, dtype=dtype, device=device)
        return buf

    def run(self, host_tensors, n: int, kernel, ins=(), outs=()):
        """``kernel(off, cnt, dev_tensors, dev_ins, dev_outs)`` updates ``cnt`` elements at offset ``off`` in
        place on the device.  ``host_tensors`` travel both ways; ``ins`` (e.g. host-resident gradients) only
        to the device, ``outs`` (e.g. host-resident 16-bit parameters) only back."""
        cur = torch.cuda.current_stream()
        dev = self.bufs[0][0].device
        k = 0
        for off in range(0, n, self.chunk):
            cnt = min(self.chunk, n - off)
            set_ = self.bufs[k & 1]
            d_in = [self._extra(k & 1, j, h.dtype, dev) for j, h in enumerate(ins)]
            d_out = [self._extra(k & 1, len(ins) + j, h.dtype, dev) for j, h in enumerate(outs)]
            with torch.cuda.stream(self.stream):
                if self.free[k & 1] is not None:
                    self.stream.wait_event(self.free[k & 1])
                for h, d in zip(host_tensors, set_):
                    d[:cnt].copy_(h[off:off + cnt], non_blocking=True)
                for h, d in zip(ins, d_in):
                    d[:cnt].copy_(h[off:off + cnt], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(self.stream)
            cur.wait_event(ready)
            kernel(off, cnt, [d[:cnt] for d in set_], [d[:cnt] for d in d_in], [d[:cnt] for d in d_out])
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(self.stream):
                self.stream.wait_event(done)
                for h, d in zip(host_tensors, set_):
                    h[off:off + cnt].copy_(d[:cnt], non_blocking=True)
                for h, d in zip(outs, d_out):
                    h[off:off + cnt].copy_(d[:cnt], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
                self.free[k & 1] = ev
            k += 1
        # later work on this stream (and the host, at the next synchronisation) sees the written-back state
        for ev in self.free:
            if ev is not None:
                cur.wait_event(ev)


def patch_optimizer(module, optimizer):
    """``module`` is the RaNNCModule that owns the ParamStorage."""
    storage = module._storage
    amp = storage.amp
    optimizer._rannc_orig_param_groups = [
        {k: (list(v) if k == "params" else v) for k, v in g.items()} for g in optimizer.param_groups]
    orig_params_flat = [p for g in optimizer._rannc_orig_param_groups for p in g["params"]]
    optimizer._rannc_orig_ids = [id(p) for p in orig_params_flat]

    # model parameter -> the tensor the optimizer updates on this rank
    local_of: Dict[int, Optional[torch.nn.Parameter]] = {}
    for g in storage.groups:
        for i, p in enumerate(g.params):
            if amp and g.master_params and g.master_params[i] is not None:
                local_of[id(p)] = g.master_params[i]
            elif amp and g.flat_master is not None:
                local_of[id(p)] = None  # empty segment on this rank
            else:
                local_of[id(p)] = p
    # global order of a parameter = its position in the traversal of the ORIGINAL param groups, which is how
    # torch numbers ``param_groups[*]['params']`` and how the reference numbers the gathered state
    # (pyrannc/opt.py, patch_optimizer: global_order counts over param_groups)
    name_of_id = {id(p): n for n, p in module.model.named_parameters(remove_duplicate=True)}
    order_by_name: Dict[str, int] = {}
    for k, p in enumerate(orig_params_flat):
        n = name_of_id.get(id(p))
        if n is not None and n not in order_by_name:
            order_by_name[n] = k
    optimizer._rannc_order_by_name = order_by_name
    local_to_global: Dict[int, int] = {}
    new_groups = []
    k = 0
    for gi, g in enumerate(optimizer.param_groups):
        kept = []
        for p in g["params"]:
            lp = local_of.get(id(p), None)
            if lp is not None:
                kept.append(lp)
                local_to_global[id(lp)] = k
            k += 1
        g["params"] = kept
        new_groups.append(g)
    optimizer.state.clear()
    optimizer._rannc_local_to_global = local_to_global
    optimizer._rannc_kind = _fusable(optimizer)
    if getattr(storage, "offload", False) and optimizer._rannc_kind is None:
        raise RuntimeError("offload_params supports Adam, AdamW and SGD (the streamed update kernels)")
    optimizer._rannc_flat_state = {}
    optimizer._rannc_module = module

    orig_step = optimizer.step
    orig_state_dict = optimizer.state_dict
    orig_load_state_dict = optimizer.load_state_dict

    def _flat_ranges():
        """(flat group, optimizer group index, a, b): maximal runs [a, b) in flat coordinates of consecutive
        parameters that belong to the same optimizer group and require gradients, clipped to the pieces this
        rank updates.  Parameters that are frozen or were not handed to the optimizer are in no run, so weight
        decay never touches them."""
        out = []
        for g in storage.groups:
            runs: List[List[int]] = []
            for i, og in enumerate(g.opt_group):
                if og < 0 or not g.params[i].requires_grad:
                    continue
                lo, hi = g.param_range(i)
                if runs and runs[-1][0] == og and runs[-1][3] == i - 1 and \
                        g.bucket_of[runs[-1][3]] == g.bucket_of[i]:
                    runs[-1][2], runs[-1][3] = hi, i
                else:
                    runs.append([og, lo, hi, i])
            for og, lo, hi, _ in runs:
                for pa, pb, _loc in g.pieces:
                    a, b = max(lo, pa), min(hi, pb)
                    if b > a:
                        out.append((g, og, a, b))
        return out

    def _publish_state(g, fs):
        """Per-parameter views of the flat moments in ``optimizer.state`` (torch's own layout).  The views are
        made once: the moment buffers live as long as the optimizer, so later steps only refresh the step
        count (one tensor shared by the group's entries) unless the entries were replaced meanwhile."""
        probe = getattr(fs, "published", None)
        if probe is not None:
            st = optimizer.state.get(probe[0])
            if st is not None and st.get(probe[1]) is probe[2] and probe[3] == fs.m.data_ptr():
                fs.step_t.fill_(float(fs.step))
                return
        fs.step_t = torch.tensor(float(fs.step))
        key = "exp_avg" if optimizer._rannc_kind == "adam" else "momentum_buffer"
        fs.published = None
        for i, p in enumerate(g.params):
            target = g.master_params[i] if (g.flat_master is not None and g.master_params) else p
            if target is None or g.opt_group[i] < 0:
                continue
            a, b = g.local_range(i)
            if b <= a:
                continue
            la = g.to_local(a)
            st = optimizer.state[target]
            # a parameter cut by a slice boundary keeps its state as a flat piece
            shp = target.shape if (b - a) == target.numel() else (b - a,)
            if optimizer._rannc_kind == "adam":
                st["step"] = fs.step_t
                st["exp_avg"] = fs.m[la:la + (b - a)].view(shp)
                st["exp_avg_sq"] = fs.v[la:la + (b - a)].view(shp)
            else:
                st["momentum_buffer"] = fs.m[la:la + (b - a)].view(shp)
            if fs.published is None:
                fs.published = (target, key, st[key], fs.m.data_ptr())

    optimizer._rannc_publish_state = _publish_state

    def _offloaded_update(g, fs, hp, og, a, b, kind, ctrl):
        """Streams [a, b) of the host-resident fp32 state through the device in chunks."""
        from .ops import kernels as K

        win = getattr(storage, "_offload_window", None)
        if win is None:
            chunk = max(1 << 20, int(conf("offload_chunk_numel")))
            win = storage._offload_window = _OffloadWindow(g.device, chunk, 3)
        la, n = g.to_local(a), b - a
        hosts = [g.flat_master[la:la + n], fs.m[la:la + n]]
        if kind == "adam":
            hosts.append(fs.v[la:la + n])

        streamed = getattr(g, "streamed", False)

        def kernel(off, cnt, dev, dev_in, dev_out):
            grad = dev_in[0] if streamed else g.flat_grad[a + off:a + off + cnt]
            model16 = dev_out[0] if streamed else g.flat_param[a + off:a + off + cnt]
            if kind == "adam":
                b1, b2 = hp["betas"]
                K.adam_flat(dev[0], grad, dev[1], dev[2], model16, float(hp["lr"]), b1, b2, float(hp["eps"]),
                            float(hp["weight_decay"]), fs.step, type(optimizer) is torch.optim.AdamW, ctrl)
            else:
                K.sgd_flat(dev[0], grad, dev[1], model16, float(hp["lr"]), float(hp["momentum"]),
                           float(hp.get("dampening", 0.0)), float(hp["weight_decay"]), bool(hp.get("nesterov")),
                           fs.step == 1, ctrl)

        if streamed:
            # gradients come from and the new 16-bit values go to host memory as well
            storage.wait_streamed()
            win.run(hosts, b - a, kernel, ins=[g.flat_grad[a:b]], outs=[g.flat_param[a:b]])
            return
        win.run(hosts, b - a, kernel)

    def fused_step(ctrl=None, only=None):
        from .ops import kernels as K

        kind = optimizer._rannc_kind
        for g in storage.groups:
            if only is not None and g not in only:
                continue
            fs = optimizer._rannc_flat_state.get(id(g))
            if fs is None:
                fs = optimizer._rannc_flat_state[id(g)] = _FlatState(
                    g.local_len, g.device, kind, host=_state_on_host(g))
            fs.step += 1
        for g, og, a, b in _flat_ranges():
            if only is not None and g not in only:
                continue
            fs = optimizer._rannc_flat_state[id(g)]
            hp = optimizer.param_groups[og]
            la, n = g.to_local(a), b - a
            is_amp = g.flat_master is not None
            if _state_on_host(g):
                _offloaded_update(g, fs, hp, og, a, b, kind, ctrl)
                continue
            master = g.flat_master[la:la + n] if is_amp else g.flat_param[a:b]
            model16 = g.flat_param[a:b] if is_amp else None
            grad = g.flat_grad[a:b]
            if kind == "adam":
                b1, b2 = hp["betas"]
                K.adam_flat(master, grad, fs.m[la:la + n], fs.v[la:la + n], model16, float(hp["lr"]), b1,
                            b2, float(hp["eps"]), float(hp["weight_decay"]), fs.step,
                            type(optimizer) is torch.optim.AdamW, ctrl)
            else:
                K.sgd_flat(master, grad, fs.m[la:la + n], model16, float(hp["lr"]), float(hp["momentum"]),
                           float(hp.get("dampening", 0.0)), float(hp["weight_decay"]), bool(hp.get("nesterov")),
                           fs.step == 1, ctrl)
        for g in storage.groups:
            if only is not None and g not in only:
                continue
            fs = optimizer._rannc_flat_state.get(id(g))
            if fs is not None:
                _publish_state(g, fs)

    def step(self, closure=None):
        mod = optimizer._rannc_module
        red = getattr(mod, "_fused_reducer", None)
        if red is not None and red.pending and mod._needs_grad_norm():
            # clipping / fp16 overflow checks need the reduced gradients first: the reduction launches that have
            # not run yet run now, without the update (the full-precision groups were reduced when backward
            # finished)
            red.ensure_reduced(sticky=False)
        ctrl = mod._amp_prepare_step() if mod is not None else None
        if ctrl is False:
            if red is not None and red.pending:
                red.skip_step()
            return None  # overflow: skipped, scale already lowered
        if red is not None and red.pending:
            # reduce-scatter + update + all-gather over peer memory, bucket by bucket (most of it already ran
            # while backward was in flight)
            plain = list(red.plain_groups)
            red.step(ctrl if isinstance(ctrl, torch.Tensor) else None)
            red.publish_state()
            if plain:
                # full-precision groups: gradients were reduced by the collective path, update them here
                fused_step(ctrl if isinstance(ctrl, torch.Tensor) else None, only=plain)
                if storage.zero:
                    storage.allgather_params_zero(only=plain)
            RF.bump_param_epoch()
            mod._after_step()
            return None
        use_fused = optimizer._rannc_kind is not None and all(
            (g.flat_grad.is_cuda or (g.streamed and g.device.type == "cuda")) and g.flat_grad.dtype == torch.float32
            for g in storage.groups)
        storage.wait_streamed(host=not use_fused)
        if use_fused:
            fused_step(ctrl if isinstance(ctrl, torch.Tensor) else None)
            loss = None
        else:
            if isinstance(ctrl, torch.Tensor):
                mul = float(ctrl[0].item())
                if mul != 1.0:
                    for g in storage.groups:
                        g.flat_grad.mul_(mul)
            loss = orig_step(closure) if closure is not None else orig_step()
            if amp:
                for g in storage.groups:
                    if g.flat_master is not None:
                        g.scatter_local(g.flat_param, g.flat_master)
        if storage.zero:
            storage.allgather_params_zero()
        RF.bump_param_epoch()
        if mod is not None:
            mod._after_step()
        return loss

    def zero_grad(self, set_to_none: bool = False):
        storage.zero_grad()

    def state_dict(self, from_global: bool = False, **kwargs):
        if not from_global:
            return orig_state_dict()
        return gather_optimizer_state_dict(optimizer, **kwargs)

    def load_state_dict(self, state_dict, from_global: bool = False, **kwargs):
        if not from_global:
            return orig_load_state_dict(state_dict)
        return load_global_optimizer_state(optimizer, state_dict)

    optimizer.step = types.MethodType(step, optimizer)
    optimizer.zero_grad = types.MethodType(zero_grad, optimizer)
    optimizer.state_dict = types.MethodType(state_dict, optimizer)
    optimizer.load_state_dict = types.MethodType(load_state_dict, optimizer)
    return optimizer


def gather_optimizer_state_dict(optimizer, root: int = 0, to_cpu: bool = True) -> Optional[dict]:
    """Collective over the world.  Returns the global state dict on ``root``, None elsewhere.  ``state`` is keyed
    by the parameter's position in the traversal of the original param groups -- the numbers
    ``param_groups[*]['params']`` hold -- so the dict loads into a plain ``torch.optim`` optimizer built the same
    way (reference: pyrannc/opt.py:98-157)."""
    mod = optimizer._rannc_module
    storage = mod._storage
    me = comm.get_rank()
    state = {}
    for name, order in sorted(optimizer._rannc_order_by_name.items(), key=lambda kv: kv[1]):
        ranks = storage.param_ranks.get(name)
        if ranks is None:
            continue
        # item names and non-tensor items from the first rank that holds state for this parameter (under ZeRO
        # the lowest owner may hold none of it: the parameter can lie wholly in other ranks' slices)
        items = None
        if name in storage.by_name:
            g, i = storage.by_name[name]
            target = g.master_params[i] if (g.flat_master is not None and g.master_params) else g.params[i]
            st = optimizer.state.get(target, {}) if target is not None else {}
            if st:
                items = {k: (("tensor", None) if _per_element(k, v) else ("value", _plain(v)))
                         for k, v in st.items()}
        items = next((x for x in comm.allgather_obj(items) if x), None)
        if not items:
            continue
        entry = {}
        p_shape, _ = mod._param_meta[name]
        for k, (kind, val) in items.items():
            if kind == "value":
                entry[k] = val
                continue
            # tensor item: assemble inside the owner set (slices under ZeRO), then hand to root
            full = _gather_state_tensor(storage, optimizer, name, k, p_shape, root)
            if me == root:
                entry[k] = full.cpu() if to_cpu else full
        if me == root:
            state[order] = entry
    if me != root:
        return None
    groups = []
    idx = 0
    for g in optimizer._rannc_orig_param_groups:
        ng = {k: v for k, v in g.items() if k != "params"}
        ng["params"] = list(range(idx, idx + len(g["params"])))
        idx += len(g["params"])
        groups.append(ng)
    return {"state": state, "param_groups": groups}


def _per_element(key, v) -> bool:
    """True for a state item with one entry per parameter element (moments, momentum buffers), including those
    of 0-dim parameters; the step counter is a tensor too but describes the whole parameter."""
    return torch.is_tensor(v) and key != "step"


def _plain(v):
    if torch.is_tensor(v):
        return v.item()
    return v


def _gather_state_tensor(storage, optimizer, name: str, key: str, shape, root: int = 0) -> Optional[torch.Tensor]:
    """Collective over the world: full fp32 tensor of optimizer-state item ``key`` of parameter ``name`` on
    ``root``.  The pieces are summed inside the parameter's owner set only (one [numel] all-reduce among the
    ranks that hold it); a rank outside the set takes part only when it is ``root``, by one point-to-point
    copy from the lowest owner."""
    ranks = storage.param_ranks[name]
    numel = 1
    for d in shape:
        numel *= d
    dev = comm.device()
    me = comm.get_rank()
    sl = storage.sliced.get(name)
    holders = tuple(sl) if sl else tuple(ranks)
    full = None
    if me in holders or me == root:
        full = torch.zeros(numel, dtype=torch.float32, device=dev)
    if name in storage.by_name:
        g, i = storage.by_name[name]
        target = g.master_params[i] if (g.flat_master is not None and g.master_params) else g.params[i]
        if target is not None and target in optimizer.state and key in optimizer.state[target]:
            a, b = g.local_range(i)
            lo, _ = g.param_range(i)
            if sl:
                # a tensor-partitioned weight: every holder contributes its column block
                ks = shape[1] // len(sl)
                idx = sl.index(me)
                full.view(shape)[:, idx * ks:(idx + 1) * ks] = \
                    optimizer.state[target][key].reshape(shape[0], ks).to(dev, torch.float32)
            elif g.zero or me == ranks[0]:
                full[a - lo:b - lo] = optimizer.state[target][key].reshape(-1).to(dev, torch.float32)
    if comm.get_world_size() > 1:
        if len(holders) > 1 and me in holders:
            comm.allreduce(full, "sum", holders)
        if root not in holders:
            # a checkpoint root outside the owner set gets the assembled tensor from the lowest owner
            comm.send_recv(full, holders[0], root)
    return full.view(shape) if full is not None else None


def load_global_optimizer_state(optimizer, sd: dict) -> None:
    """Takes a dict made by ``state_dict(from_global=True)`` (present on every rank) and keeps the
    slices this rank owns."""
    mod = optimizer._rannc_module
    storage = mod._storage
    for hp_new, hp in zip(sd["param_groups"], optimizer.param_groups):
        for k, v in hp_new.items():
            if k != "params":
                hp[k] = v
    order_to_name = {o: n for n, o in optimizer._rannc_order_by_name.items()}
    steps = {}
    for order, entry in sd["state"].items():
        name = order_to_name.get(int(order))
        if name is None or name not in storage.by_name:
            continue
        g, i = storage.by_name[name]
        target = g.master_params[i] if (g.flat_master is not None and g.master_params) else g.params[i]
        if target is None:
            continue
        a, b = g.local_range(i)
        lo, _ = g.param_range(i)
        st = optimizer.state[target]
        sl = storage.sliced.get(name)
        for k, v in entry.items():
            if _per_element(k, v):
                if sl:
                    ks = v.shape[1] // len(sl)
                    idx = sl.index(comm.get_rank())
                    v = v[:, idx * ks:(idx + 1) * ks].contiguous()
                piece = v.reshape(-1)[a - lo:b - lo].to(target.device, torch.float32)
                if piece.numel() == target.numel():
                    piece = piece.view(target.shape)
                st[k] = piece.clone()
            else:
                st[k] = torch.tensor(float(v)) if k == "step" else v
                if k == "step":
                    steps[id(g)] = int(float(v))
    # the fused step keeps flat moments: refill them from the per-parameter entries
    if optimizer._rannc_kind is not None:
        for g in storage.groups:
            fs = _FlatState(g.local_len, g.device, optimizer._rannc_kind, host=_state_on_host(g))
            fs.step = steps.get(id(g), 0)
            for i, p in enumerate(g.params):
                target = g.master_params[i] if (g.flat_master is not None and g.master_params) else p
                if target is None or target not in optimizer.state:
                    continue
                a, b = g.local_range(i)
                if b <= a:
                    continue
                la, n = g.to_local(a), b - a
                st = optimizer.state[target]
                if optimizer._rannc_kind == "adam" and "exp_avg" in st:
                    fs.m[la:la + n] = st["exp_avg"].reshape(-1)
                    fs.v[la:la + n] = st["exp_avg_sq"].reshape(-1)
                elif "momentum_buffer" in st and st["momentum_buffer"] is not None:
                    fs.m[la:la + n] = st["momentum_buffer"].reshape(-1)
            optimizer._rannc_flat_state[id(g)] = fs
