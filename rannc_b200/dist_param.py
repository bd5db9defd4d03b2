"""Parameter sharding at model construction (``dist_param``).

Same purpose and API as the reference's ``pyrannc/dist_param.py`` and
``DistributedParamLocator`` (src/comp/DistributedParamLocator.cpp:13-82): inside
``with DistributeModelParams():`` every parameter is cut to this rank's 1/world
segment right after its module is constructed, so a model that does not fit in
one host's memory can still be declared on every rank.  Segments are
``aligned_numel / world`` long with the 16-byte x ranks alignment of
``segment_range`` (csrc/core/deployment.cpp), so the last ranks may hold short or
empty segments.

What differs from the reference: tracing runs on fake tensors (``torch.export``),
which needs shapes but no values, so nothing is gathered while tracing -- the
sharded parameter keeps its full *shape* through a stride-0 view of a single
element and the reference's gather / re-shard forward hooks
(pyrannc/dist_param.py:109-132) are not needed.  The full values are assembled
once, at deployment, directly on the ranks that own the parameter.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from . import _core
from .parallel import comm


class _Entry:
    __slots__ = ("shape", "dtype", "numel", "segment", "begin", "end", "param")

    def __init__(self, shape, dtype, numel, segment, begin, end, param):
        self.shape, self.dtype, self.numel = shape, dtype, numel
        self.segment, self.begin, self.end, self.param = segment, begin, end, param


_registry: Dict[int, _Entry] = {}


def _pid(p) -> int:
    return p if isinstance(p, int) else id(p)


def _esize(dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def store_dist_param(p: torch.Tensor) -> int:
    """Keeps only this rank's segment of ``p``; ``p`` keeps its shape but no longer its values."""
    world, rank = comm.get_world_size(), comm.get_rank()
    numel = p.numel()
    begin, end = _core.segment_range(numel, _esize(p.dtype), world, rank)
    seg = p.data.reshape(-1)[begin:end].clone()
    shape = tuple(p.shape)
    _registry[id(p)] = _Entry(shape, p.dtype, numel, seg, begin, end, p)
    p.data = torch.zeros(1, dtype=p.dtype, device=p.device).expand(shape) if numel > 0 else p.data
    return id(p)


def dist_param_registered(pid) -> bool:
    return _pid(pid) in _registry


def get_dist_param_segment(pid) -> torch.Tensor:
    return _registry[_pid(pid)].segment


def get_dist_param_range(pid) -> Tuple[int, int]:
    e = _registry[_pid(pid)]
    return e.begin, e.end


def set_dist_param_dtype(pid, dtype: torch.dtype) -> None:
    e = _registry[_pid(pid)]
    e.segment = e.segment.to(dtype)
    e.dtype = dtype


def load_dist_param(pid, device: Optional[torch.device] = None) -> torch.Tensor:
    """Collective over the world: the full parameter, assembled from every rank's segment
    (reference: all-gather + ``.cpu()``, DistributedParamLocatorBase.cpp:96-153)."""
    e = _registry[_pid(pid)]
    world = comm.get_world_size()
    dev = device or comm.device()
    seg_len = _core.aligned_numel(e.numel, _esize(e.dtype), world) // world
    mine = torch.zeros(seg_len, dtype=e.dtype, device=dev)
    mine[: e.end - e.begin] = e.segment.to(dev)
    full = torch.empty(seg_len * world, dtype=e.dtype, device=dev)
    comm.allgather_into(full, mine)
    return full[: e.numel].view(e.shape)


def set_dist_param(pid, src: torch.Tensor) -> None:
    """Re-shards from a full tensor (every rank passes the same values)."""
    e = _registry[_pid(pid)]
    e.segment = src.detach().reshape(-1)[e.begin:e.end].to(e.dtype).clone()


def remove_dist_param(pid) -> None:
    _registry.pop(_pid(pid), None)


def materialize(p: torch.nn.Parameter, keep: bool, device: torch.device) -> None:
    """Collective: rebuilds the full value of a sharded parameter on the ranks that keep it."""
    full = load_dist_param(id(p), device)
    if keep:
        p.data = full.clone()
    remove_dist_param(id(p))


class DistributeModelParams:
    """``with DistributeModelParams(enable=True): model = Net()`` -- shards each parameter (and float
    buffer) as soon as the module that owns it has been constructed."""

    def __init__(self, enable: bool = True):
        self.enable = enable
        self._patched = []

    @staticmethod
    def _all_subclasses(cls):
        seen, stack = set(), [cls]
        while stack:
            c = stack.pop()
            for s in c.__subclasses__():
                if s not in seen:
                    seen.add(s)
                    stack.append(s)
        return seen

    def __enter__(self):
        if not self.enable:
            return self
        comm.start()

        def wrap(cls):
            orig = cls.__dict__.get("__init__")
            if orig is None:
                return

            def patched(mod, *args, __orig=orig, **kwargs):
                __orig(mod, *args, **kwargs)
                for p in mod.parameters(recurse=False):
                    if not dist_param_registered(id(p)):
                        store_dist_param(p)

            cls.__init__ = patched
            self._patched.append((cls, orig))

        for c in self._all_subclasses(torch.nn.Module):
            wrap(c)
        return self

    def __exit__(self, *exc):
        for cls, orig in self._patched:
            cls.__init__ = orig
        self._patched.clear()
        return False
