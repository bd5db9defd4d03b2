"""Mixed precision for wrapped models (the reference delegates this to NVIDIA Apex O2,
pyrannc/amp/__init__.py:1-70; Apex is not a dependency here).

What the middleware needs from "amp", and provides itself:

* 16-bit model parameters with fp32 master copies that the optimizer updates
  (``RaNNCModule(..., enable_apex_amp=True)`` keeps its name for compatibility);
* dynamic loss scaling for fp16 with the overflow decision AGREED ACROSS RANKS:
  the overflow flag is summed and the scale minimised over the world, exactly
  like the reference's patched Apex scaler (pyrannc/amp/__init__.py:44-65);
* bf16 mode (the default on B200) needs no loss scale.
"""
from __future__ import annotations

import contextlib
from typing import Iterator, Tuple

import torch

from ..parallel import comm

_amp_dtype = torch.bfloat16


def set_dtype(dtype: torch.dtype) -> None:
    """16-bit type used for model parameters and activations: ``torch.bfloat16`` (default) or ``torch.float16``."""
    global _amp_dtype
    if dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("amp dtype must be bfloat16 or float16")
    _amp_dtype = dtype


def get_dtype() -> torch.dtype:
    return _amp_dtype


class LossScaler:
    """Dynamic loss scale: halve on overflow, double after ``growth_interval`` clean steps."""

    def __init__(self, init_scale: float = 2.0 ** 16, growth_interval: int = 2000, min_scale: float = 1.0,
                 max_scale: float = 2.0 ** 24, dynamic: bool = True):
        self._loss_scale = float(init_scale)
        self.growth_interval = growth_interval
        self.min_scale, self.max_scale = min_scale, max_scale
        self.dynamic = dynamic
        self._unskipped = 0

    def loss_scale(self) -> float:
        return self._loss_scale

    def update_scale(self, had_overflow: bool) -> bool:
        """Shares the overflow decision with every rank; returns True when the step must be skipped."""
        if comm.get_world_size() > 1:
            flag = torch.tensor([1 if had_overflow else 0], dtype=torch.int32, device=comm.device())
            comm.allreduce(flag, "sum")
            had_overflow = bool(flag.item() > 0)
        if had_overflow and self.dynamic:
            self._loss_scale = max(self.min_scale, self._loss_scale / 2.0)
            if comm.get_world_size() > 1:
                s = torch.tensor([self._loss_scale], dtype=torch.float32, device=comm.device())
                comm.allreduce(s, "min")
                self._loss_scale = float(s.item())
            self._unskipped = 0
            return True
        if had_overflow:
            return True
        self._unskipped += 1
        if self.dynamic and self._unskipped >= self.growth_interval:
            self._loss_scale = min(self.max_scale, self._loss_scale * 2.0)
            self._unskipped = 0
        return False


_scaler = LossScaler(init_scale=1.0, dynamic=False)


def get_scaler() -> LossScaler:
    return _scaler


def set_scaler(s: LossScaler) -> None:
    global _scaler
    _scaler = s


def initialize(model, optimizer=None, opt_level: str = "O2", dtype: torch.dtype = None, loss_scale="dynamic"):
    """Apex-style entry point: picks the 16-bit type and the loss scaler; the cast itself happens when the
    model is wrapped with ``enable_apex_amp=True``."""
    if dtype is not None:
        set_dtype(dtype)
    if get_dtype() == torch.float16:
        if loss_scale == "dynamic":
            set_scaler(LossScaler())
        else:
            set_scaler(LossScaler(init_scale=float(loss_scale), dynamic=False))
    else:
        set_scaler(LossScaler(init_scale=1.0, dynamic=False))
    return (model, optimizer) if optimizer is not None else model


@contextlib.contextmanager
def scale_loss(loss, optimizer=None):
    """``with amp.scale_loss(loss, opt) as scaled: scaled.backward()``"""
    s = _scaler.loss_scale()
    yield loss * s if s != 1.0 else loss


def master_params(optimizer) -> Iterator[torch.nn.Parameter]:
    for g in optimizer.param_groups:
        yield from g["params"]


def named_master_params(model, optimizer=None, zero: bool = False) -> Iterator[Tuple[str, torch.nn.Parameter]]:
    """(name, fp32 master tensor) pairs of the parameters this rank updates (the local segment under ZeRO)."""
    storage = model._storage
    for g in storage.groups:
        for i, name in enumerate(g.names):
            if g.flat_master is None:
                yield name, g.params[i]
            elif g.master_params[i] is not None:
                yield name, g.master_params[i]


def register_amp_params(optimizer) -> None:
    """Kept for source compatibility: master parameters are registered when the model is deployed."""


def unset_master_grads(optimizer) -> None:
    """Gradients live in flat buffers owned by the middleware; clearing is ``optimizer.zero_grad()``."""
    optimizer.zero_grad()
