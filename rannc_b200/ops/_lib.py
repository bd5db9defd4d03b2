"""ctypes access to ``_kernels.so`` (the sm_100a CUDA kernels).

The library is built in-tree by :mod:`rannc_b200.build`.  When it is missing it
is built on first use; when that is impossible the import of any kernel fails
with an error instead of falling back to a stock PyTorch path.
"""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent.parent
_lock = threading.Lock()
_lib = None

# device kernels launched per C entry point (the optimizer / element-wise entries launch one)
_KERNELS_PER_CALL = {"rb_bn_fwd": 3, "rb_bn_bwd": 3, "rb_ln_bwd": 2, "rb_xent_fwd": 2, "rb_attn_bwd": 3, "rb_read_error": 0, "rb_ln_supported": 0,
                     "rb_ln_bwd_grid": 0, "rb_error_peek_async": 0}
_launches = 0


class _Counting:
    """Forwards attribute access to the CDLL and counts kernel launches per call."""

    def __init__(self, dll):
        object.__setattr__(self, "_dll", dll)
        object.__setattr__(self, "_cache", {})

    def __getattr__(self, name):
        cache = object.__getattribute__(self, "_cache")
        fn = cache.get(name)
        if fn is None:
            raw = getattr(object.__getattribute__(self, "_dll"), name)
            n = _KERNELS_PER_CALL.get(name, 1)

            def fn(*a, __raw=raw, __n=n):
                global _launches
                _launches += __n
                return __raw(*a)

            fn.raw = raw
            cache[name] = fn
        return fn


def launch_count() -> int:
    """Kernels of this library launched so far in this process."""
    return _launches


class KernelLibraryError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        import os

        debug = os.environ.get("RANNC_KERNEL_DEBUG", "0") == "1"
        path = _HERE / ("_kernels_debug.so" if debug else "_kernels.so")
        if not path.exists():
            from .. import build

            try:
                build.build_kernels(debug=debug)
            except Exception as e:  # noqa: BLE001
                raise KernelLibraryError(f"cannot build {path}: {e}") from e
        try:
            _lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelLibraryError(f"cannot load {path}: {e}") from e
        _lib.rb_read_error.restype = ctypes.c_int
        _lib = _Counting(_lib)
        return _lib


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_cur_device = getattr(torch._C, "_cuda_getDevice", None)


def stream_ptr() -> ctypes.c_void_p:
    """The current stream of the current device.  Asked of the C layer directly: ``torch.cuda.current_stream``
    spends some 15 us per call on device-index bookkeeping, which at hundreds of launches per step was a third
    of the host time of a step."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(_cur_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t):
    """Device address as an int (None for a missing tensor); for ctypes.Structure fields."""
    return None if t is None else t.data_ptr()


def vp(t) -> ctypes.c_void_p:
    """Device address as c_void_p; for positional arguments of a C function."""
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelLibraryError(f"{what} failed with code {rc}")


def read_error(clear: bool = True) -> int:
    """Device error word (synchronises): 0 ok, 1 mbarrier wait ran out, 2 peer wait ran out."""
    return int(lib().rb_read_error(1 if clear else 0))


class ErrorPeek:
    """Watches the device error word without synchronising: after every optimizer step an asynchronous copy of
    the word into pinned host memory is enqueued, and the copy made one step earlier -- complete by then -- is
    looked at.  A kernel that gave up on a wait is therefore noticed within one step instead of at the next
    checkpoint (reference: syncWithErrorCheck polls after every forward / backward,
    src/comm/NCCLWrapper.cpp:575-622)."""

    def __init__(self):
        self.host = torch.zeros(2, dtype=torch.int32).pin_memory()
        self.events = [None, None]
        self.k = 0

    def poll(self) -> int:
        """Enqueues this step's copy; returns the newest completed earlier value (0: no error seen)."""
        seen = 0
        for i in (0, 1):
            ev = self.events[i]
            if ev is not None and ev.query():
                seen = max(seen, int(self.host[i]))
                self.events[i] = None
        slot = self.k & 1
        if self.events[slot] is None:
            rc = lib().rb_error_peek_async(ctypes.c_void_p(self.host.data_ptr() + 4 * slot), stream_ptr())
            check(rc, "rb_error_peek_async")
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            self.events[slot] = ev
            self.k += 1
        return seen
