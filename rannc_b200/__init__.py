"""rannc_b200: automatic model partitioning middleware for PyTorch on B200.

Public API (same names as the reference's ``pyrannc`` package, pyrannc/__init__.py):
``RaNNCModule``, ``get_rank``, ``get_world_size``, ``barrier``, ``clear``,
``delay_grad_allreduce``, ``keep_graph``, ``sync_params_on_init``,
``recreate_all_communicators``, ``show_deployment``, ``_dump_events``, ``_run_dp_dry``.
"""
__version__ = "0.1.0"


def _load_core():
    import importlib

    try:
        return importlib.import_module("rannc_b200._core")
    except ImportError:
        from . import build

        build.build_core()
        return importlib.import_module("rannc_b200._core")


_core = _load_core()

import atexit as _atexit  # noqa: E402
import logging as _logging  # noqa: E402

from .utils import config as _config  # noqa: E402
from .utils import log as _log  # noqa: E402

_log.configure(_core.config_get("conf_dir"))
if _core.config_get("show_config_items"):
    print(_config.show())
for _w in _core.config_warnings():
    _logging.getLogger("rannc").warning(_w)

from .parallel import comm as _comm  # noqa: E402
from .module import (RaNNCModule, delay_grad_allreduce, keep_graph, sync_params_on_init)  # noqa: E402,F401
from . import amp, tensor_coll, comm_utils, utils  # noqa: E402,F401
from .tensor_coll import all_gather  # noqa: E402,F401  (re-exported by the reference: pyrannc/__init__.py:30)
from .dist_param import (DistributeModelParams, store_dist_param, load_dist_param, set_dist_param,  # noqa: E402,F401
                         get_dist_param_range, set_dist_param_dtype, get_dist_param_segment, remove_dist_param,
                         dist_param_registered)
from .opt import patch_optimizer  # noqa: E402,F401


def get_rank() -> int:
    return _comm.get_rank()


def get_world_size() -> int:
    return _comm.get_world_size()


def barrier() -> None:
    _comm.barrier()


def clear() -> None:
    """Undeploys every module and destroys the communicators (reference: main.cpp:47-53)."""
    from . import module as _m

    for mod in list(_m._live_modules):
        mod.undeploy()
    _comm.clear()


def recreate_all_communicators() -> None:
    _comm.recreate_all_communicators()


def _dump_events(path: str = None) -> None:
    """Gathers every rank's event trace and writes one Chrome-trace JSON on rank 0
    (reference: src/comp/EventRecorder.cpp:49-99)."""
    frags = _comm.allgather_obj(_core.trace_dump_local(_comm.get_rank()))
    if _comm.get_rank() == 0:
        with open(path or _core.config_get("event_trace_file"), "w") as f:
            f.write(_core.trace_merge(frags))


def _run_dp_dry(path: str, dev_num=None, dev_mem=None):
    """Re-runs only the stage search from a dumped cache, without a GPU (reference: main.cpp:412-421)."""
    with open(path, "rb") as f:
        return _core.run_dp_dry(f.read(), dev_num, dev_mem)


def abort_all_processes() -> None:
    """Ends this process at once with a failure code; the launcher takes the other ranks down (reference:
    MPI_Abort on the world communicator, src/main.cpp:510-515)."""
    import os
    import sys

    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(1)


def show_deployment(path: str, batch_size: int) -> str:
    """Prints the stages of a saved deployment and the per-rank micro-batch sizes (reference: main.cpp:423-470)."""
    with open(path, "rb") as f:
        dep, world, dev_mem = _core.load_deployment(f.read())
    lines = [str(dep), f"world_size={world} dev_mem={dev_mem}"]
    calc = _core.BatchSizeCalculator(dep.pipeline_num, batch_size)
    for name in dep.fwd_graph_order:
        ranks = sorted(dep.allocation[name])
        for i, r in enumerate(ranks):
            sizes = [calc.local_split_size(i, len(ranks), s) for s in range(dep.pipeline_num)]
            lines.append(f"  {name} rank {r}: micro-batch sizes {sizes}")
    text = "\n".join(lines)
    print(text)
    return text


def _exit_handler():
    try:
        if _core.trace_enabled() and _core.trace_size() > 0 and _comm.get_world_size() == 1:
            _dump_events()
    except Exception:  # noqa: BLE001
        pass


_atexit.register(_exit_handler)
