"""Drop-in name for scripts written against the reference package: ``import pyrannc`` gives the
``rannc_b200`` API (``RaNNCModule``, ``get_rank``, ``barrier``, ``delay_grad_allreduce``, ...), and the
sub-modules ``pyrannc.amp``, ``pyrannc.opt``, ``pyrannc.dist_param``, ``pyrannc.tensor_coll``,
``pyrannc.comm_utils`` and ``pyrannc.utils`` are the ones of ``rannc_b200``
(reference: pyrannc/__init__.py, pyrannc/amp/__init__.py, pyrannc/opt.py, pyrannc/dist_param.py,
pyrannc/tensor_coll.py, pyrannc/comm_utils.py, pyrannc/utils.py)."""
import sys as _sys

import rannc_b200 as _impl
from rannc_b200 import *  # noqa: F401,F403
from rannc_b200 import amp, comm_utils, dist_param, opt, tensor_coll, utils  # noqa: F401

for _name in ("amp", "comm_utils", "dist_param", "opt", "tensor_coll", "utils"):
    _sys.modules[__name__ + "." + _name] = getattr(_impl, _name)
__all__ = getattr(_impl, "__all__", [n for n in dir(_impl) if not n.startswith("_")])
__version__ = getattr(_impl, "__version__", "0")
