"""rannc_b200: automatic model partitioning middleware for PyTorch on B200."""
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
