"""Named loggers routed through the native logger (levels from ``<conf_dir>/logging.toml``)."""
from __future__ import annotations

import os

from .. import _core

TRACE, DEBUG, INFO, WARN, ERROR, CRITICAL = range(6)


class Logger:
    def __init__(self, name: str):
        self.name = name

    def _log(self, lv, msg, *args):
        if _core.log_enabled(self.name, lv):
            _core.log(self.name, lv, msg % args if args else msg)

    def trace(self, msg, *a):
        self._log(TRACE, msg, *a)

    def debug(self, msg, *a):
        self._log(DEBUG, msg, *a)

    def info(self, msg, *a):
        self._log(INFO, msg, *a)

    def warning(self, msg, *a):
        self._log(WARN, msg, *a)

    def error(self, msg, *a):
        self._log(ERROR, msg, *a)


_loggers = {}


def get_logger(name: str) -> Logger:
    if name not in _loggers:
        _loggers[name] = Logger(name)
    return _loggers[name]


def configure(conf_dir: str) -> None:
    path = os.path.join(conf_dir, "logging.toml")
    if os.path.exists(path):
        with open(path) as f:
            _core.configure_logging_from_toml(f.read())
    lvl = os.environ.get("RANNC_LOG_LEVEL")
    if lvl:
        _core.set_log_level("", lvl)
