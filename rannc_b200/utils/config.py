"""Python face of the native configuration store.

Items, defaults, ``<conf_dir>/rannc_conf.toml`` and ``RANNC_<NAME>`` environment
overrides are handled in ``csrc/core/runtime_util.cpp`` (same items as the
reference's src/Config.cpp:133-280, plus this runtime's own)."""
from __future__ import annotations

from .. import _core


def conf(name: str):
    return _core.config_get(name)


def set_conf(name: str, value) -> None:
    if isinstance(value, bool):
        value = "true" if value else "false"
    _core.config_set(name, str(value))


def reload() -> None:
    _core.config_reload()


def items() -> dict:
    return dict(_core.config_items())


def show() -> str:
    return "\n".join(f" {k}={v[0]}" for k, v in sorted(items().items()))
