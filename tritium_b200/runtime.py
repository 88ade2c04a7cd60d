"""Backend registry in the shape of tritium-runtime (crates/tritium-runtime/src/lib.rs:74-203).

A backend appears under ``list_backends`` iff its entry is registered and its ``init`` succeeds;
a failing ``init`` is skipped with a line on stderr, as ``Registry::init`` does (:148-166).
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Callable

from .backend import B200Backend
from .errors import BackendError


@dataclass(frozen=True)
class BackendEntry:
    name: str
    init: Callable[[], B200Backend]


def _init_b200() -> B200Backend:
    return B200Backend(0)


BACKENDS: list[BackendEntry] = [BackendEntry("b200", _init_b200)]


class Registry:
    def __init__(self, backends: dict):
        self._backends = backends

    @classmethod
    def init(cls) -> "Registry":
        live = {}
        for entry in BACKENDS:
            try:
                live[entry.name] = entry.init()
            except BackendError as err:  # a missing device is not fatal to the registry
                print(f"tritium-runtime: backend `{entry.name}` unavailable: {err}", file=sys.stderr)
        return cls(live)

    def names(self) -> list:
        return sorted(self._backends)

    def get(self, name: str):
        return self._backends.get(name)


def list_backends() -> list:
    """The lines ``tritium list-backends`` prints (crates/tritium-cli/src/backends.rs:18-53)."""
    lines = []
    reg = Registry.init()
    for name in reg.names():
        caps = reg.get(name).capabilities()
        lines.append(f"{caps.backend} — {caps.device_name}")
        lines.append(f"  features: {', '.join(caps.features)}")
        lines.append(f"  memory: {caps.total_memory_bytes} bytes")
    return lines
