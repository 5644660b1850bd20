"""B200-native kernels behind the ``miles_ext_kernels`` plug-in surface.

The package mirrors the process-level API of the reference (reference: miles_ext_kernels/__init__.py:22-52): kernels
are grouped by source (:data:`SOURCES`, one namespace each), and miles calls four hooks -- :func:`add_arguments`
before parsing, :func:`validate_args` on the parsed namespace, :func:`configure` in every worker, :func:`release`
before it sleeps or offloads.  Each forwards to the ``_runtime`` of every source.  An op is imported at miles'
dispatch seam, e.g. ``from miles_ext_kernels_b200.cake.gdn import chunk_gated_delta_rule``.

Every import inside the package is relative, so the directory also works under the name ``miles_ext_kernels``.
Importing this module imports neither torch, the native library nor any op.

The hook names and signatures are the public interface of radixark/miles-ext-kernels (Apache-2.0; see NOTICE): a
drop-in has to match them.
"""

from __future__ import annotations

from argparse import ArgumentParser, Namespace
from collections.abc import Mapping
from importlib import import_module
from types import ModuleType
from typing import Any

__all__ = ["SOURCES", "add_arguments", "configure", "release", "validate_args"]

SOURCES = ("cake",)


def _runtimes() -> list[ModuleType]:
    return [import_module(f"{__name__}.{source}._runtime") for source in SOURCES]


def add_arguments(parser: ArgumentParser) -> None:
    """Register every source's arguments in one ``miles-ext-kernels`` argument group."""
    group = parser.add_argument_group("miles-ext-kernels")
    for runtime in _runtimes():
        runtime.add_arguments(group)


def validate_args(args: Namespace) -> None:
    """Check the parsed flat namespace and fill in the values left to defaults (raises ``ValueError``)."""
    for runtime in _runtimes():
        runtime.validate_args(args)


def configure(args: Namespace | Mapping[str, Any] | None = None, /, **values: Any) -> None:
    """Configure this process from the resolved values; replaces the previous configuration."""
    for runtime in _runtimes():
        runtime.configure(args, **values)


def release() -> int:
    """Free every source's pooled scratch and cached plans; returns the bytes freed from the pools."""
    return sum(runtime.release() for runtime in _runtimes())
