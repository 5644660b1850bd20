"""The argument surface of the ops and the configuration of this process.  Torch-free.

Four hooks are called by miles through the top-level package (reference: miles_ext_kernels/cake/_runtime/config.py:91-205):

- :func:`add_arguments` before parsing registers, for every op that has a miles selector, ``--cake-<op>-variant``
  (when the op ships two variants; hidden from the help when miles may pick only one) and the op's own options,
  then the runtime options (:data:`RUNTIME_FLAGS`);
- :func:`validate_args` on the parsed flat namespace rejects an option of an op that is not selected, resolves the
  variant of every selected op and writes it back, and runs the op's own check;
- :func:`configure` in every process that calls a kernel replaces the process configuration;
- ``release`` lives in :mod:`.registry`.

Variant rules.  ``det`` repeats bit for bit for identical inputs; ``fast`` may not.  A process that never configured
an op runs ``det`` (or the op's only variant).  On the command line an unset flag of a selected op resolves to
``fast`` when miles may choose it -- and to ``det`` under ``--deterministic-mode``, where an explicit ``fast`` is an
error and an op without ``det`` is rejected.  ``configure(..., deterministic_mode=True)`` applies the same rules to
direct callers.  ``--cake-deterministic`` is accepted as an alias of deterministic mode for this package's ops.

The configuration is one immutable mapping swapped whole by every :func:`configure`; :func:`variant` and
:func:`option` read it when a call runs.
"""

from __future__ import annotations

import argparse
import logging
from argparse import Namespace
from collections.abc import Mapping
from types import MappingProxyType
from typing import Any

from . import registry
from .spec import Flag, OpSpec

__all__ = [
    "RUNTIME_FLAGS",
    "add_arguments",
    "configure",
    "deterministic_mode",
    "option",
    "validate_args",
    "variant",
    "warn_runs_det",
]

# Options of the runtime itself; read with option(None, dest).
RUNTIME_FLAGS = (
    Flag(
        "--cake-workspace-pool-bytes",
        dict(
            type=int,
            default=0,
            help=(
                "Most bytes of scratch memory the ops keep per device between calls. 0 (default) keeps nothing: "
                "every scratch buffer is a fresh allocation. A positive bound reuses buffers across calls."
            ),
        ),
    ),
    Flag(
        "--cake-deterministic",
        dict(
            action="store_true",
            default=False,
            help=(
                "Run every cake op in its bit-reproducible 'det' variant (same effect on these ops as "
                "--deterministic-mode); rejects an explicit 'fast'."
            ),
        ),
    ),
)

logger = logging.getLogger("miles_ext_kernels")


class _Process:
    """What this process is configured to: one read-only mapping, replaced as a whole."""

    settings: Mapping[str, Any] = MappingProxyType({})
    warned: set[tuple[str, str]] = set()


def _selectable_ops() -> list[OpSpec]:
    """The ops miles can switch on from its command line, in registry order."""
    return [spec for spec in map(registry.op_spec, registry.OPS) if spec.selected_by]


def deterministic_mode(args: Any) -> bool:
    """Whether ``args`` asks for deterministic mode.

    miles' flat namespace carries Megatron's ``--deterministic-mode`` as ``args.deterministic_mode``; its typed
    configuration as ``args.backend.deterministic_mode``.  ``args.cake_deterministic`` (this package's alias) counts
    too.  Anything else is not deterministic mode.
    """
    if getattr(args, "cake_deterministic", False):
        return True
    flat = getattr(args, "deterministic_mode", None)
    if flat is not None:
        return bool(flat)
    return bool(getattr(getattr(args, "backend", None), "deterministic_mode", False))


def _variant_help(spec: OpSpec) -> str:
    preferred = "fast" if "fast" in spec.cli_choices else "det"
    return (f"Variant of the cake {spec.name} kernels ({spec.summary}) under {spec.selector}: 'det' repeats bit "
            f"for bit for identical inputs; 'fast' may give that up for speed (in this build both run the same "
            f"kernels, which reduce in a fixed order). Default: '{preferred}', or 'det' under --deterministic-mode, "
            "which rejects 'fast'.")


def add_arguments(parser: Any) -> None:
    """Register the ops' arguments and the runtime options on ``parser`` (a parser or an argument group)."""
    for spec in _selectable_ops():
        if spec.has_variant_flag:
            shown = _variant_help(spec) if spec.shows_variant_flag else argparse.SUPPRESS
            parser.add_argument(spec.variant_flag, choices=spec.cli_choices, default=None, help=shown)
        for own in spec.flags:
            parser.add_argument(own.name, **own.kwargs)
    for own in RUNTIME_FLAGS:
        parser.add_argument(own.name, **own.kwargs)


def _no_det(spec: OpSpec) -> ValueError:
    if spec.selector:
        return ValueError(f"the cake {spec.name} kernels have no det variant: {spec.selector} is not deterministic")
    return ValueError(f"the cake {spec.name} kernels have no det variant: it cannot run in deterministic mode")


def _pick_variant(spec: OpSpec, asked: str | None, deterministic: bool, from_cli: bool) -> str | None:
    """The variant of ``spec`` a configuration stands for.  An explicit request must be one the op ships (on the
    command line: one miles may choose) and must not be ``fast`` in deterministic mode; no request means ``det`` in
    deterministic mode, the command line's preference on the command line, and "unset" (``None``) otherwise."""
    if asked is not None:
        choices = spec.cli_choices if from_cli else spec.variants
        if asked not in choices:
            raise ValueError(f"{spec.variant_flag} must be one of {choices}, not {asked!r}")
        if asked == "fast" and deterministic:
            raise ValueError(f"{spec.variant_flag} fast is not bit-reproducible under --deterministic-mode: use det or "
                             "leave it unset")
        return asked
    if deterministic:
        if "det" in spec.variants:
            return "det"
        raise _no_det(spec)
    if from_cli:
        return "fast" if "fast" in spec.cli_choices else "det"
    return None


def _check_runtime(dest: str, value: Any) -> None:
    if dest == "cake_workspace_pool_bytes" and value < 0:
        raise ValueError(f"--cake-workspace-pool-bytes must be >= 0, not {value}")


def _is_selected(spec: OpSpec, args: Namespace) -> bool:
    return any(getattr(args, dest, None) == wanted for dest, wanted in spec.selected_by)


def _reject_stray_options(spec: OpSpec, args: Namespace) -> None:
    """An op that is not switched on must have none of its options set."""
    if spec.has_variant_flag and getattr(args, spec.variant_dest, None) is not None:
        raise ValueError(f"{spec.variant_flag} requires {spec.selector}")
    for own in spec.flags:
        if getattr(args, own.dest, own.default) != own.default:
            raise ValueError(f"{own.name} requires {spec.selector}")


def validate_args(args: Namespace) -> None:
    """Check miles' parsed flat namespace; write the resolved variant of every selected op back to it."""
    deterministic = deterministic_mode(args)
    for spec in _selectable_ops():
        if not _is_selected(spec, args):
            _reject_stray_options(spec, args)
            continue
        chosen = _pick_variant(spec, getattr(args, spec.variant_dest, None), deterministic, from_cli=True)
        if spec.has_variant_flag:
            setattr(args, spec.variant_dest, chosen)
        if spec.validate is not None:
            spec.validate(args)
    for own in RUNTIME_FLAGS:
        _check_runtime(own.dest, getattr(args, own.dest, own.default))


def _known_keys() -> tuple[dict[str, OpSpec], set[str]]:
    """``(variant key -> its op, every option key)`` over all ops and the runtime."""
    variants = {spec.variant_dest: spec for spec in map(registry.op_spec, registry.OPS)}
    options = {own.dest for own in RUNTIME_FLAGS}
    for spec in variants.values():
        options.update(own.dest for own in spec.flags)
    return variants, options


def configure(args: Namespace | Mapping[str, Any] | None = None, /, **values: Any) -> None:
    """Replace this process's configuration with the ``cake_*`` entries of ``args`` and ``values``.

    ``args``: a namespace, a mapping (miles' ``miles_ext_kernels_args``) or ``None``; ``values`` win over it.  ``None``
    counts as unset and keys that do not start with ``cake_`` are skipped, so a whole namespace may be passed.
    ``ValueError`` for an unknown ``cake_*`` key, for a variant the op does not ship, and for ``fast`` when
    deterministic mode is on.  Each call starts again from the defaults.
    """
    given = dict(args) if isinstance(args, Mapping) else ({} if args is None else dict(vars(args)))
    given.update(values)
    deterministic = deterministic_mode(Namespace(**given))
    variants, options = _known_keys()
    settings: dict[str, Any] = {"deterministic_mode": deterministic}
    for key, value in given.items():
        if value is None or not key.startswith("cake_"):
            continue
        if key in variants:
            settings[key] = _pick_variant(variants[key], value, deterministic, from_cli=False)
        elif key in options:
            _check_runtime(key, value)
            settings[key] = value
        else:
            raise ValueError(f"unknown cake option {key!r}")
    _Process.settings = MappingProxyType(settings)


def variant(op: str) -> str:
    """The variant ``op`` runs now: the configured one, else ``det`` (or the op's only variant).  In a process
    configured with deterministic mode, ``ValueError`` for an op that ships no ``det``."""
    settings = _Process.settings
    configured = settings.get(f"cake_{op}_variant")
    if configured is not None:
        return configured
    spec = registry.op_spec(op)
    if not settings.get("deterministic_mode"):
        return spec.default_variant
    if "det" in spec.variants:
        return "det"
    raise _no_det(spec)


def option(op: str | None, dest: str) -> Any:
    """The configured value of option ``dest`` of ``op`` (``None``: a runtime option), else its default."""
    owned = RUNTIME_FLAGS if op is None else registry.op_spec(op).flags
    defaults = {own.dest: own.default for own in owned}
    if dest not in defaults:
        raise KeyError(f"{'the runtime' if op is None else op} has no option {dest!r}")
    return _Process.settings.get(dest, defaults[dest])


def warn_runs_det(op: str, reason: str) -> None:
    """Log, once per ``(op, reason)``, that a call the ``fast`` variant does not serve runs ``det``."""
    seen = (op, reason)
    if seen in _Process.warned:
        return
    _Process.warned.add(seen)
    logger.warning("miles_ext_kernels.cake.%s: the fast variant does not serve %s; running det", op, reason)
