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

_state: Mapping[str, Any] = MappingProxyType({})
_warned: set[tuple[str, str]] = set()


def _all_specs() -> list[OpSpec]:
    return [registry.op_spec(name) for name in registry.OPS]


def deterministic_mode(args: Any) -> bool:
    """Whether ``args`` asks for deterministic mode.

    miles' flat namespace carries Megatron's ``--deterministic-mode`` as ``args.deterministic_mode``; its typed
    configuration as ``args.backend.deterministic_mode``.  ``args.cake_deterministic`` (this package's alias) counts
    too.  Anything else is not deterministic mode.
    """
    flag = getattr(args, "deterministic_mode", None)
    if flag is None:
        flag = getattr(getattr(args, "backend", None), "deterministic_mode", False)
    return bool(flag) or bool(getattr(args, "cake_deterministic", False))


def add_arguments(parser: Any) -> None:
    """Register the ops' arguments and the runtime options on ``parser`` (a parser or an argument group)."""
    for spec in _all_specs():
        if not spec.selected_by:
            continue
        if spec.has_variant_flag:
            cli_default = "fast" if "fast" in spec.cli_choices else "det"
            text = (
                f"Variant of the cake {spec.name} kernels ({spec.summary}) under {spec.selector}: 'det' repeats bit "
                f"for bit for identical inputs, 'fast' is faster. Default: '{cli_default}', or 'det' under "
                "--deterministic-mode, which rejects 'fast'."
            )
            parser.add_argument(
                spec.variant_flag,
                choices=spec.cli_choices,
                default=None,
                help=text if spec.shows_variant_flag else argparse.SUPPRESS,
            )
        for flag in spec.flags:
            parser.add_argument(flag.name, **flag.kwargs)
    for flag in RUNTIME_FLAGS:
        parser.add_argument(flag.name, **flag.kwargs)


def _no_det(spec: OpSpec) -> ValueError:
    why = f": {spec.selector} is not deterministic" if spec.selector else ": it cannot run in deterministic mode"
    return ValueError(f"the cake {spec.name} kernels have no det variant{why}")


def _resolve(spec: OpSpec, requested: str | None, deterministic: bool, *, cli: bool) -> str | None:
    """The variant ``spec`` runs, ``None`` to leave it unset.  ``cli``: apply the command line's default."""
    if requested is None:
        if deterministic:
            if "det" not in spec.variants:
                raise _no_det(spec)
            return "det"
        if not cli:
            return None
        return "fast" if "fast" in spec.cli_choices else "det"
    allowed = spec.cli_choices if cli else spec.variants
    if requested not in allowed:
        raise ValueError(f"{spec.variant_flag} must be one of {allowed}, not {requested!r}")
    if deterministic and requested == "fast":
        raise ValueError(
            f"{spec.variant_flag} fast is not bit-reproducible under --deterministic-mode: use det or leave it unset"
        )
    return requested


def _check_runtime(dest: str, value: Any) -> None:
    if dest == "cake_workspace_pool_bytes" and value < 0:
        raise ValueError(f"--cake-workspace-pool-bytes must be >= 0, not {value}")


def validate_args(args: Namespace) -> None:
    """Check miles' parsed flat namespace; write the resolved variant of every selected op back to it."""
    deterministic = deterministic_mode(args)
    for spec in _all_specs():
        if not spec.selected_by:
            continue
        if any(getattr(args, dest, None) == value for dest, value in spec.selected_by):
            resolved = _resolve(spec, getattr(args, spec.variant_dest, None), deterministic, cli=True)
            if spec.has_variant_flag:
                setattr(args, spec.variant_dest, resolved)
            if spec.validate is not None:
                spec.validate(args)
            continue
        # the op is not selected: none of its options may be set
        owned = [(flag.name, flag.dest, flag.default) for flag in spec.flags]
        if spec.has_variant_flag:
            owned.insert(0, (spec.variant_flag, spec.variant_dest, None))
        for name, dest, default in owned:
            if getattr(args, dest, default) != default:
                raise ValueError(f"{name} requires {spec.selector}")
    for flag in RUNTIME_FLAGS:
        _check_runtime(flag.dest, getattr(args, flag.dest, flag.default))


def configure(args: Namespace | Mapping[str, Any] | None = None, /, **values: Any) -> None:
    """Replace this process's configuration with the ``cake_*`` entries of ``args`` and ``values``.

    ``args``: a namespace, a mapping (miles' ``miles_ext_kernels_args``) or ``None``; ``values`` win over it.  ``None``
    counts as unset and keys that do not start with ``cake_`` are skipped, so a whole namespace may be passed.
    ``ValueError`` for an unknown ``cake_*`` key, for a variant the op does not ship, and for ``fast`` when
    deterministic mode is on.  Each call starts again from the defaults.
    """
    merged: dict[str, Any] = {}
    if isinstance(args, Mapping):
        merged.update(args)
    elif args is not None:
        merged.update(vars(args))
    merged.update(values)
    deterministic = deterministic_mode(Namespace(**merged))

    accepted: dict[str, OpSpec | Flag] = {flag.dest: flag for flag in RUNTIME_FLAGS}
    for spec in _all_specs():
        accepted[spec.variant_dest] = spec
        for flag in spec.flags:
            accepted[flag.dest] = flag

    fresh: dict[str, Any] = {"deterministic_mode": deterministic}
    for key, value in merged.items():
        if value is None or not key.startswith("cake_"):
            continue
        owner = accepted.get(key)
        if owner is None:
            raise ValueError(f"unknown cake option {key!r}")
        if isinstance(owner, OpSpec):
            value = _resolve(owner, value, deterministic, cli=False)
        else:
            _check_runtime(key, value)
        fresh[key] = value
    global _state
    _state = MappingProxyType(fresh)


def variant(op: str) -> str:
    """The variant ``op`` runs now: the configured one, else ``det`` (or the op's only variant).  In a process
    configured with deterministic mode, ``ValueError`` for an op that ships no ``det``."""
    chosen = _state.get(f"cake_{op}_variant")
    if chosen is not None:
        return chosen
    spec = registry.op_spec(op)
    if _state.get("deterministic_mode"):
        if "det" not in spec.variants:
            raise _no_det(spec)
        return "det"
    return spec.default_variant


def option(op: str | None, dest: str) -> Any:
    """The configured value of option ``dest`` of ``op`` (``None``: a runtime option), else its default."""
    for flag in RUNTIME_FLAGS if op is None else registry.op_spec(op).flags:
        if flag.dest == dest:
            return _state.get(dest, flag.default)
    raise KeyError(f"{'the runtime' if op is None else op} has no option {dest!r}")


def warn_runs_det(op: str, reason: str) -> None:
    """Log, once per ``(op, reason)``, that a call the ``fast`` variant does not serve runs ``det``."""
    if (op, reason) not in _warned:
        _warned.add((op, reason))
        logger.warning("miles_ext_kernels.cake.%s: the fast variant does not serve %s; running det", op, reason)
