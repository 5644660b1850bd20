"""What the runtime knows of one op: :class:`OpSpec`, its option flags (:class:`Flag`) and the lazy export hook of an
op module.  Torch-free.

``cake/<op>.py`` declares ``OP = OpSpec(...)`` and wires :func:`lazy_exports`; the implementation package
``cake/_impl/<op>/`` is imported the first time one of the exports is touched, so importing the op module costs no
more than importing the runtime.  Same public names and rules as the reference's declaration layer (reference:
miles_ext_kernels/cake/_runtime/spec.py:26-168).
"""

from __future__ import annotations

import re
import sys
from argparse import Namespace
from collections.abc import Callable, Mapping
from dataclasses import dataclass
from importlib import import_module
from types import MappingProxyType
from typing import Any

__all__ = ["VARIANTS", "Flag", "OpSpec", "lazy_exports"]

# "det": identical inputs give identical bits.  "fast": may trade that for speed.  Order matters: det first.
VARIANTS = ("det", "fast")

_FLAG_SHAPE = re.compile(r"--cake-[a-z0-9]+(-[a-z0-9]+)*")
_MODULE_NAME = re.compile(r"[a-z][a-z0-9_]*")


class Flag:
    """One ``--cake-<op>-<what>`` command-line option: the flag and the keyword arguments of ``add_argument``.

    ``kwargs`` must carry ``default`` and ``help`` and must not carry ``dest``: the destination is the flag without
    its dashes (``--cake-gdn-recompute-state`` -> ``cake_gdn_recompute_state``).  Immutable; two flags are equal
    when their names and keywords are.
    """

    __slots__ = ("name", "kwargs", "dest")

    def __init__(self, name: str, kwargs: Mapping[str, Any]) -> None:
        if not _FLAG_SHAPE.fullmatch(name):
            raise ValueError(f"{name!r} is not a --cake-<op>-<what> flag")
        wanted = {"default", "help"} - set(kwargs)
        if wanted:
            raise ValueError(f"{name}: add_argument keywords {sorted(wanted)} are missing")
        if "dest" in kwargs:
            raise ValueError(f"{name}: the dest follows from the name")
        fix = object.__setattr__
        fix(self, "name", name)
        fix(self, "kwargs", MappingProxyType(dict(kwargs)))
        fix(self, "dest", name[2:].replace("-", "_"))

    def __setattr__(self, attribute: str, value: Any) -> None:
        raise AttributeError(f"Flag is immutable: cannot set {attribute}")

    def __eq__(self, other: object) -> bool:
        return isinstance(other, Flag) and (self.name, dict(self.kwargs)) == (other.name, dict(other.kwargs))

    def __hash__(self) -> int:
        return hash(self.name)

    def __repr__(self) -> str:
        return f"Flag({self.name!r}, {dict(self.kwargs)!r})"

    @property
    def default(self) -> Any:
        return self.kwargs["default"]


def _keeps_order(picked: tuple[str, ...], pool: tuple[str, ...]) -> bool:
    """Whether ``picked`` is a non-empty selection from ``pool`` that keeps ``pool``'s order (and repeats nothing)."""
    positions = [pool.index(item) if item in pool else -1 for item in picked]
    return bool(positions) and -1 not in positions and positions == sorted(set(positions))


def _first_repeat(names: Any) -> str | None:
    seen: set[str] = set()
    for name in names:
        if name in seen:
            return name
        seen.add(name)
    return None


@dataclass(frozen=True)
class OpSpec:
    """The declaration of one op.

    ``variants``: what ``configure`` accepts, a subset of :data:`VARIANTS` in its order.  ``cli_variants``: what
    miles may pick with ``--cake-<op>-variant`` (``None`` = all of ``variants``).  ``selected_by``: the ``(dest,
    value)`` pairs of miles arguments that route a call site to this op; the variant flag exists when there is such
    a selector and more than one variant, and is hidden from the help when miles may choose only one.  ``packages``:
    the native libraries (or kernel groups) the op launches.  ``exports``: the names ``cake.<op>`` re-exports from
    ``cake._impl.<op>``.  ``flags``: the op's options besides its variant.  ``validate``: a torch-free check of
    miles' namespace, run when the op is selected.
    """

    name: str
    summary: str
    variants: tuple[str, ...]
    cli_variants: tuple[str, ...] | None = None
    selected_by: tuple[tuple[str, str], ...] = ()
    packages: tuple[str, ...] = ()
    exports: tuple[str, ...] = ()
    flags: tuple[Flag, ...] = ()
    validate: Callable[[Namespace], None] | None = None

    def __post_init__(self) -> None:
        me = self.name
        if not _MODULE_NAME.fullmatch(me):
            raise ValueError(f"op name {me!r} is not a module name")
        if not _keeps_order(self.variants, VARIANTS):
            raise ValueError(f"{me}: variants {self.variants} must be a non-empty subset of {VARIANTS}, in order")
        if self.cli_variants is not None and not _keeps_order(self.cli_variants, self.variants):
            raise ValueError(f"{me}: cli_variants {self.cli_variants} must be a non-empty subset of variants")
        prefix = self.variant_flag[: -len("variant")]  # --cake-<op>-
        misplaced = [own.name for own in self.flags if own.name == self.variant_flag or not own.name.startswith(prefix)]
        if misplaced:
            raise ValueError(f"{me}: option {misplaced[0]} must start with {prefix} and not be its variant")
        for what, names in (("flag", [own.dest for own in self.flags]), ("package", self.packages),
                            ("export", self.exports)):
            if _first_repeat(names) is not None:
                raise ValueError(f"{me}: a {what} is listed twice in {names}")
        if "OP" in self.exports:
            raise ValueError(f"{me}: OP is not an export")

    # -- names --------------------------------------------------------------------------------------------------
    @property
    def dashed(self) -> str:
        return self.name.replace("_", "-")

    @property
    def variant_flag(self) -> str:
        return "--" + self.variant_dest.replace("_", "-")

    @property
    def variant_dest(self) -> str:
        return f"cake_{self.name}_variant"

    @property
    def selector(self) -> str:
        """The miles arguments that select this op, as typed on a command line."""
        typed = ["--" + dest.replace("_", "-") + " " + value for dest, value in self.selected_by]
        return " or ".join(typed)

    # -- variants -----------------------------------------------------------------------------------------------
    @property
    def cli_choices(self) -> tuple[str, ...]:
        return self.variants if self.cli_variants is None else self.cli_variants

    @property
    def default_variant(self) -> str:
        """What a process that never configured the op runs: ``det`` when the op has it, else its only variant."""
        return next((v for v in self.variants if v == "det"), self.variants[0])

    @property
    def has_variant_flag(self) -> bool:
        """Whether ``--cake-<op>-variant`` is registered (it carries the resolved variant to every process)."""
        return bool(self.selected_by) and len(self.variants) >= 2

    @property
    def shows_variant_flag(self) -> bool:
        """Whether the help lists the flag: only when miles has a real choice."""
        return self.has_variant_flag and len(self.cli_choices) >= 2


class _LazyModule:
    """The export hooks of one op module: the implementation package is imported at the first touch of an export,
    and every export found is cached on the op module so the hook runs once per name."""

    def __init__(self, module_name: str, op: OpSpec) -> None:
        self.module_name = module_name
        self.exports = frozenset(op.exports)
        self.public = ["OP", *op.exports]
        package = module_name.rpartition(".")[0]  # <pkg>.cake for <pkg>.cake.<op>
        self.implementation = f"{package}._impl.{op.name}"

    def getattr(self, name: str) -> Any:
        if name not in self.exports:
            raise AttributeError(f"module {self.module_name!r} has no attribute {name!r}")
        value = getattr(import_module(self.implementation), name)
        setattr(sys.modules[self.module_name], name, value)
        return value

    def dir(self) -> list[str]:
        return sorted({*vars(sys.modules[self.module_name]), *self.public})


def lazy_exports(module_name: str, op: OpSpec) -> tuple[list[str], Callable[[str], Any], Callable[[], list[str]]]:
    """``(__all__, __getattr__, __dir__)`` for the op module ``module_name``.

    ``__all__`` is ``["OP", *op.exports]``.  The first access of an export imports ``<source>._impl.<op>`` (the
    sibling of the op module's package), takes the attribute from it and caches it on the op module.
    """
    hooks = _LazyModule(module_name, op)
    return hooks.public, hooks.getattr, hooks.dir
