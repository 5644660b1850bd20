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
from dataclasses import dataclass, field
from importlib import import_module
from types import MappingProxyType
from typing import Any

__all__ = ["VARIANTS", "Flag", "OpSpec", "lazy_exports"]

# "det": identical inputs give identical bits.  "fast": may trade that for speed.  Order matters: det first.
VARIANTS = ("det", "fast")

_FLAG_SHAPE = re.compile(r"--cake-[a-z0-9]+(-[a-z0-9]+)*")
_MODULE_NAME = re.compile(r"[a-z][a-z0-9_]*")


@dataclass(frozen=True)
class Flag:
    """One ``--cake-<op>-<what>`` command-line option: the flag and the keyword arguments of ``add_argument``.

    ``kwargs`` must carry ``default`` and ``help`` and must not carry ``dest``: the destination is the flag without
    its dashes (``--cake-gdn-recompute-state`` -> ``cake_gdn_recompute_state``).
    """

    name: str
    kwargs: Mapping[str, Any]
    dest: str = field(init=False, compare=False, default="")

    def __post_init__(self) -> None:
        if _FLAG_SHAPE.fullmatch(self.name) is None:
            raise ValueError(f"{self.name!r} is not a --cake-<op>-<what> flag")
        absent = [key for key in ("default", "help") if key not in self.kwargs]
        if absent:
            raise ValueError(f"{self.name}: add_argument keywords {sorted(absent)} are missing")
        if "dest" in self.kwargs:
            raise ValueError(f"{self.name}: the dest follows from the name")
        object.__setattr__(self, "kwargs", MappingProxyType(dict(self.kwargs)))
        object.__setattr__(self, "dest", self.name.lstrip("-").replace("-", "_"))

    @property
    def default(self) -> Any:
        return self.kwargs["default"]


def _ordered_subset(values: tuple[str, ...], of: tuple[str, ...]) -> bool:
    return bool(values) and values == tuple(v for v in of if v in values)


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
        if _MODULE_NAME.fullmatch(self.name) is None:
            raise ValueError(f"op name {self.name!r} is not a module name")
        if not _ordered_subset(self.variants, VARIANTS):
            raise ValueError(f"{self.name}: variants {self.variants} must be a non-empty subset of {VARIANTS}, in order")
        if self.cli_variants is not None and not _ordered_subset(self.cli_variants, self.variants):
            raise ValueError(f"{self.name}: cli_variants {self.cli_variants} must be a non-empty subset of variants")
        stem = f"--cake-{self.dashed}-"
        for flag in self.flags:
            if flag.name == self.variant_flag or not flag.name.startswith(stem):
                raise ValueError(f"{self.name}: option {flag.name} must start with {stem} and not be its variant")
        listings = {"flag": [f.dest for f in self.flags], "package": self.packages, "export": self.exports}
        for what, names in listings.items():
            if len(names) != len(set(names)):
                raise ValueError(f"{self.name}: a {what} is listed twice in {names}")
        if "OP" in self.exports:
            raise ValueError(f"{self.name}: OP is not an export")

    # -- names --------------------------------------------------------------------------------------------------
    @property
    def dashed(self) -> str:
        return self.name.replace("_", "-")

    @property
    def variant_flag(self) -> str:
        return f"--cake-{self.dashed}-variant"

    @property
    def variant_dest(self) -> str:
        return f"cake_{self.name}_variant"

    @property
    def selector(self) -> str:
        """The miles arguments that select this op, as typed on a command line."""
        return " or ".join(f"--{dest.replace('_', '-')} {value}" for dest, value in self.selected_by)

    # -- variants -----------------------------------------------------------------------------------------------
    @property
    def cli_choices(self) -> tuple[str, ...]:
        return self.cli_variants if self.cli_variants is not None else self.variants

    @property
    def default_variant(self) -> str:
        """What a process that never configured the op runs: ``det`` when the op has it, else its only variant."""
        return "det" if "det" in self.variants else self.variants[0]

    @property
    def has_variant_flag(self) -> bool:
        """Whether ``--cake-<op>-variant`` is registered (it carries the resolved variant to every process)."""
        return len(self.variants) > 1 and bool(self.selected_by)

    @property
    def shows_variant_flag(self) -> bool:
        """Whether the help lists the flag: only when miles has a real choice."""
        return self.has_variant_flag and len(self.cli_choices) > 1


def lazy_exports(module_name: str, op: OpSpec) -> tuple[list[str], Callable[[str], Any], Callable[[], list[str]]]:
    """``(__all__, __getattr__, __dir__)`` for the op module ``module_name``.

    ``__all__`` is ``["OP", *op.exports]``.  The first access of an export imports ``<source>._impl.<op>`` (the
    sibling of the op module's package), takes the attribute from it and caches it on the op module.
    """
    public = ["OP", *op.exports]
    lazy = frozenset(op.exports)
    source = module_name.rpartition(".")[0]
    implementation = f"{source}._impl.{op.name}"

    def __getattr__(name: str) -> Any:
        if name not in lazy:
            raise AttributeError(f"module {module_name!r} has no attribute {name!r}")
        found = getattr(import_module(implementation), name)
        setattr(sys.modules[module_name], name, found)
        return found

    def __dir__() -> list[str]:
        return sorted(set(vars(sys.modules[module_name])) | set(public))

    return public, __getattr__, __dir__
