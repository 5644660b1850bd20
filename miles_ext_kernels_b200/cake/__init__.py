"""The ``cake`` source: one module per op (``.gdn``, ``.kda``; listed in ``OPS``), one runtime (``_runtime``) and the
op implementations (``_impl``).  The names below are the runtime's public API (reference:
miles_ext_kernels/cake/__init__.py:13-51).  Importing this package or an op module imports neither torch nor the
native library; an op's entry points import its implementation on first use.

The export list is the public interface of radixark/miles-ext-kernels (Apache-2.0; see NOTICE): a drop-in has to
match it name for name.
"""

from ._runtime import (
    ARCH_BY_CAPABILITY,
    MIN_CUDA,
    OPS,
    Flag,
    OpSpec,
    add_arguments,
    cache_dir,
    configure,
    deterministic_mode,
    device_arch,
    op_spec,
    option,
    prebuild,
    release,
    validate_args,
    variant,
    warn_runs_det,
)

__all__ = [
    "ARCH_BY_CAPABILITY",
    "MIN_CUDA",
    "OPS",
    "Flag",
    "OpSpec",
    "add_arguments",
    "cache_dir",
    "configure",
    "deterministic_mode",
    "device_arch",
    "op_spec",
    "option",
    "prebuild",
    "release",
    "validate_args",
    "variant",
    "warn_runs_det",
]
