"""The runtime the ops share (torch-free to import; reference: miles_ext_kernels/cake/_runtime/__init__.py):

- :mod:`.spec`: an op's declaration, ``OpSpec`` and ``Flag``.
- :mod:`.registry`: the registered ops, ``prebuild`` and ``release``.
- :mod:`.config`: the argument surface, the configuration of the process and the variant each op runs.
- :mod:`.loader`: nvcc build, file-locked cache and ctypes load of the native library.
- :mod:`.workspace`: the bounded scratch pool.

The export list is the public interface of radixark/miles-ext-kernels (Apache-2.0; see NOTICE): a drop-in has to
match it name for name.
"""

from .config import add_arguments, configure, deterministic_mode, option, validate_args, variant, warn_runs_det
from .loader import ARCH_BY_CAPABILITY, MIN_CUDA, cache_dir, device_arch
from .registry import OPS, op_spec, prebuild, release
from .spec import Flag, OpSpec

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
