"""The implementation of ``cake.gated_rmsnorm`` (reference: miles_ext_kernels/cake/_impl/gated_rmsnorm/__init__.py)."""

from ..._runtime import loader

loader.install_op("gated_rmsnorm")

from .ops import check_supported, prebuild, release, rmsnorm_silu_gate  # noqa: E402

__all__ = ["check_supported", "prebuild", "release", "rmsnorm_silu_gate"]
