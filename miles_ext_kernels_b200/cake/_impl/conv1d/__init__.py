"""The implementation of ``cake.conv1d`` (reference: miles_ext_kernels/cake/_impl/conv1d/__init__.py)."""

from ..._runtime import loader

loader.install_op("conv1d")

from .ops import (  # noqa: E402
    causal_conv1d,
    causal_conv1d_kcp,
    causal_conv1d_kcp_multi,
    check_supported,
    prebuild,
    release,
)

__all__ = ["causal_conv1d", "causal_conv1d_kcp", "causal_conv1d_kcp_multi", "check_supported", "prebuild", "release"]
