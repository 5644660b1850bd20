"""The implementation of ``cake.gdn``: entry points, context-parallel contexts, ``prebuild`` and ``release``
(reference: miles_ext_kernels/cake/_impl/gdn/__init__.py)."""

from ..._runtime import loader

loader.install_op("gdn")

from .kcp import KcpContext, build_kcp_context  # noqa: E402
from .ops import (  # noqa: E402
    chunk_gated_delta_rule,
    kcp_chunk_gated_delta_rule,
    packed_qkv_views,
    prebuild,
    release,
)

__all__ = [
    "KcpContext",
    "build_kcp_context",
    "chunk_gated_delta_rule",
    "kcp_chunk_gated_delta_rule",
    "packed_qkv_views",
    "prebuild",
    "release",
]
