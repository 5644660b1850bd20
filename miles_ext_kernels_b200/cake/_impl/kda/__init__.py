"""The implementation of ``cake.kda`` (reference: miles_ext_kernels/cake/_impl/kda/__init__.py)."""

from ..._runtime import loader

loader.install_op("kda")

from .kcp import (  # noqa: E402
    RecomputeHandle,
    build_context_kcp,
    chunk_kda_bwd_kcp,
    chunk_kda_fwd_kcp,
    chunk_kda_kcp,
    partition_kcp,
    reduce_gate_param_grads_kcp,
)
from .ops import (  # noqa: E402
    DEFAULT_SCALE,
    MAX_HEADS,
    chunk_kda,
    chunk_kda_bwd,
    chunk_kda_fwd,
    prebuild,
    release,
)

__all__ = [
    "DEFAULT_SCALE",
    "MAX_HEADS",
    "RecomputeHandle",
    "build_context_kcp",
    "chunk_kda",
    "chunk_kda_bwd",
    "chunk_kda_bwd_kcp",
    "chunk_kda_fwd",
    "chunk_kda_fwd_kcp",
    "chunk_kda_kcp",
    "partition_kcp",
    "prebuild",
    "reduce_gate_param_grads_kcp",
    "release",
]
