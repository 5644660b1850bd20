"""The implementation of ``cake.kda`` (reference: miles_ext_kernels/cake/_impl/kda/__init__.py)."""

from ..._runtime import loader

loader.install_op("kda")

from .ops import (  # noqa: E402
    DEFAULT_SCALE,
    MAX_HEADS,
    chunk_kda,
    chunk_kda_bwd,
    chunk_kda_fwd,
    prebuild,
    release,
)

__all__ = ["DEFAULT_SCALE", "MAX_HEADS", "chunk_kda", "chunk_kda_bwd", "chunk_kda_fwd", "prebuild", "release"]
