"""Packed KDA (Kimi Delta Attention: the gated delta rule with a per-key-channel decay), chunk 64, K = V = 128,
1 to 64 heads per call, per-document zero initial state, forward and backward, on hand-written sm_100a kernels.

The entry points and their argument meaning follow the reference's op (reference: miles_ext_kernels/cake/kda.py:53-78,
miles_ext_kernels/cake/_impl/kda/ops.py:142-234; the context-parallel entry points ``*_kcp``:
miles_ext_kernels/cake/_impl/kda/kcp.py:86-230).  miles selects the op with ``--kda-backend cake``, builds the library
when a layer is built (``cake.prebuild("kda", num_heads=...)``) and calls :func:`chunk_kda` in its forward.

Importing this module imports neither torch nor the implementation.
"""

from argparse import Namespace

from ._runtime.spec import OpSpec, lazy_exports


def _validate(args: Namespace) -> None:
    """Under ``--kda-backend cake`` miles' command line may not ask for context parallelism, and the layout must be
    the packed ``thd`` one.

    The op itself does run context-parallel: ``chunk_kda_kcp`` and its twins take this rank's slice of a partition of
    the packed batch that ``build_context_kcp`` describes.  What is rejected here is miles' own context-parallel KDA
    path, which hands every rank a shard of every document under flash-linear-attention's context instead of such a
    partition -- the same rule, in the same words, as the reference's op (reference:
    miles_ext_kernels/cake/kda.py:35-50).  ``bshd`` is not a packed sequence."""
    ranks = getattr(args, "context_parallel_size", None) or 1
    if ranks > 1:
        raise ValueError(
            f"--kda-backend cake does not support context parallelism yet (--context-parallel-size {ranks}); use "
            "--kda-backend fla"
        )
    layout = getattr(args, "qkv_format", "thd")
    if layout != "thd":
        raise ValueError(f"--kda-backend cake needs --qkv-format thd (one packed sequence), got {layout!r}")


OP = OpSpec(
    name="kda",
    summary="packed KDA chunked training, forward + backward, K = V = 128, 1 to 64 heads, context parallelism",
    variants=("det", "fast"),
    cli_variants=("det",),
    selected_by=(("kda_backend", "cake"),),
    packages=("libmek_b200",),
    exports=(
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
        "reduce_gate_param_grads_kcp",
    ),
    validate=_validate,
)

__all__, __getattr__, __dir__ = lazy_exports(__name__, OP)
