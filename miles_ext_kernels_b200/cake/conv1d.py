"""Packed causal depthwise conv1d + SiLU (kernel size 4), forward and backward: the short convolutions of the GDN and
KDA linear-attention layers, on hand-written sm_100a kernels.

The entry points and their argument meaning follow the reference's op (reference:
miles_ext_kernels/cake/conv1d.py:30-57, miles_ext_kernels/cake/_impl/conv1d/ops.py:144-257).  Both variants (``det``,
``fast``) run the same kernels here: the weight gradient is summed in a fixed order, so identical inputs give
identical bits.  miles selects the op with ``--linear-attention-conv-backend cake``.  The context-parallel entry points
(``causal_conv1d_kcp``, ``causal_conv1d_kcp_multi``) read the three rows across each cut of a contiguous partition
from the neighbouring rank: y and dx are the bits of the undivided call.

Importing this module imports neither torch nor the implementation.
"""

from argparse import Namespace

from ._runtime.spec import Flag, OpSpec, lazy_exports


def _validate(args: Namespace) -> None:
    """Nothing to reject: context parallelism goes through ``causal_conv1d_kcp``."""


OP = OpSpec(
    name="conv1d",
    summary="packed causal depthwise conv1d + SiLU, kernel size 4, forward + backward",
    variants=("det", "fast"),
    selected_by=(("linear_attention_conv_backend", "cake"),),
    packages=("libmek_b200",),
    exports=("causal_conv1d", "causal_conv1d_kcp", "causal_conv1d_kcp_multi", "check_supported"),
    flags=(
        Flag(
            "--cake-conv1d-silu-grad-preactivation",
            dict(
                choices=("bf16", "fp32"),
                default="bf16",
                help=(
                    "Where the short-conv backward evaluates the SiLU derivative: 'bf16' at the BF16-rounded "
                    "preactivation (flash-linear-attention's rounding point), 'fp32' at the unrounded FP32 "
                    "preactivation with an FP64 weight-gradient sum (a slower program). Default: 'bf16'. Only with "
                    "--linear-attention-conv-backend cake."
                ),
            ),
        ),
    ),
    validate=_validate,
)

__all__, __getattr__, __dir__ = lazy_exports(__name__, OP)
