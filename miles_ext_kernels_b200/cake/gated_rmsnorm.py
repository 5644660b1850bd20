"""SiLU-gated RMSNorm, forward and backward: ``RMSNorm(x) * weight * SiLU(z)`` over rows of 128, the output norm of
the GDN linear-attention layers, on hand-written sm_100a kernels.

The entry points and their argument meaning follow the reference's op (reference:
miles_ext_kernels/cake/gated_rmsnorm.py:17-24, miles_ext_kernels/cake/_impl/gated_rmsnorm/ops.py:80-148).  Both
variants (``det``, ``fast``) run the same kernels here: the weight gradient is summed in a fixed order (FP32 per block,
FP64 across the blocks), so identical inputs give identical bits.  miles selects the op with
``--linear-attention-output-norm-backend cake``.

Importing this module imports neither torch nor the implementation.
"""

from ._runtime.spec import OpSpec, lazy_exports

OP = OpSpec(
    name="gated_rmsnorm",
    summary="SiLU-gated RMSNorm, forward + backward, rows of 128, BF16",
    variants=("det", "fast"),
    selected_by=(("linear_attention_output_norm_backend", "cake"),),
    packages=("libmek_b200",),
    exports=("check_supported", "rmsnorm_silu_gate"),
)

__all__, __getattr__, __dir__ = lazy_exports(__name__, OP)
