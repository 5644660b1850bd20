"""SiLU-gated RMSNorm on the sm_100a kernels: ``rmsnorm_silu_gate``, ``check_supported``, ``prebuild``, ``release``
(reference: miles_ext_kernels/cake/_impl/gated_rmsnorm/ops.py:80-148).

Per row of 128 of BF16 ``x`` and of the gate ``z`` (``[T, H, 128]`` or ``[T * H, 128]``, each with its own token and
head strides) and a BF16 ``weight [128]`` shared by every token and head::

    rstd = 1 / sqrt(mean(x^2) + eps)                     # FP32
    y    = bf16(((x * rstd) * weight) * silu(z))         # FP32, one rounding

The autograd node saves only ``x``, ``z`` and ``weight``; the backward recomputes ``rstd``.  The weight gradient is
summed in FP32 per block and in FP64 across the blocks, in an order fixed by the row count: the same bits on every
call, in either variant.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any

import torch

from ..._runtime import config, loader, registry, workspace
from ..gdn import native

__all__ = ["check_supported", "prebuild", "release", "rmsnorm_silu_gate"]

OP = "gated_rmsnorm"
HEAD_DIM = 128
_BACKEND = "--linear-attention-output-norm-backend cake"


def check_supported(head_dim: int, activation: str, weight_dtype: torch.dtype, *, has_bias: bool = False,
                    device=None) -> None:
    """Raise ``ValueError`` unless the kernels run this gated output norm on ``device`` (default: the current CUDA
    device): a SiLU gate, rows of 128, a BF16 weight without bias, a B200 (reference: ops.py:80-98)."""
    if activation != "silu":
        raise ValueError(
            f"{_BACKEND} computes RMSNorm(x) * w * SiLU(z), but this model gates its output norm with "
            f"{activation!r}; use --linear-attention-output-norm-backend fla"
        )
    if head_dim != HEAD_DIM:
        raise ValueError(f"{_BACKEND} normalizes rows of {HEAD_DIM}, got a value head dimension of {head_dim}")
    if has_bias:
        raise ValueError(f"{_BACKEND} has no bias")
    if weight_dtype != torch.bfloat16:
        raise ValueError(f"{_BACKEND} takes a BF16 weight, got {weight_dtype}")
    if not torch.cuda.is_available():
        raise ValueError(f"{_BACKEND} needs a CUDA device of compute capability {tuple(loader.ARCH_BY_CAPABILITY)}")
    capability = tuple(torch.cuda.get_device_capability(device))
    arch = loader.ARCH_BY_CAPABILITY.get(capability)
    if arch is None:
        raise ValueError(
            f"{_BACKEND} runs on compute capability {tuple(loader.ARCH_BY_CAPABILITY)}, not {capability}; use "
            "--linear-attention-output-norm-backend fla"
        )
    loader.check_toolkit(arch, "the gated RMSNorm kernels")


def _rows_view(t: torch.Tensor, name: str) -> tuple[torch.Tensor, int, int, int]:
    """``(tensor the kernels read, heads, token stride, head stride)`` of ``t [..., 128]``: read in place when its last
    stride is 1, its token and head strides are multiples of 8 elements and it is 16-byte aligned, else copied once."""
    if t.dim() < 2 or t.shape[-1] != HEAD_DIM:
        raise ValueError(f"rmsnorm_silu_gate: {name} must be [..., {HEAD_DIM}]; got {tuple(t.shape)}")
    if t.dim() > 3:
        t = t.reshape(-1, t.shape[-2], HEAD_DIM)  # a view when the leading dimensions merge
    if t.dim() == 2:
        heads, token_stride, head_stride = 1, t.stride(0), 0
    else:
        heads, token_stride, head_stride = t.shape[1], t.stride(0), t.stride(1)
    in_place = (
        t.stride(-1) == 1 and token_stride % 8 == 0 and head_stride % 8 == 0 and t.data_ptr() % 16 == 0
        and token_stride >= 0 and head_stride >= 0
    )
    if not in_place:
        t = t.contiguous()
        token_stride, head_stride = (t.stride(0), 0) if t.dim() == 2 else (t.stride(0), t.stride(1))
    return t, heads, token_stride, head_stride


class _RmsnormSiluGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, z, weight, eps):
        if not (x.is_cuda and z.is_cuda and weight.is_cuda):
            raise ValueError("rmsnorm_silu_gate: x, z and weight must be CUDA tensors")
        if x.shape != z.shape:
            raise ValueError(f"rmsnorm_silu_gate: z must have x's shape {tuple(x.shape)}; got {tuple(z.shape)}")
        if not (x.dtype == z.dtype == weight.dtype == torch.bfloat16):
            raise NotImplementedError("rmsnorm_silu_gate: x, z and weight must be bfloat16")
        if tuple(weight.shape) != (HEAD_DIM,):
            raise ValueError(f"rmsnorm_silu_gate: weight must be [{HEAD_DIM}]; got {tuple(weight.shape)}")
        y = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
        rows = x.numel() // HEAD_DIM
        if rows:
            xv, heads, xt, xh = _rows_view(x, "x")
            zv, z_heads, zt, zh = _rows_view(z, "z")
            if z_heads != heads:
                raise ValueError("rmsnorm_silu_gate: x and z must split their rows into the same heads")
            with torch.cuda.device(x.device):
                native.launch("gated_rmsnorm_fwd", xv, zv, weight.contiguous(), y, rows, heads, xt, xh, zt, zh,
                              float(eps), device=x.device)
        ctx.save_for_backward(x, z, weight)
        ctx.eps = float(eps)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, z, weight = ctx.saved_tensors
        device = x.device
        rows = x.numel() // HEAD_DIM
        dx = torch.empty(x.shape, dtype=torch.bfloat16, device=device)
        dz = torch.empty(x.shape, dtype=torch.bfloat16, device=device)
        want_dw = ctx.needs_input_grad[2]
        dw = torch.zeros(HEAD_DIM, dtype=torch.bfloat16, device=device) if want_dw else None
        if rows:
            xv, heads, xt, xh = _rows_view(x, "x")
            zv, _, zt, zh = _rows_view(z, "z")
            dy = dy.contiguous() if dy.dtype == torch.bfloat16 else dy.to(torch.bfloat16).contiguous()
            with torch.cuda.device(device):
                partial = None
                if want_dw:
                    blocks = native.library().mek_gated_rmsnorm_partial_rows(native.ctypes.c_int64(rows))
                    partial = workspace.take(OP, "dw_partial", (blocks, HEAD_DIM), torch.float32, device)
                native.launch("gated_rmsnorm_bwd", dy, xv, zv, weight.contiguous(), dx, dz, partial, dw, rows, heads,
                              xt, xh, zt, zh, ctx.eps, device=device)
        return dx, dz, dw, None


def rmsnorm_silu_gate(x: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Autograd-enabled ``RMSNorm(x) * weight * SiLU(z)`` over the last dimension (128).

    ``x`` and ``z``: BF16 of one ``[..., 128]`` shape; a gate that is a column slice of a wider projection is read in
    place when its last stride is 1, its token and head strides are multiples of 8 elements and it is 16-byte aligned,
    else copied once (the same bits either way).  ``weight``: BF16 ``[128]``.  Returns BF16 ``y`` of ``x``'s shape;
    every gradient comes in BF16 and the weight gradient sums over the rows of this call only (reference:
    ops.py:126-148)."""
    config.variant(OP)  # both variants run the same kernels; an unknown configuration still raises here
    return _RmsnormSiluGate.apply(x, z, weight, eps)


def prebuild(*, device: Any = None, max_workers: int | None = None) -> list[Path]:
    """Build (or find) the native library for ``device``."""
    arch = loader.device_arch(device)
    loader.check_toolkit(arch, "the gated RMSNorm kernels")
    return loader.prebuild_libraries(registry.op_spec(OP).packages, arch, max_workers=max_workers)


def release() -> None:
    """Nothing is kept between calls besides the workspace pool (emptied by the runtime) and the library handle."""
