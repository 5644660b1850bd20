"""Packed causal depthwise conv1d + SiLU on the sm_100a kernels: ``causal_conv1d``, ``check_supported``, ``prebuild``,
``release`` (reference: miles_ext_kernels/cake/_impl/conv1d/ops.py:144-257).

``pre[t, c] = sum_{k<4} w[c, k] x[t - 3 + k, c]`` inside token ``t``'s document (FP32), ``y = bf16(silu(pre))``.  The
backward evaluates SiLU' at the BF16-rounded preactivation (``bf16`` policy, flash-linear-attention's rounding point)
or at the unrounded one with FP64 weight-gradient sums (``fp32`` policy); the weight gradient is summed in an order
fixed by the token count, in either variant.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any

import torch

from ..._runtime import config, loader, registry, workspace
from ..gdn import native

__all__ = ["causal_conv1d", "causal_conv1d_kcp", "causal_conv1d_kcp_multi", "check_supported", "prebuild", "release"]

OP = "conv1d"
KERNEL_SIZE = 4
CHANNEL_MULTIPLE = 8
SILU_GRAD_PREACTIVATIONS = ("bf16", "fp32")
TAP_DTYPES = (torch.float32, torch.bfloat16)
_BACKEND = "--linear-attention-conv-backend cake"


def check_supported(channels: int, kernel_size: int, activation: str, device=None, *, has_bias: bool = False) -> None:
    """Raise ``ValueError`` unless the kernels run this short convolution on ``device``: kernel size 4, SiLU, no
    bias, a channel count that is a multiple of 8, a B200 (reference: ops.py:144-160)."""
    if kernel_size != KERNEL_SIZE:
        raise ValueError(f"{_BACKEND} needs kernel size {KERNEL_SIZE}, got {kernel_size}")
    if activation != "silu":
        raise ValueError(f"{_BACKEND} applies SiLU, got activation {activation!r}")
    if has_bias:
        raise ValueError(f"{_BACKEND} convolves without a bias; use --linear-attention-conv-backend fla")
    if channels % CHANNEL_MULTIPLE:
        raise ValueError(f"{_BACKEND} needs a channel count that is a multiple of {CHANNEL_MULTIPLE}, got {channels}")
    if not torch.cuda.is_available():
        raise ValueError(f"{_BACKEND} needs a CUDA device of compute capability {tuple(loader.ARCH_BY_CAPABILITY)}")
    capability = tuple(torch.cuda.get_device_capability(device))
    arch = loader.ARCH_BY_CAPABILITY.get(capability)
    if arch is None:
        raise ValueError(f"{_BACKEND} runs on compute capability {tuple(loader.ARCH_BY_CAPABILITY)}, not {capability}")
    loader.check_toolkit(arch, "the short-convolution kernels")


def _policy(silu_grad_preactivation: str | None) -> str:
    policy = silu_grad_preactivation
    if policy is None:
        policy = config.option(OP, "cake_conv1d_silu_grad_preactivation") or "bf16"
    if policy not in SILU_GRAD_PREACTIVATIONS:
        raise ValueError(f"silu_grad_preactivation must be one of {SILU_GRAD_PREACTIVATIONS}, got {policy!r}")
    return policy


class _CausalConv1d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, cu_seqlens, policy):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        tokens, channels = x2.shape
        device = x.device
        y = torch.empty_like(x2)
        reach = None
        if tokens:
            reach = torch.empty(tokens, dtype=torch.uint8, device=device)
            with torch.cuda.device(device):
                native.launch("conv1d_reach", cu_seqlens, cu_seqlens.numel() - 1, tokens, reach, device=device)
                native.launch("conv1d_fwd", x2, weight, int(weight.dtype == torch.bfloat16), reach, y, tokens, channels,
                              device=device)
        ctx.save_for_backward(x2, weight, reach)
        ctx.policy, ctx.shape = policy, shape
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, reach = ctx.saved_tensors
        tokens, channels = x2.shape
        device = x2.device
        dx = torch.empty_like(x2)
        want_dw = ctx.needs_input_grad[1]
        dw = torch.zeros_like(weight) if want_dw else None
        if tokens:
            dy2 = dy.reshape(tokens, channels)
            dy2 = dy2.contiguous() if dy2.dtype == torch.bfloat16 else dy2.to(torch.bfloat16).contiguous()
            fp32_policy = ctx.policy == "fp32"
            with torch.cuda.device(device):
                partial = None
                if want_dw:
                    runs = native.library().mek_conv1d_runs(tokens)
                    partial = workspace.take(OP, "dw_partial", (runs, channels, KERNEL_SIZE),
                                             torch.float64 if fp32_policy else torch.float32, device)
                native.launch("conv1d_bwd", x2, weight, int(weight.dtype == torch.bfloat16), dy2, reach, dx, partial,
                              dw, int(fp32_policy), tokens, channels, device=device)
        return dx.view(ctx.shape), dw, None, None


def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, cu_seqlens: torch.Tensor | None = None, *,
                  silu_grad_preactivation: str | None = None) -> torch.Tensor:
    """Autograd-enabled ``silu(causal depthwise conv1d)`` of the packed documents of ``x``.

    ``x``: BF16 ``[1, S, C]`` or ``[S, C]`` (copied once when not contiguous); ``weight``: FP32 or BF16 ``[C, 4]``;
    ``cu_seqlens``: ``[num_docs + 1]`` prefix sums of the document lengths on ``x``'s device (``None``: one
    document, built on the device).  ``silu_grad_preactivation`` (``bf16`` / ``fp32``) defaults to the configured
    policy, read now.  Returns BF16 ``y`` of ``x``'s shape; the weight gradient comes in ``weight``'s dtype
    (reference: ops.py:226-257)."""
    if x.dim() == 3 and x.shape[0] != 1:
        raise ValueError(
            f"{_BACKEND} takes one packed batch [1, S, C] whose documents cu_seqlens delimits, got shape "
            f"{tuple(x.shape)}"
        )
    if x.dim() not in (2, 3) or not x.is_cuda or x.dtype != torch.bfloat16:
        raise ValueError(f"{_BACKEND} takes a BF16 CUDA tensor [1, S, C] or [S, C], got {x.dtype} {tuple(x.shape)}")
    channels = x.shape[-1]
    if channels % CHANNEL_MULTIPLE:
        raise ValueError(f"{_BACKEND} needs a channel count that is a multiple of {CHANNEL_MULTIPLE}, got {channels}")
    if tuple(weight.shape) != (channels, KERNEL_SIZE) or weight.dtype not in TAP_DTYPES:
        raise ValueError(f"{_BACKEND} takes FP32 or BF16 taps [{channels}, {KERNEL_SIZE}], got {weight.dtype} "
                         f"{tuple(weight.shape)}")
    config.variant(OP)
    policy = _policy(silu_grad_preactivation)
    x = x.contiguous()
    tokens = x.shape[-2]
    if cu_seqlens is None:
        cu_seqlens = torch.arange(2, dtype=torch.int32, device=x.device).mul_(tokens)  # no host copy, no sync
    else:
        cu_seqlens = cu_seqlens.to(torch.int32).contiguous()
    return _CausalConv1d.apply(x, weight.contiguous(), cu_seqlens, policy)


def causal_conv1d_kcp(x_local, weight, kcp_context, *, recompute_handle=None, cooperative=None):
    """The context-parallel route (the history tokens of a continuing fragment come from the rank that holds them) is
    not built."""
    raise NotImplementedError("causal_conv1d_kcp: the context-parallel short convolution is not built")


def causal_conv1d_kcp_multi(xs, weights, kcp_context, *, recompute_handle=None, cooperative=None):
    raise NotImplementedError("causal_conv1d_kcp_multi: the context-parallel short convolution is not built")


def prebuild(*, device: Any = None, max_workers: int | None = None, weight_dtype: torch.dtype = torch.float32) -> list[Path]:
    """Build (or find) the native library for ``device``; ``weight_dtype`` is checked (FP32 or BF16 taps)."""
    if weight_dtype not in TAP_DTYPES:
        raise ValueError(f"{_BACKEND} takes FP32 or BF16 taps, got {weight_dtype}")
    arch = loader.device_arch(device)
    loader.check_toolkit(arch, "the short-convolution kernels")
    return loader.prebuild_libraries(registry.op_spec(OP).packages, arch, max_workers=max_workers)


def release() -> None:
    """Nothing is kept between calls besides the workspace pool (emptied by the runtime) and the library handle."""
