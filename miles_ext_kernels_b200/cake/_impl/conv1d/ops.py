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


class _Span:
    """Tokens ``[lo, hi)`` of the call that one launch serves: ``cu`` (int32, on the device) are the boundaries of its
    documents relative to ``lo``, the first moved back by the history rows that belong to the first document and the
    last moved on by the continuation rows that belong to the last; ``prev`` / ``next``: per tensor the ``[3, C]``
    rows before / after the span (``None``: nothing crosses that cut)."""

    __slots__ = ("lo", "hi", "cu", "prev", "next")

    def __init__(self, lo, hi, cu, prev, next):
        self.lo, self.hi, self.cu, self.prev, self.next = lo, hi, cu, prev, next


class _Halo:
    """The spans of a call and ``swap_back``, which sends the first rows of the spans' output gradients
    (``[spans, 3, sum of C]``) to the ranks before and returns, per span, the rows after it (``None``: a call on its
    own)."""

    __slots__ = ("spans", "swap_back")

    def __init__(self, spans, swap_back=None):
        self.spans, self.swap_back = spans, swap_back


def _stacked(rows: list[torch.Tensor], like: torch.Tensor, width: int) -> torch.Tensor:
    """``[spans, 3, width]``; a rank without tokens still takes part in the exchange, with no spans."""
    if rows:
        return torch.stack(rows)
    return like.new_zeros((0, KERNEL_SIZE - 1, width))


def _split_rows(rows: torch.Tensor | None, widths: list[int]) -> list[torch.Tensor | None]:
    if rows is None:
        return [None] * len(widths)
    return [part.contiguous() for part in rows.split(widths, dim=1)]


class _CausalConv1d(torch.autograd.Function):
    """``n`` convolutions over one token layout: ``apply(halo, policy, n, *xs, *weights) -> ys``."""

    @staticmethod
    def forward(ctx, halo, policy, n, *tensors):
        xs, weights = tensors[:n], tensors[n:]
        device = xs[0].device
        ys = tuple(torch.empty_like(x) for x in xs)
        reaches = []
        with torch.cuda.device(device):
            for span in halo.spans:
                tokens = span.hi - span.lo
                if tokens <= 0:
                    reaches.append(None)
                    continue
                entries = tokens + (KERNEL_SIZE - 1 if any(r is not None for r in span.next) else 0)
                reach = torch.empty(entries, dtype=torch.uint8, device=device)
                native.launch("conv1d_reach", span.cu, span.cu.numel() - 1, entries, reach, device=device)
                for x, w, y, prev in zip(xs, weights, ys, span.prev):
                    native.launch("conv1d_fwd", x[span.lo : span.hi], prev, w, int(w.dtype == torch.bfloat16), reach,
                                  y[span.lo : span.hi], tokens, x.shape[1], device=device)
                reaches.append(reach)
        ctx.save_for_backward(*xs, *weights, *[r for r in reaches if r is not None])
        ctx.halo, ctx.policy, ctx.n = halo, policy, n
        ctx.have_reach = [r is not None for r in reaches]
        return ys

    @staticmethod
    def backward(ctx, *dys):
        n, halo = ctx.n, ctx.halo
        saved = ctx.saved_tensors
        xs, weights, kept = saved[:n], saved[n : 2 * n], list(saved[2 * n :])
        reaches = [kept.pop(0) if have else None for have in ctx.have_reach]
        device = xs[0].device
        dys = [torch.zeros_like(x) if dy is None else dy.reshape(x.shape).to(torch.bfloat16).contiguous()
               for x, dy in zip(xs, dys)]
        reachable = KERNEL_SIZE - 1
        widths = [x.shape[1] for x in xs]
        after = [None] * len(halo.spans)
        if halo.swap_back is not None:
            firsts = _stacked([torch.cat([dy[span.lo : span.lo + reachable] for dy in dys], dim=1)
                               for span in halo.spans], dys[0], sum(widths))
            after = halo.swap_back(firsts)
        fp32_policy = ctx.policy == "fp32"
        dxs = [torch.empty_like(x) for x in xs]
        dws = [torch.zeros_like(w) if ctx.needs_input_grad[3 + n + i] else None for i, w in enumerate(weights)]
        with torch.cuda.device(device):
            for span, reach, rows_after in zip(halo.spans, reaches, after):
                tokens = span.hi - span.lo
                if tokens <= 0:
                    continue
                dy_next = _split_rows(rows_after, widths)
                for i, (x, w, dy, dx, dw) in enumerate(zip(xs, weights, dys, dxs, dws)):
                    channels = x.shape[1]
                    partial = span_dw = None
                    if dw is not None:
                        runs = native.library().mek_conv1d_runs(tokens)
                        partial = workspace.take(OP, "dw_partial", (runs, channels, KERNEL_SIZE),
                                                 torch.float64 if fp32_policy else torch.float32, device)
                        span_dw = dw if len(halo.spans) == 1 else torch.empty_like(dw)
                    x_next = span.next[i] if dy_next[i] is not None else None
                    native.launch("conv1d_bwd", x[span.lo : span.hi], span.prev[i], x_next, w,
                                  int(w.dtype == torch.bfloat16), dy[span.lo : span.hi],
                                  dy_next[i] if x_next is not None else None, reach, dx[span.lo : span.hi], partial,
                                  span_dw, int(fp32_policy), tokens, channels, device=device)
                    if dw is not None and span_dw is not dw:
                        dw += span_dw  # the spans in order: a fixed sum
        return (None, None, None, *dxs, *dws)


def _checked(x: torch.Tensor, weight: torch.Tensor) -> None:
    if x.dim() not in (2, 3) or not x.is_cuda or x.dtype != torch.bfloat16:
        raise ValueError(f"{_BACKEND} takes a BF16 CUDA tensor [1, S, C] or [S, C], got {x.dtype} {tuple(x.shape)}")
    channels = x.shape[-1]
    if channels % CHANNEL_MULTIPLE:
        raise ValueError(f"{_BACKEND} needs a channel count that is a multiple of {CHANNEL_MULTIPLE}, got {channels}")
    if tuple(weight.shape) != (channels, KERNEL_SIZE) or weight.dtype not in TAP_DTYPES:
        raise ValueError(f"{_BACKEND} takes FP32 or BF16 taps [{channels}, {KERNEL_SIZE}], got {weight.dtype} "
                         f"{tuple(weight.shape)}")


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
    _checked(x, weight)
    config.variant(OP)
    policy = _policy(silu_grad_preactivation)
    x = x.contiguous()
    tokens = x.shape[-2]
    if cu_seqlens is None:
        cu_seqlens = torch.arange(2, dtype=torch.int32, device=x.device).mul_(tokens)  # no host copy, no sync
    else:
        cu_seqlens = cu_seqlens.to(torch.int32).contiguous()
    halo = _Halo([_Span(0, tokens, cu_seqlens, [None], [None])])
    (y,) = _CausalConv1d.apply(halo, policy, 1, x.view(tokens, x.shape[-1]), weight.contiguous())
    return y.view(x.shape)


def _kcp_taps(weight: torch.Tensor) -> torch.Tensor:
    """FP32 taps for the context-parallel route: BF16 taps widened (exact; autograd rounds their gradient back)
    (reference: ops.py:260-264)."""
    return (weight.float() if weight.dtype == torch.bfloat16 else weight).contiguous()


def _span_boundaries(kcp_context: Any, device: torch.device) -> list[torch.Tensor]:
    """Per span of the rank's plan: the boundaries of its fragments relative to the span's first token, the first
    moved back by the history rows of the first document and the last moved on by the continuation rows of the last;
    built once per context (one host-to-device copy)."""
    from ..gdn.meta import upload

    cached = getattr(kcp_context, "_conv1d_cu", None)
    guard = getattr(kcp_context, "_conv1d_cu_guard", None)
    if cached is not None and cached[0].device == device and guard is not None:
        guard.wait()  # a call on another stream than the one that uploaded the table
    if cached is None or cached[0].device != device:
        cu = kcp_context.cu_seqlens_cpu
        flat, extents = [], []
        for span in kcp_context.plan.spans:
            local = [cu[i] - span.token_lo for i in range(span.first, span.last + 2)]
            local[0] -= span.before
            local[-1] += span.after
            extents.append((len(flat), len(flat) + len(local)))
            flat += local
        table, guard = upload(torch.tensor(flat or [0], dtype=torch.int32), device)
        cached = [table[a:b] for a, b in extents] or [table]
        try:
            kcp_context._conv1d_cu = cached
            kcp_context._conv1d_cu_guard = guard
        except AttributeError:
            pass
    return cached


def causal_conv1d_kcp_multi(xs, weights, kcp_context: Any, *, recompute_handle: Any = None,
                            cooperative: bool | None = None) -> tuple[torch.Tensor, ...]:
    """The context-parallel convolutions of several tensors of one layer (for example its q, k and v) with one
    neighbour exchange per direction instead of one per tensor.

    ``xs``: ``n >= 1`` BF16 ``[T_r, C_i]`` (or ``[1, T_r, C_i]``) tensors, the rank's fragments back to back;
    ``weights``: their ``[C_i, 4]`` taps, the same on every rank; ``kcp_context``: the rank's context of the layer's
    GDN / KDA context-parallel route (read: ``num_tokens``, ``cu_seqlens_cpu``, ``plan.spans``, ``world_size`` and
    ``halo_exchange()``), under any of its layouts.  Every rank of the context's group makes this call for the same layers in the same order.

    The forward sends the first three rows of every span of consecutive local fragments to the rank that holds the
    tokens before it and the last three to the rank that holds the tokens after it, where a document crosses the cut
    (point to point under the contiguous layout, one small all-gather under the others); the backward sends the
    first three rows of the output gradients the same way.  A span is one launch per tensor.  y
    and dx are the bits of the undivided call; the weight gradient is the rank's partial sum over its own tokens (in
    ``weight``'s dtype; BF16 taps are widened first and autograd rounds their gradient back).  ``recompute_handle``:
    ``None`` or an object with an ``entries`` dict; the first forward stores the rows it received under ``"conv"``
    and a recompute of the call reuses them without an exchange.  ``cooperative`` (the reference's launch form of its
    backward program) is accepted and has no effect: the backward here is one ordinary launch per tensor.
    (reference: ops.py:267-340)."""
    if isinstance(xs, torch.Tensor) or isinstance(weights, torch.Tensor):
        raise TypeError("xs and weights must be sequences of tensors (one per convolution), not a tensor")
    xs, weights = list(xs), list(weights)
    if not xs or len(xs) != len(weights):
        raise ValueError(f"causal_conv1d_kcp_multi takes as many taps as tensors, got {len(xs)} and {len(weights)}")
    if cooperative not in (None, True, False):
        raise ValueError(f"cooperative must be None, True or False, got {cooperative!r}")
    for x, w in zip(xs, weights):
        _checked(x, w)
        if x.dim() == 3 and x.shape[0] != 1:
            raise ValueError(f"{_BACKEND} takes the rank's fragments as [T_r, C] or [1, T_r, C], got {tuple(x.shape)}")
    config.variant(OP)
    policy = _policy(None)
    tokens = int(kcp_context.num_tokens)
    shapes = [x.shape for x in xs]
    xs = [x.contiguous().view(-1, x.shape[-1]) for x in xs]
    if any(x.shape[0] != tokens for x in xs):
        raise ValueError(f"causal_conv1d_kcp: the context holds {tokens} tokens on this rank, the tensors "
                         f"{[x.shape[0] for x in xs]}")
    reachable = KERNEL_SIZE - 1
    world = int(kcp_context.world_size)
    if world > 1 and any(sp.token_hi - sp.token_lo < reachable for sp in kcp_context.plan.spans):
        raise NotImplementedError(f"causal_conv1d_kcp: every run of local fragments needs at least {reachable} tokens")
    weights = [_kcp_taps(w) for w in weights]
    widths = [x.shape[1] for x in xs]
    wait_ready = getattr(kcp_context, "wait_ready", None)
    if wait_ready is not None:
        wait_ready()
    plan_spans = kcp_context.plan.spans
    prev_rows, next_rows = [None] * len(plan_spans), [None] * len(plan_spans)
    exchange = kcp_context.halo_exchange() if world > 1 else None
    if exchange is not None:
        entries = getattr(recompute_handle, "entries", None)
        if entries is not None and "conv" in entries:
            prev_rows, next_rows = entries["conv"]
        else:
            with torch.no_grad():
                first = _stacked([torch.cat([x[sp.token_lo : sp.token_lo + reachable] for x in xs], dim=1)
                                  for sp in plan_spans], xs[0], sum(widths))
                last = _stacked([torch.cat([x[sp.token_hi - reachable : sp.token_hi] for x in xs], dim=1)
                                 for sp in plan_spans], xs[0], sum(widths))
                prev_rows, next_rows = exchange.forward(first, last)
            if entries is not None:
                entries["conv"] = (prev_rows, next_rows)
    boundaries = _span_boundaries(kcp_context, xs[0].device)
    spans = [_Span(sp.token_lo, sp.token_hi, cu, _split_rows(before, widths), _split_rows(after, widths))
             for sp, cu, before, after in zip(plan_spans, boundaries, prev_rows, next_rows)]
    halo = _Halo(spans, exchange.backward if exchange is not None else None)
    ys = _CausalConv1d.apply(halo, policy, len(xs), *xs, *weights)
    return tuple(y.view(shape) for y, shape in zip(ys, shapes))


def causal_conv1d_kcp(x_local: torch.Tensor, weight: torch.Tensor, kcp_context: Any, *, recompute_handle: Any = None,
                      cooperative: bool | None = None) -> torch.Tensor:
    """Autograd-enabled ``silu(causal depthwise conv1d)`` of this rank's fragments under context parallelism: one
    tensor of :func:`causal_conv1d_kcp_multi` (reference: ops.py:267-309)."""
    if not isinstance(x_local, torch.Tensor) or not isinstance(weight, torch.Tensor):
        raise TypeError("causal_conv1d_kcp takes one tensor and its taps; use causal_conv1d_kcp_multi for several")
    return causal_conv1d_kcp_multi([x_local], [weight], kcp_context, recompute_handle=recompute_handle,
                                   cooperative=cooperative)[0]


def prebuild(*, device: Any = None, max_workers: int | None = None, weight_dtype: torch.dtype = torch.float32) -> list[Path]:
    """Build (or find) the native library for ``device``; ``weight_dtype`` is checked (FP32 or BF16 taps)."""
    if weight_dtype not in TAP_DTYPES:
        raise ValueError(f"{_BACKEND} takes FP32 or BF16 taps, got {weight_dtype}")
    arch = loader.device_arch(device)
    loader.check_toolkit(arch, "the short-convolution kernels")
    return loader.prebuild_libraries(registry.op_spec(OP).packages, arch, max_workers=max_workers)


def release() -> None:
    """Nothing is kept between calls besides the workspace pool (emptied by the runtime) and the library handle."""
