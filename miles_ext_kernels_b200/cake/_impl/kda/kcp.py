"""Context-parallel packed KDA: one packed batch split over the ranks of a process group (contiguous slices, the
zigzag layouts or an explicit fragment table), with the per-document state crossing the cuts.

Entry points and argument meaning follow the reference (reference: miles_ext_kernels/cake/_impl/kda/kcp.py:86-230)::

    part = partition_kcp(cu_seqlens_global_cpu, world_size)   # the same object on every rank
    ctx = build_context_kcp(part, group, rank, device)         # this rank's tables and boundary flags
    out_local = chunk_kda_kcp(q_local, k_local, v_local, g_local, beta_local, ctx)   # autograd

A rank's operands are its shard (the tokens of its slice), with the shapes, dtypes and modes of the single-rank
:func:`chunk_kda`.  Forward: the ``[H, 128, 128]`` fp32 state at the end of a fragment goes to the rank that holds the
document's next tokens; backward: the adjoint state at the start of a fragment goes to the rank that holds the tokens
before.  Two exchanges, chosen like the GDN op's (``--cake-gdn-kcp-exchange``): the sequential hand-over along the
rank chain of the contiguous layout (point to point; bit for bit the single-rank recurrence when the cuts fall on
multiples of 64 tokens inside their documents, within the accuracy budgets otherwise), and the parallel exchange of
affine fragment summaries (pre-scan of a fragment's segments, one all-gather, a fold per fragment; every layout;
within the accuracy budgets).

Options of the ``*_kcp`` entry points (the reference passes them on to its packages; reference:
miles_ext_kernels/cake/_impl/kda/kcp.py:144-146): ``save_mode`` (``"full"`` keeps the forward's tapes for the backward,
``"light"`` keeps the operands and the states that entered this rank's fragments and replays the local kernels in the
backward, without a second exchange), ``recompute_handle`` (a :class:`RecomputeHandle`: under activation
checkpointing the region's replayed forward binds the states the original forward received instead of exchanging
again), ``checkpoint_keep`` (``"states"``: what a handle keeps) and ``exchange`` (``"auto"``, ``"sequential"``,
``"parallel"``: this call's boundary-state exchange instead of the configured one).  The packages' other options
(``boundary_mode``, ``workspace``, ``save_transfer``, ``graph``) have no counterpart here and are refused.

In the raw gate mode the gradients of ``A_log`` / ``dt_bias`` are this rank's partial sums;
:func:`reduce_gate_param_grads_kcp` sums them over the group in rank order, the same bits on every rank.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from ..._runtime import config
from ..gdn import tape as tape_module
from ..gdn.kcp import KcpContext
from . import ops

__all__ = [
    "KcpPartition",
    "RecomputeHandle",
    "build_context_kcp",
    "chunk_kda_bwd_kcp",
    "chunk_kda_fwd_kcp",
    "chunk_kda_kcp",
    "partition_kcp",
    "reduce_gate_param_grads_kcp",
]


@dataclass(frozen=True)
class KcpPartition:
    """The partition of one packed batch: the global document offsets, the number of ranks and the layout."""

    cu_seqlens_global: tuple[int, ...]
    world_size: int
    layout: str = "contiguous"
    fragments: tuple | None = None  # an explicit table per rank, instead of a layout


def partition_kcp(cu_seqlens_global_cpu: Any, world_size: int, layout: str = "contiguous", fragments: Any = None, *,
                  cut_points: Any = None) -> KcpPartition:
    """The context-parallel partition of one packed batch over ``world_size`` ranks: ``layout`` ``contiguous`` (equal
    token shares in order), ``zigzag``, ``zigzag_per_document``, or an explicit table ``fragments``
    (``[[(doc, offset, length), ...], ...]``, one list per rank).  ``cu_seqlens_global_cpu``: the whole batch's
    ``[num_docs + 1]`` document offsets on the host."""
    from ..gdn import layout as layout_module

    if cut_points is not None:
        raise NotImplementedError("partition_kcp: cut points are not served; give an explicit fragment table")
    if isinstance(cu_seqlens_global_cpu, torch.Tensor):
        if cu_seqlens_global_cpu.is_cuda:
            raise ValueError("partition_kcp: cu_seqlens_global_cpu must be on the host")
        cu_seqlens_global_cpu = cu_seqlens_global_cpu.tolist()
    cu = tuple(int(b) for b in cu_seqlens_global_cpu)
    if len(cu) < 2 or cu[0] != 0 or any(b < a for a, b in zip(cu, cu[1:])):
        raise ValueError("partition_kcp: the document offsets must start at 0 and not decrease")
    world_size = int(world_size)
    if world_size < 1:
        raise ValueError(f"partition_kcp: world_size must be positive, got {world_size}")
    frozen = None
    if fragments is not None:
        frozen = tuple(tuple(tuple(int(x) for x in f) for f in rank) for rank in fragments)
    layout_module.partition(cu, world_size, layout, frozen)  # raises for a layout the batch does not fit
    return KcpPartition(cu, world_size, "explicit" if frozen is not None else layout, frozen)


def build_context_kcp(part: KcpPartition, group: Any, rank: int, device: Any, conv_kernel_size: int = 4, *,
                      sm_count: int | None = None, heads: Any = None, stream: Any = None) -> KcpContext:
    """This rank's context of ``part``: the argument of every KCP entry point, reusable across the calls and layers
    of the same batch layout.  ``group`` is the context-parallel process group (``None`` for a one-rank partition).
    ``sm_count``, ``heads`` and ``stream`` are accepted for the reference's signature; there is one launch plan and
    the context's table copy is a few hundred bytes.  No collective runs here."""
    if not isinstance(part, KcpPartition):
        raise TypeError(f"build_context_kcp: part must come from partition_kcp, got {type(part).__name__}")
    if group is None and part.world_size != 1:
        raise ValueError("build_context_kcp: a partition over several ranks needs its process group")
    if heads is not None:
        for count in (heads if isinstance(heads, (list, tuple)) else (heads,)):
            ops.check_heads(count)
    return KcpContext(part.cu_seqlens_global, group, int(rank), part.world_size, device, conv_kernel_size,
                      "contiguous" if part.fragments is not None else part.layout, part.fragments)


class RecomputeHandle:
    """What the original forward of a checkpointed region received over the exchange, kept for the region's replay.

    Under ``torch.utils.checkpoint`` the backward re-runs the region's forward, and with it the forward's state
    exchange -- a collective inside the backward of every rank.  A call that is given a handle stores the states that
    entered this rank's fragments in it; the replayed forward (a forward that runs while autograd's backward is
    executing) finds them and launches only this rank's kernels.  One handle per layer and micro-step, created
    outside the checkpointed region; every rank passes a handle for the same call or none (reference: the
    ``recompute_handle`` option of the reference's KCP packages)."""

    def __init__(self) -> None:
        self.entries: dict[str, Any] = {}

    def drop(self) -> None:
        self.entries.clear()


_OPTION_NAMES = ("save_mode", "recompute_handle", "checkpoint_keep", "exchange")


@dataclass(frozen=True)
class _Options:
    save_mode: str = "full"
    recompute_handle: RecomputeHandle | None = None
    exchange: str | None = None


def _options(options: dict[str, Any]) -> _Options:
    unknown = sorted(set(options) - set(_OPTION_NAMES))
    if unknown:
        raise NotImplementedError(f"the KCP entry points take the options {_OPTION_NAMES} here, not {unknown}")
    save_mode = options.get("save_mode") or "full"
    if save_mode not in ("full", "light"):
        raise ValueError(f"save_mode must be 'full' or 'light', not {save_mode!r}")
    keep = options.get("checkpoint_keep") or "states"
    if keep != "states":
        raise NotImplementedError(f"checkpoint_keep={keep!r}: a handle keeps the incoming states only ('states')")
    handle = options.get("recompute_handle")
    if handle is not None and not isinstance(handle, RecomputeHandle):
        raise TypeError(f"recompute_handle must be a RecomputeHandle, not {type(handle).__name__}")
    exchange = options.get("exchange")
    if exchange is not None and exchange not in ("auto", "sequential", "parallel"):
        raise ValueError(f"exchange must be 'auto', 'sequential' or 'parallel', not {exchange!r}")
    return _Options(save_mode, handle, exchange)


def _replaying() -> bool:
    """Whether autograd's backward is executing: a forward that runs now is a checkpointed region's replay."""
    current = getattr(torch._C, "_current_graph_task_id", None)
    if current is None:
        raise NotImplementedError("this torch cannot tell a checkpoint's replay from a forward: no recompute handles")
    return current() != -1


def _context(ctx: Any) -> KcpContext:
    if not isinstance(ctx, KcpContext):
        raise TypeError(f"ctx must be a context built by build_context_kcp, got {type(ctx).__name__}")
    return ctx


def _shard(q, k, v, g, beta, ctx: KcpContext):
    q3, k3, v3, g3 = (ops._packed3(t, n).contiguous() for t, n in ((q, "q"), (k, "k"), (v, "v"), (g, "g")))
    beta3 = ops._packed_beta(beta)
    g3 = g3 if g3.dtype == torch.float32 else g3.float()
    ops._check(q3, k3, v3, g3, beta3, ctx.cu_seqlens)
    if q3.shape[0] != ctx.num_tokens:
        raise ValueError(f"this rank's shard must hold the {ctx.num_tokens} tokens of its slice; q has {q3.shape[0]}")
    return q3, k3, v3, g3, beta3.float().contiguous()


def _exchange_of(ctx: KcpContext, mode: str | None = None):
    """The state exchange of a call: ``mode``, else the GDN op's ``--cake-gdn-kcp-exchange`` (``auto``: sequential on
    two ranks of the contiguous layout, else the parallel exchange of fragment summaries, which serves every
    layout)."""
    return ctx.exchange(mode or str(config.option("gdn", "cake_gdn_kcp_exchange") or "auto"))


def _forward_local(q3, k3, v3, g3, beta32, ctx: KcpContext, scale: float, l2norm: bool, h0):
    """This rank's kernels from known incoming states (no exchange): the replay of a forward."""
    with torch.cuda.device(q3.device):
        o, saved, _ = ops._forward(q3, k3, v3, g3, beta32, ctx.cu_seqlens, scale, l2norm,
                                   cu_seqlens_cpu=ctx.cu_seqlens_cpu, h0=h0)
    return o, saved


def _forward_kcp(q3, k3, v3, g3, beta32, ctx: KcpContext, scale: float, l2norm: bool, options: _Options = _Options()):
    handle = options.recompute_handle
    if handle is not None:
        entry = handle.entries.get("kda")
        if _replaying():
            if entry is not None:  # the region's replay: what the original forward received, no collective
                owner, shape, h0 = entry
                if owner is not ctx or shape != tuple(q3.shape):
                    raise RuntimeError("the recompute handle was filled by another context or call")
                return _forward_local(q3, k3, v3, g3, beta32, ctx, scale, l2norm, h0)
        elif entry is not None:
            raise RuntimeError("the recompute handle already holds a forward: one handle per layer and micro-step")
    o, saved = _forward_exchanging(q3, k3, v3, g3, beta32, ctx, scale, l2norm, options.exchange)
    if handle is not None and not _replaying():
        handle.entries["kda"] = (ctx, tuple(q3.shape), saved.h0)
    return o, saved


def _forward_exchanging(q3, k3, v3, g3, beta32, ctx: KcpContext, scale: float, l2norm: bool, mode: str | None):
    exchange = _exchange_of(ctx, mode)
    num_seqs, heads = len(ctx.cu_seqlens_cpu) - 1, q3.shape[1]
    if hasattr(exchange, "kda_forward_state"):  # every rank works at once
        with torch.cuda.device(q3.device):
            o, saved, _ = ops._forward(q3, k3, v3, g3, beta32, ctx.cu_seqlens, scale, l2norm,
                                       cu_seqlens_cpu=ctx.cu_seqlens_cpu, state_provider=exchange.kda_forward_state)
        return o, saved
    with torch.cuda.device(q3.device):
        h0 = exchange.incoming_state(num_seqs, heads, q3.device)
        want_final = ctx.continues_out and ctx.world_size > 1
        o, saved, final = ops._forward(q3, k3, v3, g3, beta32, ctx.cu_seqlens, scale, l2norm,
                                       cu_seqlens_cpu=ctx.cu_seqlens_cpu, h0=h0, want_final=want_final)
        if want_final:
            exchange.outgoing_state(final)
    return o, saved


def _backward_kcp(saved, v3, beta32, do3, ctx: KcpContext, mode: str | None = None):
    exchange = _exchange_of(ctx, mode)
    num_seqs, heads = len(ctx.cu_seqlens_cpu) - 1, v3.shape[1]
    if hasattr(exchange, "kda_backward_state"):
        with torch.cuda.device(v3.device):
            dq, dk, dv, dg, dbeta, _ = ops._backward(saved, v3, beta32, do3,
                                                     adjoint_provider=exchange.kda_backward_state)
        return dq, dk, dv, dg, dbeta
    with torch.cuda.device(v3.device):
        dht = exchange.incoming_adjoint(num_seqs, heads, v3.device)
        want_dh0 = ctx.continues_in and ctx.world_size > 1
        dq, dk, dv, dg, dbeta, dh0 = ops._backward(saved, v3, beta32, do3, dht=dht, want_dh0=want_dh0)
        if want_dh0:
            exchange.outgoing_adjoint(dh0)
    return dq, dk, dv, dg, dbeta


@dataclass
class _LightTape:
    """What ``save_mode="light"`` keeps: the operands as the kernels read them; the incoming states ride along."""

    q: torch.Tensor
    k: torch.Tensor
    g: torch.Tensor


class _ChunkKdaKcp(torch.autograd.Function):
    @staticmethod
    def forward(fn, q, k, v, g, beta, ctx, scale, l2norm, options):
        q3, k3, v3, g3, beta32 = _shard(q, k, v, g, beta, ctx)
        o, saved = _forward_kcp(q3, k3, v3, g3, beta32, ctx, scale, l2norm, options)
        if options.save_mode == "light":
            tape_module.keep(fn, _LightTape(q3, k3, g3), v=v3, beta32=beta32, h0=saved.h0)
        else:
            tape_module.keep(fn, saved, v=v3, beta32=beta32)
        fn.kcp, fn.call = ctx, (scale, l2norm, options)
        fn.shapes = (q.shape, g.shape, beta.shape)
        fn.dtypes = (g.dtype, beta.dtype)
        return o.view(q.shape)

    @staticmethod
    def backward(fn, do):
        shape, g_shape, beta_shape = fn.shapes
        scale, l2norm, options = fn.call
        do3 = ops._packed3(do, "dout").contiguous().to(torch.bfloat16)
        saved, kept = tape_module.restore(fn)
        if isinstance(saved, _LightTape):  # replay this rank's kernels from the states the forward received
            _, saved = _forward_local(saved.q, saved.k, kept["v"], saved.g, kept["beta32"], fn.kcp, scale, l2norm,
                                      kept["h0"])
        dq, dk, dv, dg, dbeta = _backward_kcp(saved, kept["v"], kept["beta32"], do3, fn.kcp, options.exchange)
        g_dtype, beta_dtype = fn.dtypes
        return (dq.view(shape), dk.view(shape), dv.view(shape), dg.view(g_shape).to(g_dtype),
                dbeta.view(beta_shape).to(beta_dtype), None, None, None, None)


def chunk_kda_kcp(q, k, v, g, beta, ctx, *, scale=None, use_gate_in_kernel=False, A_log=None, dt_bias=None,
                  lower_bound=None, use_qk_l2norm_in_kernel=False, **options):
    """The context-parallel autograd node of this rank's slice: ``out`` BF16 like ``v`` (this rank's tokens), with
    gradients to ``q, k, v, g, beta`` and, in the raw gate mode, to ``A_log`` / ``dt_bias`` (this rank's partial sums).
    Every rank of the group calls it in the same order.  ``options``: ``save_mode``, ``recompute_handle``,
    ``checkpoint_keep``, ``exchange`` (see the module's notes; reference: kcp.py:126-155)."""
    chosen = _options(options)
    ctx = _context(ctx)
    ops.check_heads(int(v.shape[-2]))
    config.variant(ops.OP)
    v, beta = ops.seam(v, beta)
    gate = ops._gate(g, use_gate_in_kernel, A_log, dt_bias, lower_bound)
    return _ChunkKdaKcp.apply(q, k, v, gate, beta, ctx, ops.DEFAULT_SCALE if scale is None else float(scale),
                              bool(use_qk_l2norm_in_kernel), chosen)


def chunk_kda_fwd_kcp(q, k, v, g, beta, ctx, *, scale=None, save_for_backward=True, use_gate_in_kernel=False,
                      A_log=None, dt_bias=None, lower_bound=None, use_qk_l2norm_in_kernel=False, **options):
    """The context-parallel forward alone: ``(out, saved)`` (reference: kcp.py:158-184)."""
    chosen = _options(options)
    ctx = _context(ctx)
    ops.check_heads(int(v.shape[-2]))
    v, beta = ops.seam(v, beta)
    with torch.no_grad():
        gate = ops._gate(g, use_gate_in_kernel, A_log, dt_bias, lower_bound)
        q3, k3, v3, g3, beta32 = _shard(q, k, v, gate, beta, ctx)
        o, saved = _forward_kcp(q3, k3, v3, g3, beta32, ctx, ops.DEFAULT_SCALE if scale is None else float(scale),
                                bool(use_qk_l2norm_in_kernel), chosen)
    return o.view(q.shape), (saved if save_for_backward else None)


def chunk_kda_bwd_kcp(q, k, v, g, beta, ctx, dout, *, saved=None, scale=None, use_gate_in_kernel=False, A_log=None,
                      dt_bias=None, lower_bound=None, use_qk_l2norm_in_kernel=False, **options):
    """The context-parallel backward alone: ``(dq, dk, dv, dbeta, dg)`` and, in the raw gate mode,
    ``(..., dA_log, ddt_bias)`` (this rank's partial sums); ``saved=None`` replays the forward, its exchange
    included (reference: kcp.py:187-220)."""
    chosen = _options(options)
    ctx = _context(ctx)
    ops.check_heads(int(v.shape[-2]))
    beta_dtype = beta.dtype
    v, beta = ops.seam(v, beta)
    if saved is None:
        _, saved = chunk_kda_fwd_kcp(q, k, v, g, beta, ctx, scale=scale, use_gate_in_kernel=use_gate_in_kernel,
                                     A_log=A_log, dt_bias=dt_bias, lower_bound=lower_bound,
                                     use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel, **options)
    v3 = ops._packed3(v, "v").contiguous()
    beta32 = ops._packed_beta(beta).float().contiguous()
    do3 = ops._packed3(dout, "dout").contiguous().to(torch.bfloat16)
    with torch.no_grad():
        dq, dk, dv, dg, dbeta = _backward_kcp(saved, v3, beta32, do3, ctx, chosen.exchange)
    grads = [dq.view(q.shape), dk.view(q.shape), dv.view(v.shape), dbeta.view(beta.shape).to(beta_dtype),
             dg.view(g.shape)]
    if use_gate_in_kernel:
        raw = g.detach().requires_grad_(True)
        a_leaf, b_leaf = A_log.detach().requires_grad_(True), dt_bias.detach().requires_grad_(True)
        gate = ops._activate(raw, a_leaf, b_leaf, lower_bound)
        draw, da, db = torch.autograd.grad(gate, [raw, a_leaf, b_leaf], dg.view(gate.shape))
        grads[4] = draw
        grads += [da, db]
    return tuple(grads)


def reduce_gate_param_grads_kcp(ctx, dA_log: torch.Tensor, ddt_bias: torch.Tensor):
    """The raw gate mode's full ``(dA_log, ddt_bias)`` from every rank's partial sums: one all-gather on the
    context's group, then an FP32 sum in rank order, so every rank gets the same bits whatever the collective's
    algorithm (reference: kcp.py:223-230).  Every rank of the group calls it with the same shapes."""
    ctx = _context(ctx)
    if ctx.world_size == 1 or ctx.group is None and not torch.distributed.is_initialized():
        return dA_log.clone(), ddt_bias.clone()
    import torch.distributed as dist

    packed = torch.cat([dA_log.reshape(-1).float(), ddt_bias.reshape(-1).float()])
    gathered = [torch.empty_like(packed) for _ in range(ctx.world_size)]
    dist.all_gather(gathered, packed, group=ctx.group)
    total = gathered[0].clone()
    for part in gathered[1:]:
        total += part
    n = dA_log.numel()
    return total[:n].view(dA_log.shape).to(dA_log.dtype), total[n:].view(ddt_bias.shape).to(ddt_bias.dtype)
