"""``chunk_gated_delta_rule``: FLA's signature and autograd contract on the sm_100a kernels.

Mirrors the reference's entry layer (reference: miles_ext_kernels/cake/_impl/gdn/ops.py:2300-2501 entry and checks,
:1746-1805 shape checks, :1877-2048 autograd function, :2051-2081 the empty call, :2507-2537 prebuild / release):
same argument names and meaning, same exception classes and messages, checks on tensor metadata only (no device
synchronisation), outputs and gradients as fresh allocations owned by the caller, kernels enqueued on torch's
current stream of q's device.  The entry checks (``_checked``, ``_check_inputs``, ``_cp_contract``, the empty call) are
derived from the reference's (Apache-2.0; see NOTICE): same order of checks, same words, because callers and tests
match them.
"""

from __future__ import annotations

import math
from collections.abc import Sequence
from pathlib import Path
from typing import Any

import torch

from ..._runtime import config, loader, registry
from . import meta as meta_module
from . import native, stages
from . import tape as tape_module
from .kcp import KcpContext

OP = "gdn"
HEAD_DIM = 128
CHUNK = 64

_OFFSET_DTYPES = (torch.int32, torch.int64)
_INPUT_NAMES = ("q", "k", "v", "g", "beta", "initial_state", "cu_seqlens")
_FIRST_OPTIONAL = 5


# --------------------------------------------------------------------------------------------------------------------
# checks (metadata only)
# --------------------------------------------------------------------------------------------------------------------
def _checked(q, k, v, g, scale, chunk_size, unsupported) -> tuple[torch.Tensor, float]:
    """The checks every route shares; returns ``g`` in FP32 and the scale (``1 / sqrt(K)`` by default)."""
    for name, value in unsupported.items():
        if value not in (None, False):
            raise NotImplementedError(f"chunk_gated_delta_rule: {name}={value!r} is not supported by the Cake kernels")
    if chunk_size != CHUNK:
        raise NotImplementedError(f"chunk_gated_delta_rule: chunk_size must be {CHUNK}")
    if not (q.dtype == k.dtype == v.dtype == torch.bfloat16):
        raise NotImplementedError("chunk_gated_delta_rule: q/k/v must be bfloat16")
    if q.shape[-1] != HEAD_DIM or v.shape[-1] != HEAD_DIM:
        raise NotImplementedError("chunk_gated_delta_rule: head dims must be 128")
    if g.dtype != torch.float32:
        g = g.float()
    return g, float(1.0 / math.sqrt(q.shape[-1]) if scale is None else scale)


def _check_inputs(q, k, v, g, beta, initial_state, cu_seqlens, cu_seqlens_cpu) -> None:
    """Extents of a call, from tensor metadata only: CUDA tensors on one device, q / k ``[B, T, H, 128]``, v ``[B, T,
    HV, 128]`` with ``HV % H == 0``, g and beta ``[B, T, HV]``, ``cu_seqlens`` a 1-D int32 / int64 tensor of at least
    two offsets with ``B = 1`` and a host copy of as many offsets, one ``[HV, 128, 128]`` initial state per sequence."""
    home = None
    for position, tensor in enumerate((q, k, v, g, beta, initial_state, cu_seqlens)):
        if tensor is None and position >= _FIRST_OPTIONAL:
            continue
        name = _INPUT_NAMES[position]
        if not isinstance(tensor, torch.Tensor) or not tensor.is_cuda:
            raise ValueError(f"chunk_gated_delta_rule: {name} must be a CUDA tensor")
        if home is None:
            home = tensor.get_device()
        elif tensor.get_device() != home:
            raise ValueError(f"chunk_gated_delta_rule: {name} is on {tensor.device}, q on {q.device}")
    if q.dim() != 4 or q.shape[3] != HEAD_DIM:
        raise ValueError(f"chunk_gated_delta_rule: q must be [B, T, H, {HEAD_DIM}]; got {tuple(q.shape)}")
    if k.shape != q.shape:
        raise ValueError(f"chunk_gated_delta_rule: k must have q's shape {tuple(q.shape)}; got {tuple(k.shape)}")
    B, T, H = q.shape[0], q.shape[1], q.shape[2]
    if v.dim() != 4 or v.shape[0] != B or v.shape[1] != T or v.shape[3] != HEAD_DIM:
        raise ValueError(f"chunk_gated_delta_rule: v must be [{B}, {T}, HV, {HEAD_DIM}]; got {tuple(v.shape)}")
    HV = v.shape[2]
    if H == 0 or HV == 0 or HV % H:
        raise ValueError(
            f"chunk_gated_delta_rule: the value heads (HV={HV}) must be a positive multiple of the q / k heads (H={H})"
        )
    gates = v.shape[:3]
    if g.shape != gates:
        raise ValueError(f"chunk_gated_delta_rule: g must be {tuple(gates)}; got {tuple(g.shape)}")
    if beta.shape != gates:
        raise ValueError(f"chunk_gated_delta_rule: beta must be {tuple(gates)}; got {tuple(beta.shape)}")
    if cu_seqlens is None:
        num_seqs = B
    else:
        offsets = cu_seqlens.numel()
        if cu_seqlens.dim() != 1 or offsets < 2 or cu_seqlens.dtype not in _OFFSET_DTYPES:
            raise ValueError(
                "chunk_gated_delta_rule: cu_seqlens must be a 1-D int32 / int64 tensor of at least two offsets; got "
                f"{cu_seqlens.dtype} {tuple(cu_seqlens.shape)}"
            )
        if B != 1:
            raise ValueError("chunk_gated_delta_rule: cu_seqlens requires a leading batch dimension of 1")
        num_seqs = offsets - 1
        if cu_seqlens_cpu is not None:
            count = cu_seqlens_cpu.numel() if isinstance(cu_seqlens_cpu, torch.Tensor) else len(cu_seqlens_cpu)
            if count != offsets:
                raise ValueError(f"chunk_gated_delta_rule: cu_seqlens_cpu has {count} offsets, cu_seqlens {offsets}")
    if initial_state is not None:
        want = (num_seqs, HV, HEAD_DIM, HEAD_DIM)
        if tuple(initial_state.shape) != want:
            raise ValueError(
                f"chunk_gated_delta_rule: initial_state must be {want} (one state per sequence); got "
                f"{tuple(initial_state.shape)}"
            )


def _cp_contract(cp_context, initial_state, output_final_state, cu_seqlens, cu_seqlens_cpu):
    """FLA's context-parallel contract: no initial state, no final state, the context's own boundaries."""
    if cp_context is None:
        return cu_seqlens, cu_seqlens_cpu
    if initial_state is not None:
        raise ValueError("chunk_gated_delta_rule: initial_state is not supported under context parallelism")
    if output_final_state:
        raise ValueError("chunk_gated_delta_rule: output_final_state is not supported under context parallelism")
    local = getattr(cp_context, "cu_seqlens", None)
    if local is None:
        raise ValueError("chunk_gated_delta_rule: context parallelism needs the cp_context's cu_seqlens")
    host = getattr(cp_context, "cu_seqlens_cpu", None)
    return local, (cu_seqlens_cpu if host is None else host)


def _save_state() -> bool:
    """Keep w / u / h / v_new on the tape unless ``--cake-gdn-recompute-state`` is set."""
    return not config.option(OP, "cake_gdn_recompute_state")


def _scan_segments() -> int:
    """``--cake-gdn-scan-segments``: 0 = the scan planner decides, 1 = serial scans, more = that many segments."""
    return int(config.option(OP, "cake_gdn_scan_segments") or 0)


# --------------------------------------------------------------------------------------------------------------------
# the empty call
# --------------------------------------------------------------------------------------------------------------------
class _NoTokens(torch.autograd.Function):
    """A call with no token: an empty output; the final state is the initial state (zero without one), and the
    gradient of the initial state is the final state's."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, initial_state, output_final_state: bool, num_seqs: int):
        ctx.inputs = tuple((t.shape, t.dtype, t.device) for t in (q, k, v, g, beta))
        ctx.state_dtype = None if initial_state is None else initial_state.dtype
        output = torch.empty(v.shape, dtype=q.dtype, device=v.device)
        if not output_final_state:
            return output, None
        if initial_state is not None:
            return output, initial_state.detach().float().clone()
        return output, torch.zeros((num_seqs, v.shape[-2], HEAD_DIM, HEAD_DIM), dtype=torch.float32, device=v.device)

    @staticmethod
    def backward(ctx, do, dht):
        grads = [torch.zeros(shape, dtype=dtype, device=device) for shape, dtype, device in ctx.inputs]
        dh0 = None if ctx.state_dtype is None or dht is None else dht.to(ctx.state_dtype)
        return (*grads, dh0, None, None)


def _no_tokens(q, k, v, g, beta, initial_state, output_final_state, cu_seqlens):
    num_seqs = q.shape[0] if cu_seqlens is None else int(cu_seqlens.numel()) - 1
    want = (num_seqs, v.shape[-2], HEAD_DIM, HEAD_DIM)
    if initial_state is not None and tuple(initial_state.shape) != want:
        raise ValueError(
            f"chunk_gated_delta_rule: initial_state must be {want} (one state per sequence); got "
            f"{tuple(initial_state.shape)}"
        )
    return _NoTokens.apply(q, k, v, g, beta, initial_state, bool(output_final_state), num_seqs)


# --------------------------------------------------------------------------------------------------------------------
# autograd
# --------------------------------------------------------------------------------------------------------------------
def _packed(x: torch.Tensor) -> torch.Tensor:
    """``[B, T, heads, ...]`` -> contiguous ``[B * T, heads, ...]`` (a view when x is contiguous)."""
    return x.contiguous().view(x.shape[0] * x.shape[1], *x.shape[2:])


def _rows(x: torch.Tensor) -> torch.Tensor:
    """``[B, T, heads, 128]`` -> ``[B * T, heads, 128]`` without a copy when x is dense or a column slice of a wider
    packed row (heads contiguous inside a token, tokens a fixed stride apart, 16-byte aligned): the kernels take the
    token stride.  Anything else is made contiguous first."""
    B, T = x.shape[0], x.shape[1]
    if x.is_contiguous():
        return x.view(B * T, *x.shape[2:])
    pitch = x.stride(1)
    sliced = (
        x.stride(3) == 1 and x.stride(2) == HEAD_DIM and pitch >= x.shape[2] * HEAD_DIM and pitch % 8 == 0
        and (B == 1 or x.stride(0) == T * pitch) and x.data_ptr() % 16 == 0
    )
    if not sliced:
        return x.contiguous().view(B * T, *x.shape[2:])
    return x.as_strided((B * T, x.shape[2], HEAD_DIM), (pitch, HEAD_DIM, 1))


def _tile_one_row(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    """Whether q, k, v ``[T, heads, 128]`` are the column slices ``[q heads | k heads | v heads]`` of one packed row
    ``[T, (2 H + HV) * 128]``: their gradients are then written as the same slices of one packed gradient row."""
    H, HV = q.shape[1], v.shape[1]
    width = (2 * H + HV) * HEAD_DIM
    if q.is_contiguous() or not (q.stride(0) == k.stride(0) == v.stride(0) == width):
        return False
    if not (q.untyped_storage().data_ptr() == k.untyped_storage().data_ptr() == v.untyped_storage().data_ptr()):
        return False
    base = q.storage_offset()
    return k.storage_offset() == base + H * HEAD_DIM and v.storage_offset() == base + 2 * H * HEAD_DIM


class ChunkGatedDeltaRuleFunction(torch.autograd.Function):
    """The kernels with FLA's autograd contract.  ``save_state`` keeps w / u / h / v_new for the backward; without it
    the backward recomputes them with the forward's kernels (the same bits).  ``exchange`` (context parallelism)
    supplies the incoming chunk state in the forward and the incoming adjoint state in the backward."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens, cu_seqlens_cpu,
                use_qk_l2norm, save_state, exchange):
        B, T, H = q.shape[0], q.shape[1], q.shape[2]
        HV = v.shape[2]
        device = q.device
        with torch.cuda.device(device):
            meta = meta_module.chunk_meta(cu_seqlens, cu_seqlens_cpu, B, T, device)
            beta32 = _packed(beta if beta.dtype == torch.float32 else beta.float())
            qp, kp, vp, gp = _rows(q), _rows(k), _rows(v), _packed(g)
            if qp.stride(0) != kp.stride(0):  # the kernels take one token stride for q and k
                qp, kp = qp.contiguous(), kp.contiguous()
            ctx.packed_grads = _tile_one_row(qp, kp, vp)
            h0 = None if initial_state is None else initial_state.detach().float().contiguous()
            want_final = bool(output_final_state)
            ctx.scan_segments = _scan_segments()
            # under context parallelism the exchange supplies the state at this rank's start and takes the one at
            # its end (inside the stages: the parallel exchange needs the WY outputs first)
            o, final_state, tape, h0 = stages.forward(qp, kp, vp, gp, beta32, meta, scale, h0, want_final,
                                                      bool(use_qk_l2norm), keep_state=bool(save_state),
                                                      scan_segments=ctx.scan_segments, exchange=exchange)
        # every tensor of the tape through save_for_backward (version checks, saved-tensor hooks); metadata as attributes
        tape_module.keep(ctx, tape, h0=h0)
        ctx.meta, ctx.scale = meta, scale
        ctx.exchange = exchange
        ctx.shapes = (q.shape, v.shape, g.shape)
        ctx.g_dtype, ctx.beta_dtype = g.dtype, beta.dtype
        ctx.state_dtype = None if initial_state is None else initial_state.dtype
        ctx.has_initial_state = initial_state is not None
        ctx.set_materialize_grads(False)
        return o.view(v.shape), final_state

    @staticmethod
    def backward(ctx, do, dht):
        q_shape, v_shape, g_shape = ctx.shapes
        tape, kept = tape_module.restore(ctx)
        meta = ctx.meta
        device = tape.qn.device
        with torch.cuda.device(device):
            if do is None:
                do = torch.zeros(v_shape, dtype=torch.bfloat16, device=device)
            dop = _packed(do if do.dtype == torch.bfloat16 else do.bfloat16())
            dhtp = None if dht is None else dht.float().contiguous()
            want_dh0 = ctx.has_initial_state
            dq, dk, dv, dg, dbeta, dh0 = stages.backward(tape, meta, ctx.scale, dop, dhtp, kept["h0"], want_dh0,
                                                               scan_segments=ctx.scan_segments, exchange=ctx.exchange,
                                                               packed_grads=ctx.packed_grads)
        dq, dk, dv = dq.view(q_shape), dk.view(q_shape), dv.view(v_shape)
        dg = dg.view(g_shape)
        dbeta = dbeta.view(g_shape)
        if dg.dtype != ctx.g_dtype:
            dg = dg.to(ctx.g_dtype)
        if dbeta.dtype != ctx.beta_dtype:
            dbeta = dbeta.to(ctx.beta_dtype)
        if dh0 is not None and dh0.dtype != ctx.state_dtype:
            dh0 = dh0.to(ctx.state_dtype)
        return dq, dk, dv, dg, dbeta, None, dh0, None, None, None, None, None, None


def _apply(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens, cu_seqlens_cpu, use_qk_l2norm,
           exchange=None):
    _check_inputs(q, k, v, g, beta, initial_state, cu_seqlens, cu_seqlens_cpu)
    if q.shape[0] * q.shape[1] == 0 and exchange is None:
        return _no_tokens(q, k, v, g, beta, initial_state, output_final_state, cu_seqlens)
    return ChunkGatedDeltaRuleFunction.apply(
        q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens, cu_seqlens_cpu, use_qk_l2norm,
        _save_state(), exchange,
    )


# --------------------------------------------------------------------------------------------------------------------
# packed q / k / v
# --------------------------------------------------------------------------------------------------------------------
def _common_row(dq, dk, dv, H: int, HV: int):
    """The packed gradient row whose column slices ``[q heads | k heads | v heads]`` dq, dk, dv are, or None."""
    if dq is None or dk is None or dv is None:
        return None
    row = dq._base
    if row is None or dk._base is not row or dv._base is not row or not row.is_contiguous():
        return None
    width = (2 * H + HV) * HEAD_DIM
    size = dq.element_size()
    tokens = dq.numel() // (H * HEAD_DIM)
    if row.numel() != tokens * width or row.dtype != dq.dtype:
        return None
    if not (dq.stride(-1) == dk.stride(-1) == dv.stride(-1) == 1 and dq.stride(-2) == dk.stride(-2) == dv.stride(-2)
            == HEAD_DIM and dq.stride(-3) == dk.stride(-3) == dv.stride(-3) == width):
        return None
    base = row.data_ptr()
    if dq.data_ptr() != base or dk.data_ptr() != base + H * HEAD_DIM * size or \
            dv.data_ptr() != base + 2 * H * HEAD_DIM * size:
        return None
    return row


class _PackedQkvViews(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, num_qk_heads: int, num_v_heads: int):
        H, HV = int(num_qk_heads), int(num_v_heads)
        ctx.heads, ctx.shape = (H, HV), qkv.shape
        lead = qkv.shape[:-1]
        q = qkv[..., : H * HEAD_DIM].unflatten(-1, (H, HEAD_DIM))
        k = qkv[..., H * HEAD_DIM : 2 * H * HEAD_DIM].unflatten(-1, (H, HEAD_DIM))
        v = qkv[..., 2 * H * HEAD_DIM :].unflatten(-1, (HV, HEAD_DIM))
        assert q.shape[:-2] == lead
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        H, HV = ctx.heads
        row = _common_row(dq, dk, dv, H, HV)
        if row is not None:  # the op wrote the three gradients as the slices of one row: that row is the gradient
            return row.view(ctx.shape), None, None
        lead = ctx.shape[:-1]
        like = next(t for t in (dq, dk, dv) if t is not None)
        pieces = []
        for grad, heads in ((dq, H), (dk, H), (dv, HV)):
            if grad is None:
                grad = torch.zeros((*lead, heads, HEAD_DIM), dtype=like.dtype, device=like.device)
            pieces.append(grad.reshape(*lead, heads * HEAD_DIM))
        return torch.cat(pieces, dim=-1), None, None


def packed_qkv_views(qkv: torch.Tensor, num_qk_heads: int, num_v_heads: int):
    """``q [.., H, 128]``, ``k [.., H, 128]``, ``v [.., HV, 128]`` as views of one packed row ``qkv [.., (2 H + HV) *
    128]`` laid out ``[q heads | k heads | v heads]`` (the row a fused projection writes).

    :func:`chunk_gated_delta_rule` reads such views in place (no copies) and writes their gradients as the same
    slices of one packed gradient row; the backward of this split hands that row on as ``qkv``'s gradient instead of
    concatenating three tensors.  Plain ``split`` / ``view`` views of the row give the same bits, with the
    concatenation (reference: ``packed_qkv_views`` of the context-parallel packages,
    miles_ext_kernels/cake/_vendor/cake_gdn_det_train_kcp/README.md:314-356)."""
    width = (2 * int(num_qk_heads) + int(num_v_heads)) * HEAD_DIM
    if qkv.shape[-1] != width:
        raise ValueError(f"packed_qkv_views: the row must hold (2 * {num_qk_heads} + {num_v_heads}) * {HEAD_DIM} = "
                         f"{width} columns; it has {qkv.shape[-1]}")
    return _PackedQkvViews.apply(qkv, num_qk_heads, num_v_heads)


# --------------------------------------------------------------------------------------------------------------------
# entry points
# --------------------------------------------------------------------------------------------------------------------
def chunk_gated_delta_rule(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    scale: float | None = None,
    initial_state: torch.Tensor | None = None,
    output_final_state: bool = False,
    cu_seqlens: torch.LongTensor | None = None,
    cu_seqlens_cpu: torch.LongTensor | Sequence[int] | None = None,
    use_qk_l2norm_in_kernel: bool = False,
    cp_context: Any = None,
    chunk_size: int = 64,
    **unsupported: Any,
):
    """FLA v0.5.2 ``chunk_gated_delta_rule`` signature on the sm_100a kernels.

    Supported: ``[B, T, H, K]`` q / k and ``[B, T, HV, V]`` v with ``K = V = 128`` and ``HV % H == 0``, BF16 q / k / v,
    packed varlen via ``cu_seqlens`` (``B = 1``), FP32 ``initial_state`` / ``output_final_state`` (V-last ``[N, HV, K,
    V]``), ``use_qk_l2norm_in_kernel``, and ``cp_context`` state passing.  Gate fusion, beta sigmoid fusion,
    ``state_v_first``, ``head_first`` and other chunk sizes are rejected.  A call with no token returns an empty
    output (and the initial state as the final state).  Returns ``(o, final_state | None)``.

    ``cu_seqlens_cpu`` (the same boundaries on the host: a tuple of ints or a CPU tensor) selects the exact chunk
    table shared by every layer of the micro-batch; without it the table is built on the device per call.

    Under any ``cp_context`` the contract is FLA's: ``initial_state`` and ``output_final_state`` are rejected and the
    context's boundaries replace ``cu_seqlens`` / ``cu_seqlens_cpu``.  A :class:`KcpContext` holds this rank's
    contiguous token slice; the chunk state crosses the ranks of its group (:func:`kcp_chunk_gated_delta_rule`).
    Both variants (``det``, ``fast``) run the same fixed-order kernels.
    """
    g, scale = _checked(q, k, v, g, scale, chunk_size, unsupported)
    config.variant(OP)  # raises for a configuration this op cannot run; both variants share the kernels
    if cp_context is not None:
        if not isinstance(cp_context, KcpContext):
            raise TypeError(
                f"chunk_gated_delta_rule: cp_context must be a KcpContext (build_kcp_context), not "
                f"{type(cp_context).__name__}"
            )
        cu_seqlens, cu_seqlens_cpu = _cp_contract(cp_context, initial_state, output_final_state, cu_seqlens,
                                                  cu_seqlens_cpu)
        return _apply(q, k, v, g, beta, scale, None, False, cu_seqlens, cu_seqlens_cpu, use_qk_l2norm_in_kernel,
                      exchange=cp_context.exchange(str(config.option(OP, "cake_gdn_kcp_exchange") or "auto")))
    return _apply(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens, cu_seqlens_cpu,
                  use_qk_l2norm_in_kernel)


def kcp_chunk_gated_delta_rule(q, k, v, g, beta, kcp_context, scale=None, use_qk_l2norm_in_kernel=False,
                               chunk_size=64):
    """The context-parallel call: this rank's tokens of ``kcp_context``; returns ``o`` only (reference:
    miles_ext_kernels/cake/_impl/gdn/ops.py:2244-2272)."""
    if not isinstance(kcp_context, KcpContext):
        raise TypeError(f"kcp_chunk_gated_delta_rule: kcp_context must be a KcpContext, not {type(kcp_context).__name__}")
    out, _ = chunk_gated_delta_rule(q, k, v, g, beta, scale=scale, use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel,
                                    cp_context=kcp_context, chunk_size=chunk_size)
    return out


# --------------------------------------------------------------------------------------------------------------------
# prebuild and release
# --------------------------------------------------------------------------------------------------------------------
def prebuild(*, device: Any = None, max_workers: int | None = None) -> list[Path]:
    """Build (or find) the native library for the architecture of ``device``.  No model parameter: every call of
    the op launches kernels of this one library.  ``NotImplementedError`` for a device other than SM100a,
    ``RuntimeError`` when the toolkit is too old.  Returns the library paths."""
    arch = loader.device_arch(device)
    return loader.prebuild_libraries(registry.op_spec(OP).packages, arch, max_workers=max_workers)


def release() -> None:
    """Drop what the op keeps between calls besides the workspace pool: the chunk tables per layout, the cached
    contexts and the library handle."""
    meta_module.host_cache_clear()
    native.release()
    from . import kcp, scan

    scan.release()

    kcp.release()
