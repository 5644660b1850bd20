"""Packed KDA chunked training on the sm_100a kernels: ``chunk_kda``, ``chunk_kda_fwd``, ``chunk_kda_bwd``.

Entry points, argument meaning and returns follow the reference (reference:
miles_ext_kernels/cake/_impl/kda/ops.py:107-234): one packed batch ``[S, H, 128]`` (or ``[1, S, H, 128]``) of documents
described by a device ``cu_seqlens``, 1 to 64 heads, zero initial state per document, no final state; ``beta`` is
rounded to BF16 at the seam; the gate is the activated natural-log decay ``g [S, H, 128]`` (FP32), or with
``use_gate_in_kernel`` the raw gate with ``A_log [H]`` / ``dt_bias [H * 128]`` / ``lower_bound``; the q / k L2 norm may
run in the op.

The raw gate's activation ``lower_bound * sigmoid(exp(A_log)(raw + dt_bias))`` runs as torch ops under autograd
(element-wise, outside the kernels), so the gradients of ``raw``, ``A_log`` and ``dt_bias`` come from the kernels'
``dg`` through that graph.  The chunk table is built on the device from ``cu_seqlens`` without a synchronisation.
"""

from __future__ import annotations

import operator
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

from ..._runtime import config, loader, registry, workspace
from ..gdn import meta as meta_module
from ..gdn import native, scan
from ..gdn import tape as tape_module
from ..gdn.stages import check_status, dims_of

OP = "kda"
HEAD_DIM = 128
MAX_HEADS = 64
DEFAULT_SCALE = HEAD_DIM**-0.5
LOWER_BOUND = -5.0
BF16, F32 = torch.bfloat16, torch.float32

__all__ = ["DEFAULT_SCALE", "MAX_HEADS", "chunk_kda", "chunk_kda_bwd", "chunk_kda_fwd", "prebuild", "release"]


def check_heads(num_heads: Any) -> int:
    """``num_heads`` as an int when the kernels serve it (1 to :data:`MAX_HEADS`), else ``ValueError``."""
    try:
        heads = None if isinstance(num_heads, bool) else operator.index(num_heads)
    except TypeError:
        heads = None
    if heads is None or not 1 <= heads <= MAX_HEADS:
        raise ValueError(
            f"the Cake KDA kernels serve 1 to {MAX_HEADS} heads per call (per tensor-parallel rank of a head-sharded "
            f"layer), got {num_heads!r}: shard the heads over more ranks with --tensor-model-parallel-size, or use "
            "--kda-backend fla"
        )
    return heads


def seam(v: torch.Tensor, beta: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``v`` dense and ``beta`` BF16 and dense, as the kernels read them (differentiable)."""
    if beta.is_floating_point() and beta.dtype != torch.bfloat16:
        beta = beta.to(torch.bfloat16)
    return v.contiguous(), beta.contiguous()


def _activate(raw, A_log, dt_bias, lower_bound):
    """``lower_bound * sigmoid(exp(A_log)[h] (raw + dt_bias[h]))`` in FP32 (reference: tests/cake/kda/_reference.py:86-99)."""
    if A_log is None or dt_bias is None:
        raise ValueError("chunk_kda: use_gate_in_kernel needs A_log and dt_bias")
    H = raw.shape[-2]
    lb = LOWER_BOUND if lower_bound is None else float(lower_bound)
    a = torch.exp(A_log.float()).reshape(H, 1)
    return lb * torch.sigmoid(a * (raw.float() + dt_bias.float().reshape(H, HEAD_DIM)))


def _packed3(x: torch.Tensor, name: str) -> torch.Tensor:
    if x.dim() == 4:
        if x.shape[0] != 1:
            raise ValueError(f"chunk_kda: {name} must be one packed batch [1, S, H, 128]; got {tuple(x.shape)}")
        x = x[0]
    return x


def _packed_beta(beta: torch.Tensor) -> torch.Tensor:
    """``[1, S, H]`` -> ``[S, H]`` (``[S, H]`` passes through)."""
    if beta.dim() == 3:
        if beta.shape[0] != 1:
            raise ValueError(f"chunk_kda: beta must be one packed batch [1, S, H]; got {tuple(beta.shape)}")
        return beta[0]
    return beta


def _check(q, k, v, g, beta, cu_seqlens) -> None:
    for name, t in (("q", q), ("k", k), ("v", v), ("g", g), ("beta", beta), ("cu_seqlens", cu_seqlens)):
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise ValueError(f"chunk_kda: {name} must be a CUDA tensor")
        if t.get_device() != q.get_device():
            raise ValueError(f"chunk_kda: {name} is on {t.device}, q on {q.device}")
    if q.dim() != 3 or q.shape[-1] != HEAD_DIM:
        raise ValueError(f"chunk_kda: q must be [S, H, {HEAD_DIM}]; got {tuple(q.shape)}")
    for name, t in (("k", k), ("v", v), ("g", g)):
        if t.shape != q.shape:
            raise ValueError(f"chunk_kda: {name} must have q's shape {tuple(q.shape)}; got {tuple(t.shape)}")
    if beta.shape != q.shape[:2]:
        raise ValueError(f"chunk_kda: beta must be {tuple(q.shape[:2])}; got {tuple(beta.shape)}")
    if not (q.dtype == k.dtype == v.dtype == torch.bfloat16):
        raise NotImplementedError("chunk_kda: q/k/v must be bfloat16")
    if cu_seqlens.dim() != 1 or cu_seqlens.numel() < 2 or cu_seqlens.dtype not in (torch.int32, torch.int64):
        raise ValueError("chunk_kda: cu_seqlens must be a 1-D int32 / int64 tensor of at least two offsets")


@dataclass
class Saved:
    """What the forward leaves for :func:`chunk_kda_bwd` (packed layouts; read by this package only)."""

    meta: Any
    scale: float
    qn: torch.Tensor
    kn: torch.Tensor
    q_raw: torch.Tensor | None
    k_raw: torch.Tensor | None
    rstd_q: torch.Tensor | None
    rstd_k: torch.Tensor | None
    g2: torch.Tensor
    gl2: torch.Tensor
    qg: torch.Tensor
    kg: torch.Tensor
    kr: torch.Tensor
    a: torch.Tensor
    aqk: torch.Tensor
    w: torch.Tensor
    h: torch.Tensor
    v_new: torch.Tensor
    status: torch.Tensor
    h0: torch.Tensor | None = None  # the states that entered this rank's fragments (context parallelism), else None


def _scan_segments() -> int:
    """0: the scan planner decides; 1: serial walks; more: that many segments per long sequence (the GDN op's
    ``--cake-gdn-scan-segments``, which the two ops share with the planner)."""
    try:
        return int(config.option("gdn", "cake_gdn_scan_segments") or 0)
    except (KeyError, ValueError):
        return 0


def _scan_forward(dims, meta, kr, w, u, gl2, h0, h, v_new, want_final: bool, status):
    """The state scan: one serial walk per (sequence, head), or -- when the call has fewer chains than half the SMs
    and the planner's cost model gains -- pre-scan, stitch and a walk over segments from their true start states
    (every summary exact: the gate-adaptive warm-up reads scalar gates and stays off).  Returns the final states or
    None."""
    device = kr.device
    H = w.shape[1]
    plan = scan.plan_for(meta, H, device, _scan_segments())
    shape = (HEAD_DIM, HEAD_DIM)
    if plan is None:
        final = torch.empty((meta.num_seqs, H, *shape), dtype=F32, device=device) if want_final else None
        native.launch("kda_fwd_h", dims, kr, w, u, gl2, h0, h, v_new, final, status, device=device)
        return final
    seg_dims = scan.segment_dims(dims, plan)
    summary = workspace.take(OP, "scan_summary", (plan.segments, H, 2, *shape), F32, device)
    seg_state = workspace.take(OP, "scan_state", (plan.segments, H, *shape), F32, device)
    native.launch("kda_fwd_h_prescan", seg_dims, kr, w, u, gl2, h0, plan.flags_fwd, plan.state_row, summary, status,
                  device=device)
    native.launch("gdn_scan_stitch", seg_dims, plan.num_seqs, plan.seq_seg_start, summary, h0, None, seg_state, None, 0,
                  0, 0.0, 0, device=device)
    seg_final = workspace.take(OP, "scan_final", (plan.segments, H, *shape), F32, device) if want_final else None
    native.launch("kda_fwd_h", seg_dims, kr, w, u, gl2, seg_state, h, v_new, seg_final, status, device=device)
    return seg_final.index_select(0, plan.last_index) if want_final else None


def _scan_backward(dims, meta, s, do, dht, dh, dv_new, want_dh0: bool):
    """The adjoint scan, serial or segmented like the forward's.  Returns dh0 or None."""
    device = do.device
    H = do.shape[1]
    plan = scan.plan_for(meta, H, device, _scan_segments())
    shape = (HEAD_DIM, HEAD_DIM)
    if plan is None:
        dh0 = torch.empty((meta.num_seqs, H, *shape), dtype=F32, device=device) if want_dh0 else None
        native.launch("kda_bwd_dh", dims, s.qg, s.kr, s.w, do, s.aqk, s.gl2, dht, dh, dv_new, dh0, s.status,
                      device=device)
        return dh0
    seg_dims = scan.segment_dims(dims, plan)
    summary = workspace.take(OP, "scan_summary", (plan.segments, H, 2, *shape), F32, device)
    seg_state = workspace.take(OP, "scan_state", (plan.segments, H, *shape), F32, device)
    native.launch("kda_bwd_dh_prescan", seg_dims, s.qg, s.kr, s.w, do, s.aqk, s.gl2, dht, plan.flags_bwd,
                  plan.state_row, summary, s.status, device=device)
    native.launch("gdn_scan_stitch", seg_dims, plan.num_seqs, plan.seq_seg_start, summary, dht, None, seg_state, None,
                  1, 0, 0.0, 0, device=device)
    seg_dh0 = workspace.take(OP, "scan_final", (plan.segments, H, *shape), F32, device) if want_dh0 else None
    native.launch("kda_bwd_dh", seg_dims, s.qg, s.kr, s.w, do, s.aqk, s.gl2, seg_state, dh, dv_new, seg_dh0, s.status,
                  device=device)
    return seg_dh0.index_select(0, plan.first_index) if want_dh0 else None


def _forward(q, k, v, g, beta32, cu_seqlens, scale, use_qk_l2norm, *, cu_seqlens_cpu=None, h0=None,
             want_final=False, state_provider=None):
    """q, k, v ``[S, H, 128]`` bf16 contiguous; g fp32 ``[S, H, 128]``; beta32 fp32 ``[S, H]``.  ``h0`` (fp32
    ``[N, H, 128, 128]`` or None) and ``want_final`` are the boundary states of a context-parallel call;
    ``state_provider(dims, meta, kr, w, u, gl2, status) -> h0`` computes them from the scan's operands instead (the
    parallel exchange, which summarises this rank's fragments first).  Returns ``(o, saved, final_state | None)``."""
    device = q.device
    S, H = q.shape[0], q.shape[1]
    meta = meta_module.chunk_meta(cu_seqlens, cu_seqlens_cpu, 1, S, device)
    NC = meta.num_chunks
    dims = dims_of(meta, H, H, scale)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    q_raw = k_raw = rstd_q = rstd_k = None
    if use_qk_l2norm:
        q_raw, k_raw = q, k
        rstd_q, rstd_k = (torch.empty((S, H), dtype=F32, device=device) for _ in range(2))
        q, k = torch.empty_like(q), torch.empty_like(k)
        native.launch("gdn_l2norm", q_raw, q, rstd_q, S * H, H, 0, device=device)
        native.launch("gdn_l2norm", k_raw, k, rstd_k, S * H, H, 0, device=device)
    g2 = torch.empty((S, H, HEAD_DIM), dtype=F32, device=device)
    qg, kg, kr = (torch.empty_like(q) for _ in range(3))
    # pad chunks of the device route are never written: their tiles must not hold NaN bit patterns
    alloc = torch.empty if meta.exact else torch.zeros
    gl2 = alloc((NC, H, HEAD_DIM), dtype=F32, device=device)
    native.launch("kda_prep", dims, q, k, g, g2, qg, kg, kr, gl2, device=device)
    a = alloc((NC, H, 64, 64), dtype=BF16, device=device)
    aqk = alloc((NC, H, 64, 64), dtype=BF16, device=device)
    w, u = torch.empty_like(v), torch.empty_like(v)
    native.launch("kda_intra", dims, q, k, v, kg, g2, beta32, a, aqk, w, u, status, device=device)
    h = alloc((NC, H, HEAD_DIM, HEAD_DIM), dtype=BF16, device=device)
    v_new = torch.empty_like(v)
    if state_provider is not None:
        h0 = state_provider(dims, meta, kr, w, u, gl2, status)
    final = _scan_forward(dims, meta, kr, w, u, gl2, h0, h, v_new, want_final, status)
    o = torch.empty_like(v)
    native.launch("kda_fwd_o", dims, qg, aqk, v_new, h, o, status, device=device)
    saved = Saved(meta, scale, q, k, q_raw, k_raw, rstd_q, rstd_k, g2, gl2, qg, kg, kr, a, aqk, w, h, v_new, status, h0)
    return o, saved, final


def _backward(s: Saved, v, beta32, do, *, dht=None, want_dh0=False, adjoint_provider=None):
    """Returns ``(dq, dk, dv, dg, dbeta, dh0 | None)``; ``dht`` / ``want_dh0``: the boundary adjoint states of a
    context-parallel call (fp32 ``[N, H, 128, 128]``)."""
    device = do.device
    S, H = v.shape[0], v.shape[1]
    meta = s.meta
    NC = meta.num_chunks
    dims = dims_of(meta, H, H, s.scale)
    take = lambda role, shape, dtype: workspace.take(OP, role, shape, dtype, device)  # noqa: E731
    if meta.exact:
        dh = take("dh_tape", (NC, H, HEAD_DIM, HEAD_DIM), BF16)
    else:  # pad chunks are never written
        dh = torch.zeros((NC, H, HEAD_DIM, HEAD_DIM), dtype=BF16, device=device)
    dv_new = take("dv_new", (S, H, HEAD_DIM), BF16)
    if adjoint_provider is not None:
        dht = adjoint_provider(dims, meta, s, do)
    dh0 = _scan_backward(dims, meta, s, do, dht, dh, dv_new, want_dh0)
    m1 = take("m1", (NC, H, 64, 64), F32)
    m2 = take("m2", (NC, H, 64, 64), F32)
    dqg, dkr, dkg = (take(role, (S, H, HEAD_DIM), F32) for role in ("dqg", "dkr", "dkg"))
    hdh = take("hdh", (NC, H, HEAD_DIM), F32)
    dbeta_part = take("dbeta_part", (S, H), F32)
    dq32, dk32 = take("dq32", (S, H, HEAD_DIM), F32), take("dk32", (S, H, HEAD_DIM), F32)
    dv = torch.empty_like(v)
    dg = torch.empty((S, H, HEAD_DIM), dtype=F32, device=device)
    dbeta = torch.empty((S, H), dtype=F32, device=device)
    native.launch("kda_bwd_tail", dims, s.qn, s.kn, v, s.kg, s.g2, beta32, s.a, s.h, dh, s.v_new, dv_new, do, m1, m2,
                  dqg, dkr, dkg, hdh, dbeta_part, dq32, dk32, dv, dg, dbeta, s.status, device=device)
    dq, dk = torch.empty_like(v), torch.empty_like(v)
    native.launch("qk_grad_finish", dq32, s.q_raw, s.rstd_q, dq, S * H, device=device)
    native.launch("qk_grad_finish", dk32, s.k_raw, s.rstd_k, dk, S * H, device=device)
    return dq, dk, dv, dg, dbeta, dh0


class _ChunkKda(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, g, beta, cu_seqlens, scale, use_qk_l2norm, cu_seqlens_cpu=None):
        shape = q.shape
        q3, k3, v3, g3 = (_packed3(t, n).contiguous() for t, n in ((q, "q"), (k, "k"), (v, "v"), (g, "g")))
        beta3 = _packed_beta(beta)
        g3 = g3 if g3.dtype == F32 else g3.float()
        _check(q3, k3, v3, g3, beta3, cu_seqlens)
        beta32 = beta3.float().contiguous()
        with torch.cuda.device(q.device):
            o, saved, _ = _forward(q3, k3, v3, g3, beta32, cu_seqlens, scale, use_qk_l2norm,
                                   cu_seqlens_cpu=cu_seqlens_cpu)
        tape_module.keep(ctx, saved, v=v3, beta32=beta32)
        ctx.shapes = (shape, g.shape, beta.shape)
        ctx.dtypes = (g.dtype, beta.dtype)
        return o.view(shape)

    @staticmethod
    def backward(ctx, do):
        shape, g_shape, beta_shape = ctx.shapes
        do3 = _packed3(do, "dout").contiguous()
        if do3.dtype != BF16:
            do3 = do3.to(BF16)
        saved, kept = tape_module.restore(ctx)
        with torch.cuda.device(do.device):
            dq, dk, dv, dg, dbeta, _ = _backward(saved, kept["v"], kept["beta32"], do3)
        g_dtype, beta_dtype = ctx.dtypes
        return (dq.view(shape), dk.view(shape), dv.view(shape), dg.view(g_shape).to(g_dtype),
                dbeta.view(beta_shape).to(beta_dtype), None, None, None, None)


def _gate(g, use_gate_in_kernel, A_log, dt_bias, lower_bound):
    return _activate(g, A_log, dt_bias, lower_bound) if use_gate_in_kernel else g


def chunk_kda(q, k, v, g, beta, cu_seqlens, *, scale=None, use_gate_in_kernel=False, A_log=None, dt_bias=None,
              lower_bound=None, use_qk_l2norm_in_kernel=False, cu_seqlens_cpu=None):
    """Packed KDA chunked training as an autograd node: ``out`` BF16 like ``v``, with gradients to ``q, k, v, g, beta``
    and, with ``use_gate_in_kernel=True``, to ``A_log`` / ``dt_bias`` (reference: ops.py:142-165).
    ``cu_seqlens_cpu`` (not in the reference's signature; the GDN op's FLA signature has it): the same boundaries on
    the host, a tuple or a CPU tensor.  With them the chunk tables are built on the host without a device read, and
    the scan planner may cut the scans of a call with few long documents into parallel segments."""
    check_heads(int(v.shape[-2]))
    config.variant(OP)
    v, beta = seam(v, beta)
    gate = _gate(g, use_gate_in_kernel, A_log, dt_bias, lower_bound)
    if cu_seqlens_cpu is not None and isinstance(cu_seqlens_cpu, torch.Tensor):
        cu_seqlens_cpu = tuple(int(b) for b in cu_seqlens_cpu.tolist())
    return _ChunkKda.apply(q, k, v, gate, beta, cu_seqlens, DEFAULT_SCALE if scale is None else float(scale),
                           bool(use_qk_l2norm_in_kernel), None if cu_seqlens_cpu is None else tuple(cu_seqlens_cpu))


def chunk_kda_fwd(q, k, v, g, beta, cu_seqlens, *, scale=None, save_for_backward=True, use_gate_in_kernel=False,
                  A_log=None, dt_bias=None, lower_bound=None, use_qk_l2norm_in_kernel=False):
    """The forward alone: ``(out, saved)``; ``saved`` is what :func:`chunk_kda_bwd` takes (``None`` without
    ``save_for_backward``) (reference: ops.py:168-195)."""
    check_heads(int(v.shape[-2]))
    v, beta = seam(v, beta)
    with torch.no_grad():
        gate = _gate(g, use_gate_in_kernel, A_log, dt_bias, lower_bound)
        q3, k3, v3, g3 = (_packed3(t, n).contiguous() for t, n in ((q, "q"), (k, "k"), (v, "v"), (gate, "g")))
        beta3 = _packed_beta(beta)
        _check(q3, k3, v3, g3, beta3, cu_seqlens)
        with torch.cuda.device(q.device):
            o, saved, _ = _forward(q3, k3, v3, g3.float(), beta3.float().contiguous(), cu_seqlens,
                                   DEFAULT_SCALE if scale is None else float(scale), bool(use_qk_l2norm_in_kernel))
    return o.view(q.shape), (saved if save_for_backward else None)


def chunk_kda_bwd(q, k, v, g, beta, cu_seqlens, dout, *, saved=None, scale=None, use_gate_in_kernel=False, A_log=None,
                  dt_bias=None, lower_bound=None, use_qk_l2norm_in_kernel=False):
    """The backward alone, from the forward's operands and modes: ``(dq, dk, dv, dbeta, dg)`` and, with
    ``use_gate_in_kernel=True``, ``(dq, dk, dv, dbeta, dg, dA_log, ddt_bias)``; ``dbeta`` in ``beta``'s dtype.
    ``saved=None`` replays the forward first (the same kernels: the same bits) (reference: ops.py:198-234)."""
    check_heads(int(v.shape[-2]))
    beta_dtype = beta.dtype
    v, beta = seam(v, beta)
    if saved is None:
        _, saved = chunk_kda_fwd(q, k, v, g, beta, cu_seqlens, scale=scale, use_gate_in_kernel=use_gate_in_kernel,
                                 A_log=A_log, dt_bias=dt_bias, lower_bound=lower_bound,
                                 use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel)
    v3 = _packed3(v, "v").contiguous()
    beta3 = _packed_beta(beta)
    do3 = _packed3(dout, "dout").contiguous().to(BF16)
    with torch.no_grad(), torch.cuda.device(v.device):
        dq, dk, dv, dg, dbeta, _ = _backward(saved, v3, beta3.float().contiguous(), do3)
    grads = [dq.view(q.shape), dk.view(q.shape), dv.view(v.shape), dbeta.view(beta.shape).to(beta_dtype),
             dg.view(g.shape)]
    if use_gate_in_kernel:
        raw = g.detach().requires_grad_(True)
        a_leaf, b_leaf = A_log.detach().requires_grad_(True), dt_bias.detach().requires_grad_(True)
        gate = _activate(raw, a_leaf, b_leaf, lower_bound)
        draw, da, db = torch.autograd.grad(gate, [raw, a_leaf, b_leaf], dg.view(gate.shape))
        grads[4] = draw
        grads += [da, db]
    return tuple(grads)


def prebuild(*, device: Any = None, max_workers: int | None = None, num_heads: int) -> list[Path]:
    """Build (or find) the native library for ``device``; ``num_heads`` is checked first (1 to 64, ``ValueError``)."""
    check_heads(num_heads)
    arch = loader.device_arch(device)
    loader.check_toolkit(arch, "the KDA kernels")
    return loader.prebuild_libraries(registry.op_spec(OP).packages, arch, max_workers=max_workers)


def release() -> None:
    """Nothing is kept between calls besides the workspace pool (emptied by the runtime) and the library handle."""
    native.release()
