"""The stages of the GDN forward and backward as launches of the native library, on packed ``[T, heads, 128]``
operands.  No stage synchronises; all run on torch's current stream.

Forward (reference launch order: miles_ext_kernels/cake/_impl/gdn/ops.py:1320-1450): prep -> wy -> fwd_ho (the state
scan with the output fused in; the separate fwd_o launch remains in the library).
Backward (reference: ops.py:1474-1735): bwd_dh (adjoint scan with dv_local fused) -> bwd_tail (dq, dk, dv, dbeta, dg
with the group sum, the norm's pull-back and the in-chunk gate suffix sum fused).

Scratch that does not outlive a call comes from the runtime's workspace pool; tensors that the autograd tape or the
caller keeps are fresh allocations.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..._runtime import workspace
from . import native, scan
from .meta import ChunkMeta

OP = "gdn"
HEAD_DIM = 128
BF16, F32 = torch.bfloat16, torch.float32

__all__ = ["ForwardTape", "dims_of", "forward", "backward", "check_status"]


def pitch_of(x: torch.Tensor | None) -> int:
    """The token stride (elements) a kernel is told for ``x [T, heads, 128]``: 0 when dense, else ``x.stride(0)`` (x
    is then a column slice of a wider packed row; its heads are contiguous inside a token)."""
    if x is None or x.is_contiguous():
        return 0
    if x.stride(2) != 1 or x.stride(1) != HEAD_DIM or x.stride(0) % 8 or x.data_ptr() % 16:
        raise ValueError(f"a strided operand must keep its heads contiguous inside a token; strides {x.stride()}")
    return int(x.stride(0))


def dims_of(meta: ChunkMeta, num_qk_heads: int, num_v_heads: int, scale: float, *, qk_pitch: int = 0,
            v_pitch: int = 0, raw_pitch: int = 0, dqk_pitch: int = 0, dv_pitch: int = 0) -> native.Dims:
    return native.Dims(
        meta.total_tokens, num_qk_heads, num_v_heads, HEAD_DIM, meta.num_seqs, meta.num_chunks, float(scale),
        meta.chunk_start.data_ptr(), meta.chunk_len.data_ptr(), meta.chunk_seq.data_ptr(),
        meta.seq_chunk_start.data_ptr(), qk_pitch, v_pitch, raw_pitch, dqk_pitch, dv_pitch,
        None if meta.seq_order is None else meta.seq_order.data_ptr(),
    )


@dataclass
class ForwardTape:
    """What the forward leaves for the backward (packed layouts)."""

    qn: torch.Tensor  # [T, H, 128] bf16, normalised when the op normalises
    kn: torch.Tensor
    v: torch.Tensor  # [T, HV, 128]
    beta32: torch.Tensor  # [T, HV] fp32
    g_cs: torch.Tensor  # [T, HV] fp32, log2 domain
    a: torch.Tensor  # [NC, HV, 64, 64] bf16
    aqk: torch.Tensor
    w: torch.Tensor | None  # [T, HV, 128] bf16
    u: torch.Tensor | None
    h: torch.Tensor | None  # [NC, HV, 128, 128] bf16
    v_new: torch.Tensor | None
    q_raw: torch.Tensor | None  # raw rows and their rstd when the op normalised
    k_raw: torch.Tensor | None
    rstd_q: torch.Tensor | None
    rstd_k: torch.Tensor | None
    status: torch.Tensor  # int32 [1]: nonzero when a bounded wait in a kernel ran out


def check_status(status: torch.Tensor) -> None:
    """Raise when a kernel recorded an error.  Synchronises: for tests and debugging, never on the hot path."""
    word = int(status.item())
    if word:
        raise RuntimeError(f"a GDN kernel gave up a bounded wait (code {word & 0xFF}, stage {word >> 8})")


def _l2norm(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """x ``[T, heads, 128]``, dense or a column slice of a packed row -> dense normalised rows and their rstd."""
    y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    rstd = torch.empty(x.shape[:-1], dtype=F32, device=x.device)
    native.launch("gdn_l2norm", x, y, rstd, x.numel() // HEAD_DIM, x.shape[1], pitch_of(x), device=x.device)
    return y, rstd


def _walk_forward(dims, k, w, u, g_cs, h0, h, v_new, final, status, output) -> None:
    """One launch of the state scan over ``dims``' sequences; with ``output = (q, aqk, o)`` the walk writes the op's
    output too."""
    if output is None:
        native.launch("gdn_fwd_h", dims, k, w, u, g_cs, h0, h, v_new, final, status, device=k.device)
    else:
        q, aqk, o = output
        native.launch("gdn_fwd_ho", dims, q, k, w, u, aqk, g_cs, h0, h, v_new, o, final, status, device=k.device)


def _scan_forward(dims, meta: ChunkMeta, k, w, u, g_cs, h0, h, v_new, want_final: bool, status, scan_segments: int,
                  output=None, prepared=None):
    """The state scan: one serial walk per (sequence, value head), or the planner's segmented form (pre-scan,
    stitch, real walk over the segments).  ``prepared``: a context-parallel exchange's ``(plan, seg_dims, summary)``
    with every segment of this rank's slice already summarised from zero and from the identity -- the pre-scan is
    skipped and the stitch chains all of them from ``h0``.  Returns the final state or None."""
    device = k.device
    HV = w.shape[1]
    if prepared is not None:
        plan, seg_dims, summary = prepared
        seg_state = workspace.take(OP, "scan_state", (plan.segments, HV, HEAD_DIM, HEAD_DIM), F32, device)
        native.launch("gdn_scan_stitch", seg_dims, plan.num_seqs, plan.seq_seg_start, summary, h0, g_cs, seg_state, None,
                      0, plan.warm_chunks, plan.warm_log2, 4, device=device)
        seg_final = None
        if want_final:
            seg_final = workspace.take(OP, "scan_final", (plan.segments, HV, HEAD_DIM, HEAD_DIM), F32, device)
        _walk_forward(seg_dims, k, w, u, g_cs, seg_state, h, v_new, seg_final, status, output)
        return seg_final.index_select(0, plan.last_index) if want_final else None
    plan = scan.plan_for(meta, HV, device, scan_segments)
    if plan is None:
        final = torch.empty((meta.num_seqs, HV, HEAD_DIM, HEAD_DIM), dtype=F32, device=device) if want_final else None
        _walk_forward(dims, k, w, u, g_cs, h0, h, v_new, final, status, output)
        return final
    seg_dims = scan.segment_dims(dims, plan)
    summary = workspace.take(OP, "scan_summary", (plan.segments, HV, 2, HEAD_DIM, HEAD_DIM), F32, device)
    seg_state = workspace.take(OP, "scan_state", (plan.segments, HV, HEAD_DIM, HEAD_DIM), F32, device)
    # every segment of a cut sequence is summarised from zero / the identity, the first too, and the stitch chains
    # them from h0: where the warm-up rule applies no segment is walked in full before the real walk
    native.launch("gdn_fwd_h_prescan", seg_dims, k, w, u, g_cs, None, plan.flags_fwd_all, plan.state_row,
                  plan.warm_chunks, plan.warm_log2, summary, status, device=device)
    native.launch("gdn_scan_stitch", seg_dims, plan.num_seqs, plan.seq_seg_start, summary, h0, g_cs, seg_state, None, 0,
                  plan.warm_chunks, plan.warm_log2, 4, device=device)
    seg_final = None
    if want_final:
        seg_final = workspace.take(OP, "scan_final", (plan.segments, HV, HEAD_DIM, HEAD_DIM), F32, device)
    _walk_forward(seg_dims, k, w, u, g_cs, seg_state, h, v_new, seg_final, status, output)
    return seg_final.index_select(0, plan.last_index) if want_final else None


def _scan_backward(dims, meta: ChunkMeta, tape, do, dht, dh_tape, dv_new, want_dh0: bool, scan_segments: int,
                   prepared=None):
    """The adjoint scan, serial or segmented like the forward's (``prepared``: as there).  Returns dh0 or None."""
    device = do.device
    HV = tape.v.shape[1]
    if prepared is not None:
        plan, seg_dims, summary = prepared
        seg_state = workspace.take(OP, "scan_state", (plan.segments, HV, HEAD_DIM, HEAD_DIM), F32, device)
        native.launch("gdn_scan_stitch", seg_dims, plan.num_seqs, plan.seq_seg_start, summary, dht, tape.g_cs, seg_state,
                      None, 1, plan.warm_chunks, plan.warm_log2, 4, device=device)
        seg_dh0 = None
        if want_dh0:
            seg_dh0 = workspace.take(OP, "scan_final", (plan.segments, HV, HEAD_DIM, HEAD_DIM), F32, device)
        native.launch("gdn_bwd_dh", seg_dims, tape.qn, tape.kn, tape.w, do, tape.aqk, tape.g_cs, seg_state, dh_tape,
                      dv_new, seg_dh0, tape.status, device=device)
        return seg_dh0.index_select(0, plan.first_index) if want_dh0 else None
    plan = scan.plan_for(meta, HV, device, scan_segments)
    if plan is None:
        dh0 = torch.empty((meta.num_seqs, HV, HEAD_DIM, HEAD_DIM), dtype=F32, device=device) if want_dh0 else None
        native.launch("gdn_bwd_dh", dims, tape.qn, tape.kn, tape.w, do, tape.aqk, tape.g_cs, dht, dh_tape, dv_new, dh0,
                      tape.status, device=device)
        return dh0
    seg_dims = scan.segment_dims(dims, plan)
    summary = workspace.take(OP, "scan_summary", (plan.segments, HV, 2, HEAD_DIM, HEAD_DIM), F32, device)
    seg_state = workspace.take(OP, "scan_state", (plan.segments, HV, HEAD_DIM, HEAD_DIM), F32, device)
    native.launch("gdn_bwd_dh_prescan", seg_dims, tape.qn, tape.kn, tape.w, do, tape.aqk, tape.g_cs, None,
                  plan.flags_bwd_all, plan.state_row, plan.warm_chunks, plan.warm_log2, summary, tape.status,
                  device=device)
    native.launch("gdn_scan_stitch", seg_dims, plan.num_seqs, plan.seq_seg_start, summary, dht, tape.g_cs, seg_state,
                  None, 1, plan.warm_chunks, plan.warm_log2, 4, device=device)
    seg_dh0 = None
    if want_dh0:
        seg_dh0 = workspace.take(OP, "scan_final", (plan.segments, HV, HEAD_DIM, HEAD_DIM), F32, device)
    native.launch("gdn_bwd_dh", seg_dims, tape.qn, tape.kn, tape.w, do, tape.aqk, tape.g_cs, seg_state, dh_tape, dv_new,
                  seg_dh0, tape.status, device=device)
    return seg_dh0.index_select(0, plan.first_index) if want_dh0 else None


def forward(q, k, v, g, beta32, meta: ChunkMeta, scale: float, h0, output_final_state: bool, use_qk_l2norm: bool,
            keep_state: bool = True, scan_segments: int = 0, exchange=None):
    """q, k ``[T, H, 128]`` bf16; v ``[T, HV, 128]`` bf16; g, beta32 ``[T, HV]`` fp32; h0 ``[N, HV, 128, 128]`` fp32
    or None.  ``scan_segments``: 0 lets the scan planner decide, 1 forces the serial walk, more forces that many
    segments per long sequence.  ``exchange`` (context parallelism) supplies the state that enters this rank's first
    fragment and takes the one that leaves its last.  Returns ``(o [T, HV, 128] bf16, final_state or None, tape,
    h0 used)``."""
    device = q.device
    T, H = q.shape[0], q.shape[1]
    HV = v.shape[1]
    NC = meta.num_chunks
    status = torch.zeros(1, dtype=torch.int32, device=device)

    q_raw = k_raw = rstd_q = rstd_k = None
    if use_qk_l2norm:
        q_raw, k_raw = q, k
        q, rstd_q = _l2norm(q)
        k, rstd_k = _l2norm(k)
    # q, k, v may be column slices of one packed row (dense heads inside a token): the kernels read them in place
    dims = dims_of(meta, H, HV, scale, qk_pitch=pitch_of(q), v_pitch=pitch_of(v))
    g_cs = torch.empty_like(g)
    native.launch("gdn_gate_cumsum", dims, g, g_cs, device=device)

    # pad chunks of the device route are never written: their A / Aqk / h rows must not hold NaN bit patterns
    alloc = torch.empty if meta.exact else torch.zeros
    a = alloc((NC, HV, 64, 64), dtype=BF16, device=device)
    aqk = alloc((NC, HV, 64, 64), dtype=BF16, device=device)
    w = torch.empty((T, HV, HEAD_DIM), dtype=BF16, device=device)
    u = torch.empty((T, HV, HEAD_DIM), dtype=BF16, device=device)
    native.launch("gdn_wy_fwd", dims, q, k, v, beta32, g_cs, a, aqk, w, u, status, device=device)

    h = alloc((NC, HV, HEAD_DIM, HEAD_DIM), dtype=BF16, device=device)
    v_new = torch.empty((T, HV, HEAD_DIM), dtype=BF16, device=device)
    prepared = None
    if exchange is not None:
        h0, output_final_state = exchange.forward_begin(dims, meta, k, w, u, g_cs, status, scan_segments)
        prepared = exchange.take_prepared()
    # the output is written by the walk itself (h_tape and v_new are consumed from shared memory, not read back)
    o = torch.empty((T, HV, HEAD_DIM), dtype=BF16, device=device)
    final_state = _scan_forward(dims, meta, k, w, u, g_cs, h0, h, v_new, output_final_state, status, scan_segments,
                                output=(q, aqk, o), prepared=prepared)
    if exchange is not None:
        exchange.forward_end(final_state)
        final_state = None

    if not keep_state:
        w = u = h = v_new = None
    tape = ForwardTape(q, k, v, beta32, g_cs, a, aqk, w, u, h, v_new, q_raw, k_raw, rstd_q, rstd_k, status)
    return o, final_state, tape, h0


def recompute_state(tape: ForwardTape, meta: ChunkMeta, scale: float, h0, scan_segments: int = 0) -> None:
    """Rebuild ``w, u, h, v_new`` of a tape that dropped them (the same kernels on the same inputs: the same bits)."""
    device = tape.qn.device
    T, H = tape.qn.shape[0], tape.qn.shape[1]
    HV = tape.v.shape[1]
    NC = meta.num_chunks
    dims = dims_of(meta, H, HV, scale, qk_pitch=pitch_of(tape.qn), v_pitch=pitch_of(tape.v))
    alloc = torch.empty if meta.exact else torch.zeros
    a = workspace.take(OP, "recompute_a", (NC, HV, 64, 64), BF16, device)
    aqk = workspace.take(OP, "recompute_aqk", (NC, HV, 64, 64), BF16, device)
    tape.w = torch.empty((T, HV, HEAD_DIM), dtype=BF16, device=device)
    tape.u = torch.empty((T, HV, HEAD_DIM), dtype=BF16, device=device)
    native.launch("gdn_wy_fwd", dims, tape.qn, tape.kn, tape.v, tape.beta32, tape.g_cs, a, aqk, tape.w, tape.u,
                  tape.status, device=device)
    tape.h = alloc((NC, HV, HEAD_DIM, HEAD_DIM), dtype=BF16, device=device)
    tape.v_new = torch.empty((T, HV, HEAD_DIM), dtype=BF16, device=device)
    _scan_forward(dims, meta, tape.kn, tape.w, tape.u, tape.g_cs, h0, tape.h, tape.v_new, False, tape.status,
                  scan_segments)


def backward(tape: ForwardTape, meta: ChunkMeta, scale: float, do, dht, h0, want_dh0: bool, scan_segments: int = 0,
             exchange=None, packed_grads: bool = False, inspect: dict | None = None):
    """``do [T, HV, 128]`` bf16, ``dht [N, HV, 128, 128]`` fp32 or None.  Returns ``(dq, dk [T, H, 128] bf16, dv
    [T, HV, 128] bf16, dg, dbeta [T, HV] fp32, dh0 [N, HV, 128, 128] fp32 or None)``.  With ``packed_grads`` dq, dk
    and dv are the column slices ``[q heads | k heads | v heads]`` of one ``[T, (2 H + HV) * 128]`` row.

    The adjoint scan's tapes (``dh_tape``, ``dv_new``) are pooled scratch, which never leaves this function; a stage
    test that wants to look at them passes a dict as ``inspect`` and finds them there as fresh allocations."""
    device = do.device
    T, H = tape.qn.shape[0], tape.qn.shape[1]
    HV = tape.v.shape[1]
    NC = meta.num_chunks
    if packed_grads:
        row = torch.empty((T, (2 * H + HV) * HEAD_DIM), dtype=BF16, device=device)
        dq = row[:, : H * HEAD_DIM].view(T, H, HEAD_DIM)
        dk = row[:, H * HEAD_DIM : 2 * H * HEAD_DIM].view(T, H, HEAD_DIM)
        dv = row[:, 2 * H * HEAD_DIM :].view(T, HV, HEAD_DIM)
    else:
        dq = torch.empty((T, H, HEAD_DIM), dtype=BF16, device=device)
        dk = torch.empty((T, H, HEAD_DIM), dtype=BF16, device=device)
        dv = torch.empty((T, HV, HEAD_DIM), dtype=BF16, device=device)
    raw_pitch = pitch_of(tape.q_raw)
    if tape.k_raw is not None and pitch_of(tape.k_raw) != raw_pitch:
        raise ValueError("q and k must share their token stride")
    dims = dims_of(meta, H, HV, scale, qk_pitch=pitch_of(tape.qn), v_pitch=pitch_of(tape.v), raw_pitch=raw_pitch,
                   dqk_pitch=pitch_of(dq), dv_pitch=pitch_of(dv))
    if tape.w is None:
        recompute_state(tape, meta, scale, h0, scan_segments)
    if inspect is not None:
        dh_tape = torch.zeros((NC, HV, HEAD_DIM, HEAD_DIM), dtype=BF16, device=device)
        dv_new = torch.empty((T, HV, HEAD_DIM), dtype=BF16, device=device)
        inspect.update(dh_tape=dh_tape, dv_new=dv_new)
    else:
        if meta.exact:
            dh_tape = workspace.take(OP, "dh_tape", (NC, HV, HEAD_DIM, HEAD_DIM), BF16, device)
        else:  # pad chunks are never written
            dh_tape = torch.zeros((NC, HV, HEAD_DIM, HEAD_DIM), dtype=BF16, device=device)
        dv_new = workspace.take(OP, "dv_new", (T, HV, HEAD_DIM), BF16, device)
    prepared = None
    if exchange is not None:
        dht, want_dh0 = exchange.backward_begin(dims, meta, tape, do, scan_segments)
        prepared = exchange.take_prepared()
    dh0 = _scan_backward(dims, meta, tape, do, dht, dh_tape, dv_new, want_dh0, scan_segments, prepared=prepared)
    if exchange is not None:
        exchange.backward_end(dh0)
        dh0 = None
    dbeta = torch.empty((T, HV), dtype=F32, device=device)
    dg = torch.empty((T, HV), dtype=F32, device=device)
    native.launch("gdn_bwd_tail", dims, tape.qn, tape.kn, tape.v, tape.beta32, tape.g_cs, tape.a, tape.aqk, tape.w, tape.u,
                  tape.h, dh_tape, tape.v_new, dv_new, do, tape.q_raw, tape.k_raw, tape.rstd_q, tape.rstd_k, dq, dk, dv,
                  dbeta, dg, tape.status, device=device)
    return dq, dk, dv, dg, dbeta, dh0
