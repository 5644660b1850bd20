"""The launch plan of the two state scans (reference: ``choose_scan_plan`` / ``scan_plans`` / ``finalize_stage``,
miles_ext_kernels/cake/_impl/gdn/ops.py:405-531, 733-860).

A scan is one chain of dependent chunk steps per (sequence, value head).  With fewer chains than SMs and long
sequences the serial walk leaves most of the GPU idle, so the planner may cut every long sequence into segments of
whole chunks and run three launches instead of one: a pre-scan (each segment's affine summary ``S_out = M S_in + B``,
all segments in parallel), a stitch (the summaries chained per sequence) and the real walk (all segments in parallel
from their true start states).  When a segment's closing gates are strong enough (below ``WARM_NATS`` nats over its
last ``WARM_CHUNKS`` chunks) the kernels shorten the pre-scan to those chunks and take ``M`` as zero.

The plan is a pure function of the layout, the head count and the SM count: the same call always takes the same plan
and gives the same bits.  A segmented scan is not bit-identical to the serial one (the state crosses a segment
boundary as ``M S + B`` in fp32 instead of through the chunk steps); both are inside the accuracy budgets.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from functools import lru_cache

import torch

from . import native
from .meta import device_index, upload

MIN_SEGMENT_CHUNKS = 16  # a segment shorter than this does not pay for its summary
MAX_PARTS = 16
WARM_CHUNKS = 2
WARM_NATS = -10.0
MIN_GAIN = 0.95  # take a segmented plan only when its modelled time is below this fraction of the serial walk's
STITCH_STEPS = 3  # modelled cost of one stitch step, in chunk steps


@dataclass(frozen=True)
class Segmentation:
    """The segments of a layout for ``parts`` segments per long sequence (host lists)."""

    parts: int
    seg_chunk_start: tuple[int, ...]  # [segments + 1]
    seq_seg_start: tuple[int, ...]  # [N + 1]

    @property
    def segments(self) -> int:
        return len(self.seg_chunk_start) - 1


def segment(seq_chunk_start: tuple[int, ...], parts: int) -> Segmentation:
    """Cut every sequence into at most ``parts`` segments of at least :data:`MIN_SEGMENT_CHUNKS` chunks, as equal
    as whole chunks allow."""
    starts, first = [], [0]
    for begin, end in zip(seq_chunk_start, seq_chunk_start[1:]):
        chunks = end - begin
        pieces = max(1, min(parts, chunks // MIN_SEGMENT_CHUNKS))
        for p in range(pieces):
            starts.append(begin + (chunks * p) // pieces)
        first.append(len(starts))
    starts.append(seq_chunk_start[-1])
    return Segmentation(parts, tuple(starts), tuple(first))


def _waves(ctas: int, sms: int) -> int:
    return -(-ctas // sms)


def modelled_steps(seg: Segmentation, num_v_heads: int, sms: int) -> float:
    """Chunk steps on the critical path of the three launches, every summary exact (no warm-up)."""
    longest = max((b - a for a, b in zip(seg.seg_chunk_start, seg.seg_chunk_start[1:])), default=0)
    per_seq = [b - a for a, b in zip(seg.seq_seg_start, seg.seq_seg_start[1:])]
    offset = sum(max(p - 1, 0) for p in per_seq)
    transfer = sum(max(p - 2, 0) for p in per_seq)
    pre = longest * _waves((offset + transfer) * num_v_heads, sms) if offset else 0
    real = longest * _waves(seg.segments * num_v_heads, sms)
    return pre + real + STITCH_STEPS * max(per_seq, default=0)


@lru_cache(maxsize=256)
def choose_parts(seq_chunk_start: tuple[int, ...], num_v_heads: int, sms: int, forced: int = 0) -> int:
    """How many segments per long sequence: 1 = the serial walk.  ``forced`` > 0 overrides the model."""
    if forced > 0:
        return min(forced, MAX_PARTS)
    num_seqs = len(seq_chunk_start) - 1
    if num_seqs <= 0 or num_seqs * num_v_heads * 2 > sms:
        return 1
    serial = modelled_steps(segment(seq_chunk_start, 1), num_v_heads, sms)
    best, best_steps = 1, serial
    for parts in range(2, MAX_PARTS + 1):
        seg = segment(seq_chunk_start, parts)
        if seg.segments == num_seqs:
            break  # no sequence is long enough to cut
        steps = modelled_steps(seg, num_v_heads, sms)
        if steps < best_steps:
            best, best_steps = parts, steps
    return best if best_steps < MIN_GAIN * serial else 1


@dataclass
class ScanPlan:
    """Device tables of a segmented scan."""

    segments: int
    num_seqs: int
    seg_chunk_start: torch.Tensor  # int32 [segments + 1]
    seq_seg_start: torch.Tensor  # int32 [N + 1]
    flags_fwd: torch.Tensor  # int32 [segments]: bit 0 not the sequence's first, bit 1 its last
    flags_bwd: torch.Tensor  # int32 [segments]: bit 0 not the sequence's last, bit 1 its first
    state_row: torch.Tensor  # int32 [segments]: the sequence of each segment
    first_index: torch.Tensor  # int64 [N]: each sequence's first segment
    last_index: torch.Tensor  # int64 [N]: each sequence's last segment
    # the same flags with the first segment of a cut sequence taken from zero / the identity like the others (its
    # summary is chained from the boundary state by the stitch): under the warm-up rule no segment is then walked in
    # full before the real walk
    flags_fwd_all: torch.Tensor | None = None
    flags_bwd_all: torch.Tensor | None = None
    warm_chunks: int = WARM_CHUNKS
    warm_log2: float = WARM_NATS * math.log2(math.e)
    guards: tuple = ()  # UploadGuards of the cached tables


_PLANS: dict[tuple, ScanPlan] = {}


def device_plan(seg: Segmentation, device: torch.device) -> ScanPlan:
    key = (seg, device.type, device_index(device))
    found = _PLANS.get(key)
    if found is not None:
        for guard in found.guards:
            guard.wait()
        return found
    first, last, rows, fwd, bwd, fwd_all, bwd_all = [], [], [], [], [], [], []
    for n, (a, b) in enumerate(zip(seg.seq_seg_start, seg.seq_seg_start[1:])):
        first.append(a)
        last.append(b - 1)
        cut = 1 if b - a > 1 else 0
        for s in range(a, b):
            rows.append(n)
            fwd.append((1 if s > a else 0) | (2 if s == b - 1 else 0))
            bwd.append((1 if s < b - 1 else 0) | (2 if s == a else 0))
            fwd_all.append(cut | (2 if s == b - 1 else 0))
            bwd_all.append(cut | (2 if s == a else 0))
    flat, guard_a = upload(torch.tensor([*seg.seg_chunk_start, *seg.seq_seg_start, *fwd, *bwd, *rows, *fwd_all, *bwd_all],
                                        dtype=torch.int32), device)
    index, guard_b = upload(torch.tensor([*first, *last], dtype=torch.int64), device)
    ns, n = seg.segments, len(seg.seq_seg_start) - 1
    at = [0, ns + 1, ns + n + 2, 2 * ns + n + 2, 3 * ns + n + 2, 4 * ns + n + 2, 5 * ns + n + 2, 6 * ns + n + 2]
    plan = ScanPlan(ns, n, flat[at[0]:at[1]], flat[at[1]:at[2]], flat[at[2]:at[3]], flat[at[3]:at[4]],
                    flat[at[4]:at[5]], index[:n], index[n:],
                    guards=tuple(g for g in (guard_a, guard_b) if g is not None),
                    flags_fwd_all=flat[at[5]:at[6]], flags_bwd_all=flat[at[6]:at[7]])
    if len(_PLANS) >= 64:
        _PLANS.clear()
    _PLANS[key] = plan
    return plan


@lru_cache(maxsize=8)
def sm_count(index: int) -> int:
    return int(torch.cuda.get_device_properties(index).multi_processor_count)


def plan_for(meta, num_v_heads: int, device: torch.device, forced: int = 0) -> ScanPlan | None:
    """The segmented plan of a layout, or ``None`` for the serial walk (also for layouts whose tables were built on
    the device: the planner needs the chunk counts on the host)."""
    if meta.host_seq_chunk_start is None or device.type != "cuda":
        return None
    parts = choose_parts(meta.host_seq_chunk_start, num_v_heads, sm_count(device_index(device) or 0), forced)
    if parts <= 1:
        return None
    seg = segment(meta.host_seq_chunk_start, parts)
    if seg.segments == meta.num_seqs:
        return None
    return device_plan(seg, device)


def segment_dims(dims: native.Dims, plan: ScanPlan) -> native.Dims:
    """The call's extents with the segments in place of the sequences."""
    return native.Dims(dims.total_tokens, dims.num_qk_heads, dims.num_v_heads, dims.head_dim, plan.segments,
                       dims.num_chunks, dims.scale, dims.chunk_start, dims.chunk_len, dims.chunk_seq,
                       plan.seg_chunk_start.data_ptr(), dims.qk_pitch, dims.v_pitch, dims.raw_pitch, dims.dqk_pitch,
                       dims.dv_pitch, None)  # the operands' pitches stay; the segments are taken as numbered


# --------------------------------------------------------------------------------------------------------------------
# summaries of one fragment and folds over ranks (context parallelism with ranks working in parallel)
# --------------------------------------------------------------------------------------------------------------------
def fragment_plan(chunk_begin: int, chunk_end: int, num_v_heads: int, device: torch.device) -> ScanPlan:
    """Segments of the chunk range of one document fragment, every segment walked from zero / the identity and none
    skipped: what a rank's summary ``(B, M)`` of the fragment is composed from."""
    chunks = chunk_end - chunk_begin
    sms = sm_count(device_index(device) or 0)
    parts = max(1, min(MAX_PARTS, chunks // MIN_SEGMENT_CHUNKS, sms // max(1, num_v_heads)))
    seg = Segmentation(-parts, tuple(chunk_begin + (chunks * p) // parts for p in range(parts)) + (chunk_end,),
                       (0, parts))
    key = (seg, device.type, device_index(device))
    found = _PLANS.get(key)
    if found is not None:
        for guard in found.guards:
            guard.wait()
        return found
    ns = parts
    flat, guard = upload(torch.tensor([*seg.seg_chunk_start, 0, ns, *([1] * ns), *([0] * ns)], dtype=torch.int32),
                         device)
    plan = ScanPlan(ns, 1, flat[: ns + 1], flat[ns + 1 : ns + 3], flat[ns + 3 : 2 * ns + 3], flat[ns + 3 : 2 * ns + 3],
                    flat[2 * ns + 3 :], None, None, guards=() if guard is None else (guard,))
    if len(_PLANS) >= 64:
        _PLANS.clear()
    _PLANS[key] = plan
    return plan


def compose_summary(seg_dims: native.Dims, plan: ScanPlan, summary: torch.Tensor, g_cs: torch.Tensor, reverse: bool,
                    out: torch.Tensor | None = None):
    """``[HV, 2, 128, 128]``: the (B, M) of the whole run of segments, from the segments' summaries (B: from zero with
    the offsets; M: from the identity without them), one launch, written into ``out`` when given."""
    device = summary.device
    HV = summary.shape[1]
    if out is None:
        out = torch.empty((HV, 2, 128, 128), dtype=torch.float32, device=device)
    native.launch("gdn_scan_compose", seg_dims, plan.seq_seg_start, summary, g_cs, out, int(reverse), plan.warm_chunks,
                  plan.warm_log2, device=device)
    return out


def fold_ranks(dims: native.Dims, gathered: torch.Tensor, first: int, last: int, reverse: bool,
               out: torch.Tensor | None = None) -> torch.Tensor:
    """The state that the ranks ``first .. last`` (inclusive) hand on, from their gathered summaries
    ``[W, HV, 2, 128, 128]``: ``S = B_first``, then ``S = M_r S + B_r`` along the chain (``reverse``: from ``last``
    down to ``first``).  ``[1, HV, 128, 128]``."""
    device = gathered.device
    HV = gathered.shape[1]
    span = _small_table((first, last + 1), torch.int32, device)
    if out is None:
        out = torch.empty((1, HV, 128, 128), dtype=torch.float32, device=device)
    native.launch("gdn_scan_stitch", dims, 1, span, gathered, None, None, None, out, int(reverse), 0, 0.0, 0,
                  device=device)
    return out


_TABLES: dict[tuple, tuple] = {}


def _small_table(values: tuple[int, ...], dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    """A few integers on the device, uploaded once per distinct content and kept: a call neither allocates pinned
    memory nor copies from a temporary (so it can be captured in a CUDA graph and replayed)."""
    key = (values, dtype, device.type, device_index(device))
    found = _TABLES.get(key)
    if found is not None:
        if found[1] is not None:
            found[1].wait()
        return found[0]
    if len(_TABLES) >= 256:
        _TABLES.clear()
    table, guard = upload(torch.tensor(values, dtype=dtype), device)
    _TABLES[key] = (table, guard)
    return table


def release() -> None:
    _PLANS.clear()
    _TABLES.clear()
    choose_parts.cache_clear()
