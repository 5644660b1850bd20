"""Context parallelism of the GDN op: one packed batch split over the ranks of a process group (contiguous slices, or
the load-balanced zigzag layouts, or an explicit table of fragments); the chunk state crosses the cuts.

:class:`KcpContext` is one rank's view of the partition (reference: miles_ext_kernels/cake/_impl/gdn/kcp.py:71-169):
``rank``, ``world_size``, ``num_tokens`` (this rank's), ``cu_seqlens`` / ``cu_seqlens_cpu`` (local boundaries: one
sequence per document fragment), ``layout``, ``group`` and ``fla_compatible``.  :func:`build_kcp_context` builds and
caches it (reference: kcp.py:185-226).

Contract under a context (FLA's): no ``initial_state``, no final state; tokens never move, only ``[HV, 128, 128]``
fp32 states.  Forward: the state at the end of this rank's last fragment goes to the next rank when the document
continues there; backward: the adjoint state at the start of this rank's first fragment goes to the previous rank.
Two exchanges serve that: the sequential hand-over (point to point along the rank chain: rank r waits for rank
r - 1) and the parallel one (every rank summarises its boundary fragment as an affine map, one all-gather, a local
fold: ranks do not wait for one another; ``--cake-gdn-kcp-exchange``).  Either way the states land in this GPU's own
memory before any kernel reads them (NCCL over NVLink between GPUs; gloo in the CPU tests).

Layouts (``layout.py``): ``contiguous``, ``zigzag``, ``zigzag_per_document`` and explicit fragment tables.  The
sequential hand-over follows the rank chain and serves the contiguous layout only; the parallel exchange serves every
layout: each rank publishes the summaries of its fragments whose documents go on, and folds, per fragment, the chain
of the fragments before it in its document.
"""

from __future__ import annotations

import dataclasses
from collections import OrderedDict
from collections.abc import Sequence
from typing import Any

import torch

from . import layout as layout_module

LAYOUTS = layout_module.KCP_LAYOUTS
_CACHE_LIMIT = 32
_CONTEXTS: OrderedDict[tuple[Any, ...], KcpContext] = OrderedDict()

__all__ = ["ExchangeLog", "KcpContext", "build_kcp_context", "document_run", "halo_rows", "local_partition", "release",
           "set_exchange_log"]


class ExchangeLog:
    """Brackets every boundary-state exchange (pre-scan, gather, fold; or the point-to-point hand-over) with CUDA
    events on the launching stream and counts the bytes a rank receives.  ``bench.py`` reads the exchange's own device
    time from it; ordinary calls never time."""

    def __init__(self) -> None:
        self.events: list[tuple[str, Any, Any]] = []
        self.bytes_received = 0

    def milliseconds(self) -> dict[str, float]:
        """Total device time per direction (call after synchronising)."""
        total: dict[str, float] = {}
        for name, start, end in self.events:
            total[name] = total.get(name, 0.0) + start.elapsed_time(end)
        return total


_exchange_log: ExchangeLog | None = None


def set_exchange_log(log: ExchangeLog | None) -> None:
    global _exchange_log
    _exchange_log = log


class _Timed:
    """``with _Timed("forward"):`` records the bracket in the active :class:`ExchangeLog`, if any."""

    def __init__(self, name: str) -> None:
        self.name, self.log = name, _exchange_log

    def __enter__(self):
        if self.log is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()
        return self

    def __exit__(self, *exc):
        if self.log is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self.log.events.append((self.name, self.start, end))


def local_partition(cu_global: Sequence[int], rank: int, world_size: int):
    """This rank's slice of a contiguous partition.

    Returns ``(local_cu, continues_in, continues_out)``: the local boundaries (starting at 0; one entry per document
    fragment that has tokens here), whether the first fragment continues a document begun on an earlier rank, and
    whether the last fragment's document continues on a later rank.  The token count must divide by the world size.
    """
    total = int(cu_global[-1])
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} is not in a world of {world_size}")
    if total % world_size:
        raise ValueError(f"a contiguous partition needs the token count ({total}) to divide by the world size "
                         f"({world_size})")
    part = total // world_size
    lo, hi = rank * part, (rank + 1) * part
    cuts = sorted({min(max(int(b), lo), hi) for b in cu_global} | {lo, hi})
    local = tuple(b - lo for b in cuts)
    bounds = set(int(b) for b in cu_global)
    continues_in = part > 0 and lo not in bounds
    continues_out = part > 0 and hi not in bounds
    return local, continues_in, continues_out


def halo_rows(cu_global: Sequence[int], rank: int, world_size: int, reach: int) -> tuple[int, int]:
    """``(before, after)``: how many of the ``reach`` tokens just before this rank's slice belong to the document its
    first fragment continues, and how many of the ``reach`` tokens just after it belong to the document its last
    fragment continues into (what a causal convolution of width ``reach + 1`` reads across the cuts)."""
    total = int(cu_global[-1])
    part = total // world_size
    lo, hi = rank * part, (rank + 1) * part
    bounds = sorted(int(b) for b in cu_global)
    before = after = 0
    if part > 0 and lo not in bounds:
        before = min(reach, lo - max(b for b in bounds if b < lo))
    if part > 0 and hi not in bounds:
        after = min(reach, min(b for b in bounds if b > hi) - hi)
    return before, after


class _HaloExchange:
    """The rows a short causal convolution reads across the cuts of a CONTIGUOUS partition: three messages between
    neighbours, none where no document crosses the cut.  Every rank of the group makes the same calls in the same
    order.  Rows travel stacked per span, ``[1, reach, C]`` here (a contiguous slice is one span)."""

    def __init__(self, context: KcpContext) -> None:
        self.context = context

    def _swap(self, to_prev, to_next, want_prev: bool, want_next: bool):
        import torch.distributed as dist

        ctx = self.context
        peer = lambda offset: (ctx.rank + offset if ctx.group is None
                               else dist.get_global_rank(ctx.group, ctx.rank + offset))
        ops, from_prev, from_next = [], None, None
        template = to_prev if to_prev is not None else to_next
        if to_next is not None and ctx.continues_out:
            ops.append(dist.P2POp(dist.isend, to_next.contiguous(), peer(+1), ctx.group))
        if to_prev is not None and ctx.continues_in:
            ops.append(dist.P2POp(dist.isend, to_prev.contiguous(), peer(-1), ctx.group))
        if want_prev and ctx.continues_in:
            from_prev = torch.empty_like(template)
            ops.append(dist.P2POp(dist.irecv, from_prev, peer(-1), ctx.group))
        if want_next and ctx.continues_out:
            from_next = torch.empty_like(template)
            ops.append(dist.P2POp(dist.irecv, from_next, peer(+1), ctx.group))
        if ops and ctx.world_size > 1:
            for work in dist.batch_isend_irecv(ops):
                work.wait()
        return from_prev, from_next

    def forward(self, first_rows: torch.Tensor, last_rows: torch.Tensor):
        """``first_rows``, ``last_rows``: ``[spans, reach, C]``, the first and last rows of every local span.  Sends
        them to the ranks that hold the neighbouring spans; returns ``(rows before, rows after)``, a list per side
        with one ``[reach, C]`` tensor per span, ``None`` where no document crosses the cut."""
        if first_rows.shape[0] == 0:
            return [], []
        prev, nxt = self._swap(first_rows[0], last_rows[-1], True, True)
        return [prev], [nxt]

    def backward(self, first_rows: torch.Tensor):
        """Sends the first rows of the spans' output gradients to the ranks before; returns the rows after."""
        if first_rows.shape[0] == 0:
            return []
        return [self._swap(first_rows[0], None, False, True)[1]]


class _GatherHalo:
    """The same rows under any layout: one all-gather of every span's first and last rows (a few rows per span), from
    which a rank picks its neighbours' (``RankPlan.spans``)."""

    def __init__(self, context: KcpContext) -> None:
        self.context = context

    def _gather(self, local: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        ctx = self.context
        padded = local.new_zeros((ctx.plan.max_spans, *local.shape[1:]))
        padded[: local.shape[0]] = local
        gathered = padded.new_empty((ctx.world_size * padded.shape[0], *padded.shape[1:]))
        dist.all_gather_into_tensor(gathered, padded.contiguous(), group=ctx.group)
        return gathered.view(ctx.world_size, *padded.shape)

    def forward(self, first_rows: torch.Tensor, last_rows: torch.Tensor):
        both = self._gather(torch.stack([first_rows, last_rows], dim=1))  # [W, spans, 2, reach, C]
        spans = self.context.plan.spans
        prev = [None if sp.prev is None else both[sp.prev[0], sp.prev[1], 1].contiguous() for sp in spans]
        nxt = [None if sp.next is None else both[sp.next[0], sp.next[1], 0].contiguous() for sp in spans]
        return prev, nxt

    def backward(self, first_rows: torch.Tensor):
        rows = self._gather(first_rows)  # [W, spans, reach, C]
        return [None if sp.next is None else rows[sp.next[0], sp.next[1]].contiguous() for sp in self.context.plan.spans]


def document_run(cu_global: Sequence[int], rank: int, world_size: int) -> tuple[int, int]:
    """``(first, last)``: the first rank that holds tokens of the document this rank's first fragment continues, and
    the last rank that holds tokens of the document its last fragment continues into (``rank`` itself when nothing
    continues on that side)."""
    total = int(cu_global[-1])
    part = total // world_size
    lo, hi = rank * part, (rank + 1) * part
    bounds = sorted(int(b) for b in cu_global)
    first, last = rank, rank
    if part > 0 and lo not in bounds:
        begin = max(b for b in bounds if b < lo)  # where the document that crosses `lo` starts
        first = begin // part
    if part > 0 and hi not in bounds:
        end = min(b for b in bounds if b > hi)  # where the document that crosses `hi` ends
        last = (end - 1) // part
    return first, last


class _Exchange:
    """The state hand-over of one call: receive before the scan, send after it (forward: to the next rank; backward:
    to the previous one).  The hand-over is sequential along the rank chain, which reproduces the single-rank
    recurrence exactly."""

    def __init__(self, context: KcpContext) -> None:
        self.context = context

    # the hooks the stages call: around the state scan ...
    def forward_begin(self, dims, meta, k, w, u, g_cs, status, scan_segments: int = 0):
        """-> ``(h0 or None, keep the final state?)``"""
        ctx = self.context
        with _Timed("forward"):  # includes the wait for the rank before
            h0 = self.incoming_state(meta.num_seqs, w.shape[1], w.device)
        return h0, ctx.continues_out and ctx.world_size > 1

    def forward_end(self, final_state) -> None:
        if final_state is not None:
            self.outgoing_state(final_state)

    # ... and around the adjoint scan
    def backward_begin(self, dims, meta, tape, do, scan_segments: int = 0):
        """-> ``(dht or None, keep dh0?)``"""
        ctx = self.context
        with _Timed("backward"):  # includes the wait for the rank after
            dht = self.incoming_adjoint(meta.num_seqs, tape.v.shape[1], do.device)
        return dht, ctx.continues_in and ctx.world_size > 1

    def backward_end(self, dh0) -> None:
        if dh0 is not None:
            self.outgoing_adjoint(dh0)

    def take_prepared(self):
        """The hand-over leaves the scan as it is."""
        return None

    def _peer(self, offset: int) -> int:
        import torch.distributed as dist

        ctx = self.context
        peer = ctx.rank + offset
        return peer if ctx.group is None else dist.get_global_rank(ctx.group, peer)

    def incoming_state(self, num_local_seqs: int, num_v_heads: int, device) -> torch.Tensor | None:
        """``h0 [N_local, HV, 128, 128]``: zero, except the first fragment's when its document began earlier."""
        ctx = self.context
        if not ctx.continues_in or ctx.world_size == 1:
            return None
        import torch.distributed as dist

        h0 = torch.zeros(num_local_seqs, num_v_heads, 128, 128, dtype=torch.float32, device=device)
        dist.recv(h0[0], src=self._peer(-1), group=ctx.group)
        if _exchange_log is not None:
            _exchange_log.bytes_received += h0[0].numel() * 4
        return h0

    def outgoing_state(self, final_state: torch.Tensor) -> None:
        ctx = self.context
        if not ctx.continues_out or ctx.world_size == 1:
            return
        import torch.distributed as dist

        dist.send(final_state[-1].contiguous(), dst=self._peer(+1), group=ctx.group)

    def incoming_adjoint(self, num_local_seqs: int, num_v_heads: int, device) -> torch.Tensor | None:
        """``dht [N_local, HV, 128, 128]``: zero, except the last fragment's when its document continues later."""
        ctx = self.context
        if not ctx.continues_out or ctx.world_size == 1:
            return None
        import torch.distributed as dist

        dht = torch.zeros(num_local_seqs, num_v_heads, 128, 128, dtype=torch.float32, device=device)
        dist.recv(dht[-1], src=self._peer(+1), group=ctx.group)
        if _exchange_log is not None:
            _exchange_log.bytes_received += dht[-1].numel() * 4
        return dht

    def outgoing_adjoint(self, dh0: torch.Tensor) -> None:
        ctx = self.context
        if not ctx.continues_in or ctx.world_size == 1:
            return
        import torch.distributed as dist

        dist.send(dh0[0].contiguous(), dst=self._peer(-1), group=ctx.group)


class _ParallelExchange:
    """Every rank works at once: a rank summarises each of its fragments through which a state leaves it as
    ``(B, M)`` with ``S_out = M S_in + B`` (pre-scan of the fragment's segments, composed by the stitch kernel), one
    all-gather shares the summaries, and each rank folds, per fragment, the chain of the fragments before it in its
    document into the state that enters it (reference: the affine summaries of
    miles_ext_kernels/cake/_impl/gdn/kcp.py and _vendor/cake_gdn_det_train_kcp).  The cost per rank is one pre-scan
    per published fragment, one gather and its own scan, whatever the number of ranks; the result agrees with the
    sequential hand-over within the accuracy budgets, not bit for bit (a state crosses a fragment as ``M S + B`` in
    fp32 instead of through the chunk steps).  Serves every layout: under the contiguous one a rank publishes at
    most one summary per direction."""

    def __init__(self, context: KcpContext) -> None:
        self.context = context
        self._prepared = None

    def take_prepared(self):
        """``(plan, seg_dims, summary)`` when the exchange has already summarised the segments this rank's scan is cut
        into (every segment from zero and from the identity): the scan then needs no pre-scan of its own, only the
        stitch from the state that entered.  ``None`` otherwise.  Handed over once."""
        prepared, self._prepared = self._prepared, None
        return prepared

    def _gather(self, local: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        ctx = self.context
        gathered = torch.empty((ctx.world_size * local.shape[0], *local.shape[1:]), dtype=local.dtype,
                               device=local.device)
        dist.all_gather_into_tensor(gathered, local, group=ctx.group)
        if _exchange_log is not None:
            _exchange_log.bytes_received += (ctx.world_size - 1) * local.numel() * local.element_size()
        return gathered.view(ctx.world_size, *local.shape)

    @staticmethod
    def _chain(flat: torch.Tensor, slots: int, chain) -> torch.Tensor:
        """The summaries ``[(rank, slot), ...]`` of ``flat [W * slots, HV, 2, 128, 128]`` as one tensor, in order."""
        index = [r * slots + s for r, s in chain]
        if index == list(range(index[0], index[0] + len(index))):
            return flat[index[0] : index[0] + len(index)]
        from . import scan

        return flat.index_select(0, scan._small_table(tuple(index), torch.int64, flat.device))

    def _exchange(self, dims, meta, HV, device, publish, slots, chains, summarise, reverse, scan_segments: int = 0):
        from . import scan

        # slots nobody publishes are read by nobody: a chain names published (rank, slot) pairs only
        local = torch.empty((max(slots, 1), HV, 2, 128, 128), dtype=torch.float32, device=device)
        table = meta.host_seq_chunk_start
        self._prepared = None
        shared = None
        if meta.num_seqs == 1 and not getattr(self, "_exact", False):
            # One sequence on this rank (a slice of a long document): its summary is composed from the very segments
            # the scan planner cuts the slice into, so one pre-scan serves the exchange and the scan.  Every rank does
            # it before the gather, the last one too, whose summary nobody reads.
            shared = scan.plan_for(meta, HV, device, scan_segments)
        if shared is not None:
            ones = scan._small_table((1,) * shared.segments, torch.int32, device)
            seg_dims = scan.segment_dims(dims, shared)
            summary = torch.empty((shared.segments, HV, 2, 128, 128), dtype=torch.float32, device=device)
            summarise(seg_dims, dataclasses.replace(shared, flags_fwd=ones, flags_bwd=ones), summary)
            if publish:
                scan.compose_summary(seg_dims, shared, summary, self._g_cs, reverse=reverse, out=local[0])
            self._prepared = (shared, seg_dims, summary)
            publish = ()
        for slot, f in enumerate(publish):
            plan = scan.fragment_plan(table[f], table[f + 1], HV, device)
            if getattr(self, "_exact", False):
                plan = dataclasses.replace(plan, warm_chunks=0)
            seg_dims = scan.segment_dims(dims, plan)
            summary = torch.empty((plan.segments, HV, 2, 128, 128), dtype=torch.float32, device=device)
            summarise(seg_dims, plan, summary)
            scan.compose_summary(seg_dims, plan, summary, self._g_cs, reverse=reverse, out=local[slot])
        gathered = self._gather(local)
        if not any(chains):
            return None
        flat = gathered.view(-1, HV, 2, 128, 128)
        alloc = torch.empty if all(chains) else torch.zeros  # a sequence nothing enters starts from zero
        states = alloc((meta.num_seqs, HV, 128, 128), dtype=torch.float32, device=device)
        for f, chain in enumerate(chains):
            if chain:
                run = self._chain(flat, max(slots, 1), chain)
                scan.fold_ranks(dims, run, 0, len(chain) - 1, reverse=reverse, out=states[f : f + 1])
        return states

    def forward_begin(self, dims, meta, k, w, u, g_cs, status, scan_segments: int = 0):
        from . import native

        plan = self.context.plan
        device, HV = w.device, w.shape[1]
        self._g_cs, self._exact = g_cs, False

        def summarise(seg_dims, frag, summary):
            native.launch("gdn_fwd_h_prescan", seg_dims, k, w, u, g_cs, None, frag.flags_fwd, frag.state_row,
                          frag.warm_chunks, frag.warm_log2, summary, status, device=device)

        with _Timed("forward"):
            h0 = self._exchange(dims, meta, HV, device, plan.publish_forward, plan.slots_forward, plan.chain_forward,
                                summarise, reverse=False, scan_segments=scan_segments)
        return h0, False

    def forward_end(self, final_state) -> None:
        pass

    # the per-channel-decay variant (KDA): the same exchange on its scan operands; its pre-scans have no warm-up rule
    def kda_forward_state(self, dims, meta, kr, w, u, gl2, status):
        from . import native

        plan = self.context.plan
        device, H = w.device, w.shape[1]
        self._g_cs, self._exact = None, True

        def summarise(seg_dims, frag, summary):
            native.launch("kda_fwd_h_prescan", seg_dims, kr, w, u, gl2, None, frag.flags_fwd, frag.state_row, summary,
                          status, device=device)

        return self._exchange(dims, meta, H, device, plan.publish_forward, plan.slots_forward, plan.chain_forward,
                              summarise, reverse=False)

    def kda_backward_state(self, dims, meta, saved, do):
        from . import native

        plan = self.context.plan
        device, H = do.device, do.shape[1]
        self._g_cs, self._exact = None, True

        def summarise(seg_dims, frag, summary):
            native.launch("kda_bwd_dh_prescan", seg_dims, saved.qg, saved.kr, saved.w, do, saved.aqk, saved.gl2, None,
                          frag.flags_bwd, frag.state_row, summary, saved.status, device=device)

        return self._exchange(dims, meta, H, device, plan.publish_backward, plan.slots_backward, plan.chain_backward,
                              summarise, reverse=True)

    def backward_begin(self, dims, meta, tape, do, scan_segments: int = 0):
        from . import native

        plan = self.context.plan
        device, HV = do.device, tape.v.shape[1]
        self._g_cs, self._exact = tape.g_cs, False

        def summarise(seg_dims, frag, summary):
            native.launch("gdn_bwd_dh_prescan", seg_dims, tape.qn, tape.kn, tape.w, do, tape.aqk, tape.g_cs, None,
                          frag.flags_bwd, frag.state_row, frag.warm_chunks, frag.warm_log2, summary, tape.status,
                          device=device)

        with _Timed("backward"):
            dht = self._exchange(dims, meta, HV, device, plan.publish_backward, plan.slots_backward,
                                 plan.chain_backward, summarise, reverse=True, scan_segments=scan_segments)
        return dht, False

    def backward_end(self, dh0) -> None:
        pass


class KcpContext:
    """One rank's view of a partition of a packed batch (reference:
    miles_ext_kernels/cake/_impl/gdn/kcp.py:71-169): ``rank``, ``world_size``, ``num_tokens`` (this rank's),
    ``cu_seqlens`` / ``cu_seqlens_cpu`` (local boundaries, one sequence per fragment), ``fragments``, ``layout``,
    ``group``, ``fla_compatible`` and the ``plan`` of what crosses the cuts (``layout.RankPlan``)."""

    def __init__(self, cu_seqlens_global, group, rank: int, world_size: int, device, conv_kernel_size: int = 4,
                 layout: str = "contiguous", fragments=None) -> None:
        self.cu_seqlens_global = tuple(int(b) for b in cu_seqlens_global)
        if not self.cu_seqlens_global or self.cu_seqlens_global[0] != 0:
            raise ValueError("KcpContext: cu_seqlens_global must start at 0")
        self.group = group
        self.rank, self.world_size = int(rank), int(world_size)
        if not 0 <= self.rank < self.world_size:
            raise ValueError(f"rank {rank} is not in a world of {world_size}")
        self.device = torch.device(device)
        self.conv_kernel_size = int(conv_kernel_size)
        self.layout = "explicit" if fragments is not None else layout
        table = layout_module.partition(self.cu_seqlens_global, self.world_size, layout, fragments)
        self.plan = layout_module.rank_plan(self.cu_seqlens_global, table, self.rank, self.conv_kernel_size - 1)
        self.fragments = self.plan.fragments
        self.cu_seqlens_cpu = self.plan.cu_seqlens
        self.num_tokens = self.cu_seqlens_cpu[-1]
        lengths = [b - a for a, b in zip(self.cu_seqlens_global, self.cu_seqlens_global[1:])]
        # of the slice as a whole: what the rank-to-rank hand-over of the contiguous layout looks at
        self.continues_in = bool(self.fragments) and self.fragments[0].offset > 0
        self.continues_out = bool(self.fragments) and self.fragments[-1].end < lengths[self.fragments[-1].doc]
        self.cu_seqlens = torch.tensor(self.cu_seqlens_cpu, dtype=torch.int32, device=self.device)
        self.fla_compatible = self.layout == "contiguous"  # a contiguous partition is FLA's
        spans = self.plan.spans
        self.halo = (spans[0].before, spans[-1].after) if spans else (0, 0)

    def halo_exchange(self):
        """The neighbour exchange of the layer's short convolutions: point to point along the rank chain under the
        contiguous layout, one small all-gather under the others."""
        return _HaloExchange(self) if self.layout == "contiguous" else _GatherHalo(self)

    def exchange(self, mode: str = "auto"):
        """The boundary-state exchange of one call: ``"sequential"`` (rank to rank; the single-rank bits on aligned
        boundaries; contiguous layout only), ``"parallel"`` (affine fragment summaries, one all-gather; every rank
        works at once) or ``"auto"`` (parallel from three ranks on and under every other layout)."""
        if mode not in ("auto", "sequential", "parallel"):
            raise ValueError(f"unknown exchange mode {mode!r}")
        if self.layout != "contiguous" and self.world_size > 1:
            if mode == "sequential":
                raise NotImplementedError(
                    f"the sequential hand-over follows the rank chain of the contiguous layout; the {self.layout} "
                    "layout takes the parallel exchange")
            return _ParallelExchange(self)
        if mode == "auto":
            mode = "parallel" if self.world_size > 2 else "sequential"
        if mode == "parallel" and self.world_size > 1:
            return _ParallelExchange(self)
        return _Exchange(self)

    def __repr__(self) -> str:
        return (f"KcpContext(rank={self.rank}, world_size={self.world_size}, num_tokens={self.num_tokens}, "
                f"layout={self.layout!r}, cu_seqlens_cpu={self.cu_seqlens_cpu})")


def build_kcp_context(cu_seqlens_global, group=None, *, device=None, conv_kernel_size: int = 4,
                      layout: str = "contiguous", fragments=None) -> KcpContext:
    """The :class:`KcpContext` of this process for the global boundaries ``cu_seqlens_global`` (a sequence of ints or
    a CPU tensor) and the process group ``group`` (default: the world).  Cached per layout, so every layer of a
    micro-batch shares one context."""
    import torch.distributed as dist

    if isinstance(cu_seqlens_global, torch.Tensor):
        if cu_seqlens_global.is_cuda:
            raise ValueError("build_kcp_context: cu_seqlens_global must be on the host (a tuple or a CPU tensor)")
        cu_seqlens_global = cu_seqlens_global.tolist()
    boundaries = tuple(int(b) for b in cu_seqlens_global)
    if dist.is_available() and dist.is_initialized():
        rank, world = dist.get_rank(group), dist.get_world_size(group)
    else:
        rank, world = 0, 1
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"
    device = torch.device(device)
    if layout not in LAYOUTS:
        raise ValueError(f"build_kcp_context: layout must be one of {LAYOUTS}, not {layout!r}")
    frozen = None if fragments is None else tuple(tuple(tuple(int(x) for x in f) for f in rank_) for rank_ in fragments)
    key = (boundaries, id(group), rank, world, str(device), conv_kernel_size, layout, frozen)
    found = _CONTEXTS.get(key)
    if found is not None:
        _CONTEXTS.move_to_end(key)
        return found
    context = KcpContext(boundaries, group, rank, world, device, conv_kernel_size, layout, fragments)
    _CONTEXTS[key] = context
    while len(_CONTEXTS) > _CACHE_LIMIT:
        _CONTEXTS.popitem(last=False)
    return context


def release() -> None:
    _CONTEXTS.clear()
