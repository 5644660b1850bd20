"""Which tokens of a packed batch a rank of a context-parallel group holds, and what crosses its cuts.

A partition is a table per rank of document fragments ``(doc, offset, length)`` in the rank's local token order
(reference: the ``layout`` / ``fragments`` arguments of ``build_kcp_context``,
miles_ext_kernels/cake/_impl/gdn/kcp.py:185-226, and :data:`KCP_LAYOUTS` there).  Three layouts generate such tables:

``contiguous``           rank r holds tokens ``[r T / W, (r + 1) T / W)``
``zigzag``               the tokens are cut into 2 W equal pieces; rank r holds pieces r and 2 W - 1 - r, so that a
                         causal workload is balanced
``zigzag_per_document``  the same per document: every document is cut into 2 W equal pieces

and an explicit table may be given instead.  Host logic only: every rank derives every rank's table from the global
boundaries, so no collective is needed to know who holds what.

From the tables follow, per rank (:class:`RankPlan`):

* the local sequences (one per fragment; fragments of one document that touch are merged),
* for the chunk state: which fragments publish a summary of themselves (those that are not the last of their
  document in the forward direction, not the first in the backward one) and, per fragment, the chain of fragments
  before (after) it in its document whose summaries fold into the state that enters it,
* for the short convolution: the spans of consecutive local fragments that one launch serves (a span starts at a
  fragment that continues a document and ends at one whose document goes on elsewhere) with the ranks and spans that
  hold the three rows before and after each.
"""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass

__all__ = ["KCP_LAYOUTS", "Fragment", "RankPlan", "Span", "partition", "rank_plan"]

KCP_LAYOUTS = ("contiguous", "zigzag", "zigzag_per_document")


@dataclass(frozen=True)
class Fragment:
    """Tokens ``[offset, offset + length)`` of document ``doc``."""

    doc: int
    offset: int
    length: int

    @property
    def end(self) -> int:
        return self.offset + self.length


@dataclass(frozen=True)
class Span:
    """Local fragments ``[first, last]`` (tokens ``[token_lo, token_hi)``) that one convolution launch serves:
    ``before`` rows of history from the end of span ``prev[1]`` of rank ``prev[0]``, ``after`` rows of continuation
    from the start of span ``next[1]`` of rank ``next[0]`` (``None``: nothing on that side)."""

    first: int
    last: int
    token_lo: int
    token_hi: int
    before: int
    after: int
    prev: tuple[int, int] | None
    next: tuple[int, int] | None


@dataclass(frozen=True)
class RankPlan:
    fragments: tuple[Fragment, ...]
    cu_seqlens: tuple[int, ...]
    publish_forward: tuple[int, ...]   # local fragments whose documents go on after them: slot = position here
    publish_backward: tuple[int, ...]  # local fragments whose documents began before them
    chain_forward: tuple[tuple[tuple[int, int], ...], ...]   # per local fragment: (rank, forward slot) of every
    chain_backward: tuple[tuple[tuple[int, int], ...], ...]  # fragment before / after it, in document order
    slots_forward: int                 # the most slots any rank publishes (the gathered tensor's second extent)
    slots_backward: int
    spans: tuple[Span, ...]
    max_spans: int


def _cuts(cu: Sequence[int], lo: int, hi: int) -> list[Fragment]:
    """The document fragments inside the global token range ``[lo, hi)``."""
    out = []
    for doc, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
        x, y = max(a, lo), min(b, hi)
        if y > x:
            out.append(Fragment(doc, x - a, y - x))
    return out


def _merged(fragments: Sequence[Fragment]) -> tuple[Fragment, ...]:
    out: list[Fragment] = []
    for f in fragments:
        if f.length <= 0:
            continue
        if out and out[-1].doc == f.doc and out[-1].end == f.offset:
            out[-1] = Fragment(f.doc, out[-1].offset, out[-1].length + f.length)
        else:
            out.append(f)
    return tuple(out)


def partition(cu_seqlens_global: Sequence[int], world_size: int, layout: str = "contiguous",
              fragments=None) -> tuple[tuple[Fragment, ...], ...]:
    """Every rank's fragments, in local order.  ``fragments``: an explicit table
    ``[[(doc, offset, length), ...], ...]`` (one list per rank) instead of a layout; it must cover every document
    exactly once."""
    cu = [int(b) for b in cu_seqlens_global]
    if len(cu) < 1 or cu[0] != 0 or any(b < a for a, b in zip(cu, cu[1:])):
        raise ValueError("cu_seqlens_global must start at 0 and not decrease")
    total = cu[-1]
    if world_size <= 0:
        raise ValueError(f"a world of {world_size} ranks")
    if fragments is not None:
        if len(fragments) != world_size:
            raise ValueError(f"an explicit table needs one fragment list per rank ({world_size}), got {len(fragments)}")
        table = tuple(_merged([Fragment(int(d), int(o), int(n)) for d, o, n in rank]) for rank in fragments)
        _check_cover(cu, table)
        return table
    if layout not in KCP_LAYOUTS:
        raise ValueError(f"layout must be one of {KCP_LAYOUTS}, not {layout!r}")
    if layout == "contiguous":
        if total % world_size:
            raise ValueError(f"a contiguous partition needs the token count ({total}) to divide by the world size "
                             f"({world_size})")
        part = total // world_size
        return tuple(_merged(_cuts(cu, r * part, (r + 1) * part)) for r in range(world_size))
    pieces = 2 * world_size
    if layout == "zigzag":
        if total % pieces:
            raise ValueError(f"a zigzag partition needs the token count ({total}) to divide by twice the world size "
                             f"({pieces})")
        part = total // pieces
        return tuple(_merged(_cuts(cu, r * part, (r + 1) * part) +
                             _cuts(cu, (pieces - 1 - r) * part, (pieces - r) * part)) for r in range(world_size))
    lengths = [b - a for a, b in zip(cu, cu[1:])]
    bad = [n for n in lengths if n % pieces]
    if bad:
        raise ValueError(f"a per-document zigzag partition needs every document length to divide by twice the world "
                         f"size ({pieces}); got a document of {bad[0]} tokens")
    table = []
    for r in range(world_size):
        mine = []
        for doc, n in enumerate(lengths):
            part = n // pieces
            mine += [Fragment(doc, r * part, part), Fragment(doc, (pieces - 1 - r) * part, part)]
        table.append(_merged(mine))
    return tuple(table)


def _check_cover(cu: Sequence[int], table) -> None:
    lengths = [b - a for a, b in zip(cu, cu[1:])]
    seen: dict[int, list[tuple[int, int]]] = {}
    for rank in table:
        for f in rank:
            if not 0 <= f.doc < len(lengths) or f.offset < 0 or f.end > lengths[f.doc]:
                raise ValueError(f"fragment {f} is outside its document")
            seen.setdefault(f.doc, []).append((f.offset, f.end))
    for doc, n in enumerate(lengths):
        at = 0
        for a, b in sorted(seen.get(doc, [])):
            if a != at:
                raise ValueError(f"document {doc}: tokens [{at}, {a}) are held by no rank or by two")
            at = b
        if at != n:
            raise ValueError(f"document {doc}: tokens [{at}, {n}) are held by no rank")


def rank_plan(cu_seqlens_global: Sequence[int], table, rank: int, reach: int = 3) -> RankPlan:
    """What ``rank`` publishes, folds and exchanges under the partition ``table`` (:func:`partition`); ``reach``:
    the short convolution's width minus one."""
    cu = [int(b) for b in cu_seqlens_global]
    lengths = [b - a for a, b in zip(cu, cu[1:])]
    world = len(table)
    # forward / backward slots of every rank's fragments, and every document's fragments in order
    slot_f: list[dict[int, int]] = []
    slot_b: list[dict[int, int]] = []
    by_doc: dict[int, list[tuple[int, int, int]]] = {}  # doc -> [(offset, rank, local index)]
    for r, frags in enumerate(table):
        sf, sb = {}, {}
        for i, f in enumerate(frags):
            if f.end < lengths[f.doc]:
                sf[i] = len(sf)
            if f.offset > 0:
                sb[i] = len(sb)
            by_doc.setdefault(f.doc, []).append((f.offset, r, i))
        slot_f.append(sf)
        slot_b.append(sb)
    for entries in by_doc.values():
        entries.sort()
    mine = table[rank]
    chain_f, chain_b = [], []
    for i, f in enumerate(mine):
        order = by_doc[f.doc]
        at = order.index((f.offset, rank, i))
        chain_f.append(tuple((r, slot_f[r][j]) for _, r, j in order[:at]))
        chain_b.append(tuple((r, slot_b[r][j]) for _, r, j in order[at + 1:]))
    # spans of every rank (the convolution's launches): a new span starts at a fragment that continues a document
    # and after a fragment whose document goes on
    def spans_of(r: int):
        frags = table[r]
        out, first, tok = [], 0, 0
        starts = [0]
        for f in frags:
            starts.append(starts[-1] + f.length)
        for i, f in enumerate(frags):
            last_of_span = i + 1 == len(frags) or f.end < lengths[f.doc] or frags[i + 1].offset > 0
            if last_of_span:
                out.append((first, i, starts[first], starts[i + 1]))
                first = i + 1
        return out

    all_spans = [spans_of(r) for r in range(world)]
    span_starting = {}  # (rank, local fragment index) -> span index on that rank
    span_ending = {}
    for r, spans in enumerate(all_spans):
        for s, (a, b, _, _) in enumerate(spans):
            span_starting[(r, a)] = s
            span_ending[(r, b)] = s
    my_spans = []
    for a, b, lo, hi in all_spans[rank]:
        head, tail = mine[a], mine[b]
        prev = nxt = None
        before = after = 0
        if head.offset > 0:
            order = by_doc[head.doc]
            _, pr, pi = order[order.index((head.offset, rank, a)) - 1]
            before = min(reach, head.offset)
            if table[pr][pi].length < before:
                raise NotImplementedError(
                    f"the short convolution reads {before} rows before a fragment; the fragment before it holds "
                    f"{table[pr][pi].length}")
            prev = (pr, span_ending[(pr, pi)])
        if tail.end < lengths[tail.doc]:
            order = by_doc[tail.doc]
            _, nr, ni = order[order.index((tail.offset, rank, b)) + 1]
            after = min(reach, lengths[tail.doc] - tail.end)
            if table[nr][ni].length < after:
                raise NotImplementedError(
                    f"the short convolution's backward reads {after} rows after a fragment; the fragment after it "
                    f"holds {table[nr][ni].length}")
            nxt = (nr, span_starting[(nr, ni)])
        my_spans.append(Span(a, b, lo, hi, before, after, prev, nxt))
    cu_local = [0]
    for f in mine:
        cu_local.append(cu_local[-1] + f.length)
    return RankPlan(
        fragments=tuple(mine), cu_seqlens=tuple(cu_local),
        publish_forward=tuple(sorted(slot_f[rank], key=slot_f[rank].get)),
        publish_backward=tuple(sorted(slot_b[rank], key=slot_b[rank].get)),
        chain_forward=tuple(chain_f), chain_backward=tuple(chain_b),
        slots_forward=max((len(s) for s in slot_f), default=0),
        slots_backward=max((len(s) for s in slot_b), default=0),
        spans=tuple(my_spans), max_spans=max((len(s) for s in all_spans), default=0),
    )
