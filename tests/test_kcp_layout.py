"""The partitions of a packed batch over a context-parallel group and what crosses their cuts (host logic; CPU):
every layout covers every token exactly once, the chains list a fragment's predecessors in document order, the
convolution's spans name the ranks that hold the neighbouring rows (reference: the ``layout`` / ``fragments``
arguments of miles_ext_kernels/cake/_impl/gdn/kcp.py:185-226)."""

from __future__ import annotations

import pytest

from miles_ext_kernels_b200.cake._impl.gdn import layout as L


def _tokens(cu, fragments):
    return [cu[f.doc] + t for f in fragments for t in range(f.offset, f.end)]


@pytest.mark.parametrize("layout,cu,world", [
    ("contiguous", (0, 15, 20, 64), 4), ("zigzag", (0, 15, 20, 64), 4), ("zigzag", (0, 64), 2),
    ("zigzag_per_document", (0, 16, 48, 64), 2), ("zigzag_per_document", (0, 64, 128), 4), ("zigzag", (0, 5, 5, 16), 1),
])
def test_every_token_is_held_once_and_balanced(layout, cu, world):
    table = L.partition(cu, world, layout)
    held = sorted(t for rank in table for t in _tokens(cu, rank))
    assert held == list(range(cu[-1]))
    assert len({sum(f.length for f in rank) for rank in table}) == 1  # the same number of tokens on every rank
    for rank in range(world):
        plan = L.rank_plan(cu, table, rank)
        assert plan.cu_seqlens[-1] == cu[-1] // world and len(plan.cu_seqlens) == len(plan.fragments) + 1
        for f, before, after in zip(plan.fragments, plan.chain_forward, plan.chain_backward):
            assert (len(before) > 0) == (f.offset > 0)
            assert (len(after) > 0) == (f.end < cu[f.doc + 1] - cu[f.doc])


def test_zigzag_pieces_and_chains():
    cu = (0, 6000, 8192)
    table = L.partition(cu, 4, "zigzag")
    assert [(f.doc, f.offset, f.length) for f in table[2]] == [(0, 2048, 1024), (0, 5120, 880), (1, 0, 144)]
    plan = L.rank_plan(cu, table, 2)
    assert plan.publish_forward == (0, 2) and plan.publish_backward == (0, 1)
    # document 0 before [5120, 6000): pieces 0..4 = rank 0, rank 1, rank 2 (its own first fragment), rank 3 (merged 3, 4)
    assert plan.chain_forward[1] == ((0, 0), (1, 0), (2, 0), (3, 0))
    assert plan.chain_forward[2] == () and plan.chain_backward[1] == ()
    # the spans: [2048, 3072) alone; the tail of document 0 and the head of document 1 together
    assert [(s.first, s.last, s.before, s.after, s.prev, s.next) for s in plan.spans] == [
        (0, 0, 3, 3, (1, 0), (3, 0)), (1, 2, 3, 3, (3, 0), (1, 1))]
    assert plan.slots_forward == 2 and plan.max_spans == 2


def test_explicit_tables_and_rejections():
    cu = (0, 10, 30)
    table = L.partition(cu, 2, fragments=[[(0, 0, 4), (1, 5, 15)], [(0, 4, 6), (1, 0, 5)]])
    plan = L.rank_plan(cu, table, 0)
    assert plan.cu_seqlens == (0, 4, 19) and plan.chain_forward[1] == ((1, 0),)
    with pytest.raises(ValueError, match="held by no rank"):
        L.partition(cu, 2, fragments=[[(0, 0, 4)], [(0, 4, 6), (1, 0, 5)]])
    with pytest.raises(ValueError, match="by no rank or by two"):
        L.partition(cu, 2, fragments=[[(0, 0, 4), (1, 0, 20)], [(0, 5, 5)]])
    with pytest.raises(ValueError, match="twice the world size"):
        L.partition((0, 10), 2, "zigzag")
    with pytest.raises(ValueError, match="every document length"):
        L.partition((0, 8, 14), 2, "zigzag_per_document")
    with pytest.raises(ValueError, match="layout must be one of"):
        L.partition((0, 8), 2, "striped")
    short = L.partition((0, 2, 16), 2, fragments=[[(0, 0, 2), (1, 0, 6)], [(1, 6, 8)]])
    assert L.rank_plan((0, 2, 16), short, 0).spans[0].after == 3
    tiny = L.partition((0, 16), 3, fragments=[[(0, 0, 4)], [(0, 4, 2)], [(0, 6, 10)]])
    with pytest.raises(NotImplementedError, match="rows before a fragment"):
        L.rank_plan((0, 16), tiny, 2)  # the three rows before token 6 lie on two ranks


def test_the_context_under_each_layout():
    from miles_ext_kernels_b200.cake._impl.gdn.kcp import KcpContext, _Exchange, _ParallelExchange

    cu = (0, 6000, 8192)
    ctx = KcpContext(cu, None, 1, 4, "cpu", layout="zigzag")
    assert ctx.layout == "zigzag" and not ctx.fla_compatible and ctx.num_tokens == 2048
    assert ctx.cu_seqlens_cpu == (0, 1024, 2048) and ctx.cu_seqlens.tolist() == [0, 1024, 2048]
    assert isinstance(ctx.exchange("auto"), _ParallelExchange)
    with pytest.raises(NotImplementedError, match="sequential hand-over"):
        ctx.exchange("sequential")
    flat = KcpContext(cu, None, 1, 2, "cpu")
    assert flat.fla_compatible and isinstance(flat.exchange("auto"), _Exchange) and flat.halo == (3, 0)
    assert flat.continues_in and not flat.continues_out
    explicit = KcpContext((0, 10, 30), None, 0, 2, "cpu", fragments=[[(0, 0, 4), (1, 5, 15)], [(0, 4, 6), (1, 0, 5)]])
    assert explicit.layout == "explicit" and explicit.num_tokens == 19
