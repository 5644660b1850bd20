"""The scan planner (CPU) and the segmented scans against the serial ones and the FP64 recurrence (GPU)."""

from __future__ import annotations

import pytest
import torch

from gdn_cases import draw
from oracle import gdn_oracle as O


def test_segments_cover_the_chunks_and_keep_a_minimum_length():
    from miles_ext_kernels_b200.cake._impl.gdn import scan

    table = (0, 49, 53, 86, 86, 101)  # sequences of 49, 4, 33, 0 and 15 chunks
    for parts in (1, 2, 3, 5, 16):
        seg = scan.segment(table, parts)
        assert seg.seg_chunk_start[0] == 0 and seg.seg_chunk_start[-1] == table[-1]
        assert all(b >= a for a, b in zip(seg.seg_chunk_start, seg.seg_chunk_start[1:]))
        assert len(seg.seq_seg_start) == len(table)
        for n, (a, b) in enumerate(zip(seg.seq_seg_start, seg.seq_seg_start[1:])):
            assert seg.seg_chunk_start[a] == table[n] and seg.seg_chunk_start[b] == table[n + 1]
            pieces = b - a
            assert 1 <= pieces <= max(1, min(parts, (table[n + 1] - table[n]) // scan.MIN_SEGMENT_CHUNKS))
            for s in range(a, b):
                length = seg.seg_chunk_start[s + 1] - seg.seg_chunk_start[s]
                assert pieces == 1 or length >= scan.MIN_SEGMENT_CHUNKS
    assert scan.segment(table, 3).seq_seg_start == (0, 3, 4, 6, 7, 8)


def test_the_planner_cuts_only_when_chains_are_few_and_long():
    from miles_ext_kernels_b200.cake._impl.gdn import scan

    cfg1 = tuple(range(0, 4 * 128 + 1, 128))  # 4 sequences of 128 chunks, 32 value heads: 128 chains
    assert scan.choose_parts(cfg1, 32, 148) == 1
    cfg4 = (0, 512)  # one 32,768-token slice, 32 value heads: 32 chains
    parts = scan.choose_parts(cfg4, 32, 148)
    assert parts > 1
    cut, serial = scan.segment(cfg4, parts), scan.segment(cfg4, 1)
    assert scan.modelled_steps(cut, 32, 148) < scan.MIN_GAIN * scan.modelled_steps(serial, 32, 148)
    assert scan.choose_parts((0, 20), 32, 148) == 1  # too short to cut
    assert scan.choose_parts(cfg1, 32, 148, forced=4) == 4 and scan.choose_parts(cfg4, 32, 148, forced=1) == 1
    assert scan.choose_parts(cfg4, 32, 148, forced=99) == scan.MAX_PARTS


SEQ_LENS = (3100, 200)  # 49 and 4 chunks: three segments with a middle one (offset and transfer walks), one uncut
HEADS = (1, 2)


@pytest.mark.gpu
@pytest.mark.parametrize("gate", ["weak", "strong"])
def test_segmented_scans_against_the_serial_ones_and_the_fp64_recurrence(gate):
    """Weak gates take the exact summaries (M S + B across every cut); the benchmark's strong gates take the
    warm-up rule (the offset walk of the closing chunks only)."""
    import miles_ext_kernels_b200 as package
    from test_gdn_gpu import assert_within, run

    x = draw(SEQ_LENS, HEADS, seed=31, gate=gate, state=True, normalised=gate == "strong")
    l2 = gate != "strong"
    ref = O.recurrence_fp64(x["q"], x["k"], x["v"], x["g"], x["beta"], SEQ_LENS, h0=x["h0"], do=x["do"],
                            dht=x["dht"], use_qk_l2norm=l2, output_final_state=True)
    try:
        package.configure(cake_gdn_scan_segments=1)
        serial = run(x, SEQ_LENS, state=True, l2=l2)
        package.configure(cake_gdn_scan_segments=3)
        cut = run(x, SEQ_LENS, state=True, l2=l2)
        again = run(x, SEQ_LENS, state=True, l2=l2)
    finally:
        package.configure()
    names = ("o", "dq", "dk", "dv", "dg", "dbeta", "final_state", "dh0")
    assert_within(cut, ref, f"segmented, {gate} gates", names=names)
    for name in names:  # the same plan gives the same bits; the serial walk agrees far inside the budgets
        assert torch.equal(cut[name], again[name]), name
        m = O.metrics(cut[name].float(), serial[name].float())
        assert m["finite"] and m["rel_rms"] <= 2e-3 and m["max_abs"] <= 1e-2 * max(m["max_ref"], 1e-6), (name, m)


@pytest.mark.gpu
def test_the_planner_engages_on_few_long_chains_and_the_recomputed_backward_follows_it():
    import miles_ext_kernels_b200 as package
    from miles_ext_kernels_b200.cake._impl.gdn import meta as meta_module
    from miles_ext_kernels_b200.cake._impl.gdn import scan
    from test_gdn_gpu import run

    seq_lens = (4096,)
    x = draw(seq_lens, (1, 2), seed=32, gate="weak")
    meta = meta_module.chunk_meta(torch.tensor((0, 4096)), (0, 4096), 1, 4096, torch.device("cuda"))
    assert scan.plan_for(meta, 2, torch.device("cuda")) is not None  # 2 chains of 64 chunks: cut
    try:
        saved = run(x, seq_lens)
        package.configure(cake_gdn_recompute_state=True)
        recomputed = run(x, seq_lens)
        package.configure(cake_gdn_scan_segments=1)
        serial = run(x, seq_lens)
    finally:
        package.configure()
    for name in saved:
        assert torch.equal(saved[name], recomputed[name]), name
        m = O.metrics(saved[name].float(), serial[name].float())
        assert m["finite"] and m["rel_rms"] <= 2e-3, (name, m)


@pytest.mark.gpu
@pytest.mark.parametrize("reverse", [False, True])
def test_a_run_of_segments_composed_in_one_launch_equals_the_two_stitches(reverse):
    """``mek_gdn_scan_compose`` writes the (B, M) of a run of segments per head, interleaved, in one launch: the same
    bits as the stitch kernel run once from zero with the offsets (B) and once from the identity without them (M)."""
    from miles_ext_kernels_b200.cake._impl.gdn import meta as meta_module
    from miles_ext_kernels_b200.cake._impl.gdn import native, scan
    from miles_ext_kernels_b200.cake._impl.gdn.stages import dims_of

    dev = torch.device("cuda")
    heads, tokens = 3, 64 * 40
    meta = meta_module.chunk_meta(torch.tensor((0, tokens)), (0, tokens), 1, tokens, dev)
    plan = scan.fragment_plan(0, meta.num_chunks, heads, dev)
    assert plan.segments > 1
    dims = dims_of(meta, heads, heads, 1.0)
    seg_dims = scan.segment_dims(dims, plan)
    torch.manual_seed(5)
    summary = (0.3 * torch.randn(plan.segments, heads, 2, 128, 128, device=dev)).contiguous()
    g_cs = -torch.rand(tokens, heads, device=dev)  # mild gates: the warm-up rule does not apply, M matters
    one = scan.compose_summary(seg_dims, plan, summary, g_cs, reverse=reverse)
    two = torch.empty((2, heads, 128, 128), dtype=torch.float32, device=dev)
    for which, mode in ((0, 4), (1, 7)):
        native.launch("gdn_scan_stitch", seg_dims, 1, plan.seq_seg_start, summary, None, g_cs, None, two[which],
                      int(reverse), plan.warm_chunks, plan.warm_log2, mode, device=dev)
    torch.cuda.synchronize()
    assert torch.equal(one[:, 0], two[0]) and torch.equal(one[:, 1], two[1])
    assert float(one[:, 1].abs().max()) > 0  # the transfer part is not trivially zero here
