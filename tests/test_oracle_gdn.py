"""The CPU oracle pinned: its chunked restatement and its FP64 recurrence against outputs of the reference's own torch
emulation (``tests/golden/gdn_fake_backend_*.pt``, made by ``tests/golden/make_gdn_golden.py``), and against each
other on the edge cases the reference tests (ragged lengths, partial chunks, initial / final state, GVA heads)."""

from __future__ import annotations

from pathlib import Path

import pytest
import torch

from oracle import gdn_oracle as O

GOLDEN = sorted((Path(__file__).parent / "golden").glob("gdn_fake_backend_*.pt"))
NAMES = ("o", "dq", "dk", "dv", "dg", "dbeta")


def _flat(record):
    i = record["inputs"]
    return {n: i[n][0].float() for n in ("q", "k", "v", "g", "beta", "do")}


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_chunked_oracle_matches_the_reference_emulation(path):
    record = torch.load(path)
    x = _flat(record)
    got = O.chunked_forward_backward(x["q"], x["k"], x["v"], x["g"], x["beta"], record["seq_lens"], x["do"],
                                     use_qk_l2norm=record["use_qk_l2norm"])
    for name in NAMES:
        want = record["outputs"][name][0].float()
        have = got[name]
        if name == "dbeta":  # the reference returns dbeta in beta's dtype (bf16)
            have = have.bfloat16().float()
        m = O.metrics(have, want)
        # same algorithm, same rounding points: only FP32 summation order differs, which can flip a BF16 rounding
        assert m["finite"] and m["rel_rms"] <= 1e-3 and m["max_abs"] <= 8e-3 * m["max_ref"], (name, m)


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_fp64_recurrence_matches_the_reference_emulation_within_its_budgets(path):
    record = torch.load(path)
    x = _flat(record)
    ref = O.recurrence_fp64(x["q"], x["k"], x["v"], x["g"], x["beta"], record["seq_lens"], do=x["do"],
                            use_qk_l2norm=record["use_qk_l2norm"])
    for name in NAMES:
        ok, m = O.within_budget(record["outputs"][name][0].float(), ref[name])
        assert ok, (name, m)


def test_chunked_oracle_matches_the_reference_cpu_path_run_live():
    """Where ``oracle/_ref`` (the files of the reference's own CPU path, put there by ``oracle/make_ref.py``) is at
    hand, the restatement is checked against the reference itself on inputs the stored fixtures do not hold: the
    benchmark's strong gates on GVA heads with a ragged layout."""
    from oracle import reference_arm

    if not reference_arm.available():
        pytest.skip("oracle/_ref is absent (no reference checkout on this machine)")
    from gdn_cases import draw

    seq_lens = (65, 200, 31)
    cu = (0, 65, 265, 296)
    x = draw(seq_lens, (2, 4), seed=21, gate="strong", normalised=True)
    want = reference_arm.forward_backward(x["q"], x["k"], x["v"], x["g"], x["beta"].bfloat16(), x["do"], cu)
    got = O.chunked_forward_backward(x["q"].float(), x["k"].float(), x["v"].float(), x["g"], x["beta"], seq_lens,
                                     x["do"].float())
    for name in NAMES:
        have = got[name].bfloat16().float() if name == "dbeta" else got[name]
        m = O.metrics(have, want[name].float())
        assert m["finite"] and m["rel_rms"] <= 1e-3 and m["max_abs"] <= 8e-3 * m["max_ref"], (name, m)


CASES = {
    "single_token": ((1,), (1, 1), False),
    "ragged": ((1, 63, 64, 65, 130), (2, 4), True),
    "state": ((70, 129), (1, 2), True),
    "mha_nostate": ((200,), (2, 2), False),
}


@pytest.mark.parametrize("name", list(CASES))
def test_chunked_algorithm_is_the_recurrence_in_fp32(name):
    seq_lens, (H, HV), state = CASES[name]
    gen = torch.Generator().manual_seed(5)
    T = sum(seq_lens)
    q, k = torch.randn(T, H, 128, generator=gen), torch.randn(T, H, 128, generator=gen)
    v, do = torch.randn(T, HV, 128, generator=gen), torch.randn(T, HV, 128, generator=gen)
    g, beta = -0.5 * torch.rand(T, HV, generator=gen), torch.rand(T, HV, generator=gen)
    h0 = 0.1 * torch.randn(len(seq_lens), HV, 128, 128, generator=gen) if state else None
    dht = 0.1 * torch.randn(len(seq_lens), HV, 128, 128, generator=gen) if state else None
    ref = O.recurrence_fp64(q, k, v, g, beta, seq_lens, h0=h0, do=do, dht=dht, use_qk_l2norm=True,
                            output_final_state=state)
    got = O.chunked_forward_backward(q, k, v, g, beta, seq_lens, do, h0=h0, dht=dht, use_qk_l2norm=True,
                                     rounding=None, output_final_state=state)
    assert set(got) == set(ref)
    for key in got:
        m = O.metrics(got[key], ref[key])
        assert m["finite"] and m["max_abs"] <= 2e-5 * max(m["max_ref"], 1e-3), (key, m)


def test_config0_fp32_small_heads():
    """The CPU plumbing configuration: B=1, T=256, H=HV=4, dk=dv=64, fp32, strong gates, zero initial state."""
    gen = torch.Generator().manual_seed(0)
    T, H, d = 256, 4, 64
    q, k = torch.randn(T, H, d, generator=gen), torch.randn(T, H, d, generator=gen)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6)
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    v = torch.randn(T, H, d, generator=gen)
    beta = torch.sigmoid(torch.randn(T, H, generator=gen))
    a, u = torch.randn(T, H, generator=gen), torch.rand(T, H, generator=gen)
    g = -torch.nn.functional.softplus(a) * torch.exp(u * torch.log(torch.tensor(16.0)))
    do = torch.randn(T, H, d, generator=gen)
    ref = O.recurrence_fp64(q, k, v, g, beta, (T,), do=do)
    got = O.chunked_forward_backward(q, k, v, g, beta, (T,), do, rounding=None)
    for key in got:
        m = O.metrics(got[key], ref[key])
        assert m["finite"] and m["max_abs"] <= 2e-5 * max(m["max_ref"], 1e-3), (key, m)


def test_config0_workload_through_both_oracles():
    """The benchmark's configuration 0 as ``make_workload`` draws it (fp32, dk = dv = 64): the chunked oracle without
    rounding agrees with the FP64 recurrence.  It is an oracle-only configuration: the product, like the reference's
    kernels (reference: miles_ext_kernels/cake/_impl/gdn/ops.py:2307-2310), serves head dims of 128 in bf16 only."""
    from miles_ext_kernels_b200.workloads import make_workload

    w = make_workload("cfg0")
    assert w.q.dtype == torch.float32 and w.q.shape == (1, 256, 4, 64) and w.v.shape == (1, 256, 4, 64)
    args = (w.q[0], w.k[0], w.v[0], w.g[0], w.beta[0], (256,))
    ref = O.recurrence_fp64(*args, do=w.do[0])
    got = O.chunked_forward_backward(*args, w.do[0], rounding=None)
    for key in got:
        m = O.metrics(got[key], ref[key])
        assert m["finite"] and m["max_abs"] <= 2e-5 * max(m["max_ref"], 1e-3), (key, m)


def test_chunk_table_never_straddles_sequences():
    table = O.chunk_table((1, 63, 64, 65, 130))
    assert table.chunk_len == (1, 63, 64, 64, 1, 64, 64, 2)
    assert table.seq_chunk_start == (0, 1, 2, 3, 5, 8)
    assert table.chunk_start == (0, 1, 64, 128, 192, 193, 257, 321)
    assert table.chunk_seq == (0, 1, 2, 3, 3, 4, 4, 4)
