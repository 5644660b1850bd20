"""Every forward and backward stage of the CUDA path against the CPU oracle's tape of the same stage, on ragged
packed sequences (lengths 1, 63, 64, 65, 130: empty tail rows, full chunks, a chunk boundary, a multi-chunk scan)."""

from __future__ import annotations

import math

import pytest
import torch

from gdn_cases import draw, to_token_major
from oracle import gdn_oracle as O

pytestmark = pytest.mark.gpu

LOG2E = 1.4426950408889634


def close(got, want, name, rel_rms=4e-3, max_rel=2e-2):
    m = O.metrics(got.float().cpu(), want.float())
    assert m["finite"], (name, m)
    assert m["rel_rms"] <= rel_rms and m["max_abs"] <= max_rel * max(m["max_ref"], 1e-6), (name, m)


CASES = {
    "ragged_gva_state": ((1, 63, 64, 65, 130), (2, 4), "weak", True, True),
    "mha_strong": ((200, 64), (2, 2), "strong", False, False),
    "long_scan": ((700,), (1, 2), "weak", False, True),
}


@pytest.mark.parametrize("name", list(CASES))
def test_forward_stages(name):
    from miles_ext_kernels_b200.cake._impl.gdn import meta as M
    from miles_ext_kernels_b200.cake._impl.gdn import stages

    seq_lens, heads, gate, state, l2 = CASES[name]
    x = draw(seq_lens, heads, seed=3, gate=gate, state=state, normalised=not l2)
    dev = torch.device("cuda")
    cu = [0]
    for n in seq_lens:
        cu.append(cu[-1] + n)
    meta = M.chunk_meta(torch.tensor(cu, dtype=torch.int32, device=dev), tuple(cu), 1, cu[-1], dev)
    scale = 1.0 / math.sqrt(128)
    d = {n: t.to(dev) for n, t in x.items()}
    o, final, tape, _ = stages.forward(d["q"], d["k"], d["v"], d["g"], d["beta"], meta, scale, d.get("h0"), state, l2)
    torch.cuda.synchronize()
    stages.check_status(tape.status)

    o_ref, final_ref, t = O.chunked_forward(x["q"], x["k"], x["v"], x["g"], x["beta"], seq_lens, h0=x.get("h0"),
                                            use_qk_l2norm=l2, output_final_state=state)
    table = t.table
    if l2:
        close(tape.qn, to_token_major(t.q, table), "qn", rel_rms=1e-3)
        close(tape.kn, to_token_major(t.k, table), "kn", rel_rms=1e-3)
        close(tape.rstd_q.unsqueeze(-1), t.q_rstd, "rstd_q", rel_rms=1e-5, max_rel=1e-5)
    close(tape.g_cs, to_token_major(t.G, table) * LOG2E, "g_cs", rel_rms=1e-5, max_rel=1e-4)
    close(tape.aqk, t.Aqk, "Aqk")
    close(tape.a, t.A, "A")
    close(tape.w, to_token_major(t.w, table), "w")
    close(tape.u, to_token_major(t.u, table), "u")
    close(tape.h, t.h, "h")
    close(tape.v_new, to_token_major(t.v_new, table), "v_new")
    close(o, o_ref, "o")
    if state:
        close(final, final_ref, "final_state", rel_rms=3e-3, max_rel=1e-2)


@pytest.mark.parametrize("name", list(CASES))
def test_backward_stages(name):
    from miles_ext_kernels_b200.cake._impl.gdn import meta as M
    from miles_ext_kernels_b200.cake._impl.gdn import stages

    seq_lens, heads, gate, state, l2 = CASES[name]
    x = draw(seq_lens, heads, seed=3, gate=gate, state=state, normalised=not l2)
    dev = torch.device("cuda")
    cu = [0]
    for n in seq_lens:
        cu.append(cu[-1] + n)
    meta = M.chunk_meta(torch.tensor(cu, dtype=torch.int32, device=dev), tuple(cu), 1, cu[-1], dev)
    scale = 1.0 / math.sqrt(128)
    d = {n: t.to(dev) for n, t in x.items()}
    o, final, tape, _ = stages.forward(d["q"], d["k"], d["v"], d["g"], d["beta"], meta, scale, d.get("h0"), state, l2)
    seen = {}
    dq, dk, dv, dg, dbeta, dh0 = stages.backward(tape, meta, scale, d["do"], d.get("dht"), d.get("h0"), state,
                                                 inspect=seen)
    dh_tape, dv_new = seen["dh_tape"], seen["dv_new"]
    torch.cuda.synchronize()
    stages.check_status(tape.status)

    _, _, t = O.chunked_forward(x["q"], x["k"], x["v"], x["g"], x["beta"], seq_lens, h0=x.get("h0"),
                                use_qk_l2norm=l2, output_final_state=state)
    ref = O.chunked_backward(t, x["do"].float(), dht=x.get("dht"))
    close(dh_tape, ref["dh_tape"], "dh_tape")
    close(dv_new, to_token_major(ref["dv_new"], t.table), "dv_new")
    if state:
        close(dh0, ref["dh0"], "dh0", rel_rms=3e-3, max_rel=1e-2)
    close(dv, ref["dv"], "dv")
    close(dq, ref["dq"], "dq")
    close(dk, ref["dk"], "dk")
    close(dbeta, ref["dbeta"], "dbeta")
    close(dg, ref["dg"], "dg")
