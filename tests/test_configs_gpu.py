"""The benchmark configurations at their FULL sizes on a B200, checked through size-independent properties:

* a (sequence, key-head group) slice of the call equals the oracle run on that slice alone (chains are independent,
  so the slice of the big call and the small call must agree within the budgets) -- o, every gradient, final state;
* the call repeats bit for bit;
* a batch element computed alone gives the bits it has inside the batch.
"""

from __future__ import annotations

import pytest
import torch

from miles_ext_kernels_b200.workloads import make_workload
from oracle import gdn_oracle as O
from oracle import kda_oracle as K

pytestmark = pytest.mark.gpu
NAMES = ("o", "dq", "dk", "dv", "dg", "dbeta")


def run_gdn(w, *, batch_slice=None):
    from miles_ext_kernels_b200.cake import gdn

    dev = torch.device("cuda")
    sl = slice(None) if batch_slice is None else batch_slice
    t = {n: getattr(w, n)[sl].to(dev).requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
    h0 = w.h0.to(dev).requires_grad_(True) if w.h0 is not None else None
    cu = None if w.cu_seqlens is None else torch.tensor(w.cu_seqlens, dtype=torch.int32, device=dev)
    o, final = gdn.chunk_gated_delta_rule(t["q"], t["k"], t["v"], g=t["g"], beta=t["beta"], initial_state=h0,
                                          output_final_state=w.config.final_state, cu_seqlens=cu,
                                          cu_seqlens_cpu=w.cu_seqlens)
    if final is not None and w.dht is not None:
        torch.autograd.backward([o, final], [w.do[sl].to(dev), w.dht.to(dev)])
    else:
        o.backward(w.do[sl].to(dev))
    torch.cuda.synchronize()
    out = {"o": o.detach(), **{f"d{n}": t[n].grad for n in ("q", "k", "v", "g", "beta")}}
    if final is not None:
        out["final_state"] = final.detach()
    if h0 is not None:
        out["dh0"] = h0.grad
    return out


def check(got, ref, what):
    for name in ref:
        ok, m = O.within_budget(got[name].float().cpu(), ref[name])
        assert ok, (what, name, m)


def test_cfg1_full_size():
    w = make_workload("cfg1")  # B=4, T=8192, H=16, HV=32
    first = run_gdn(w)
    again = run_gdn(w)
    for name in first:
        assert torch.equal(first[name], again[name]), name
    alone = run_gdn(w, batch_slice=slice(2, 3))
    for name in NAMES:
        assert torch.equal(alone[name][0], first[name][2]), f"batch element alone: {name}"
    assert torch.equal(alone["final_state"][0], first["final_state"][2])
    # the oracle on a sequence and a key-head group (hq -> value heads 2 hq, 2 hq + 1): the first, a middle and the
    # last key head, each on another batch element
    for b, hq in ((0, 0), (1, 5), (3, 15)):
        ref = O.chunked_forward_backward(w.q[b, :, hq:hq + 1].float(), w.k[b, :, hq:hq + 1].float(),
                                         w.v[b, :, 2 * hq:2 * hq + 2].float(), w.g[b, :, 2 * hq:2 * hq + 2],
                                         w.beta[b, :, 2 * hq:2 * hq + 2].float(), (w.q.shape[1],),
                                         w.do[b, :, 2 * hq:2 * hq + 2].float(), output_final_state=True)
        got = {"o": first["o"][b, :, 2 * hq:2 * hq + 2], "dq": first["dq"][b, :, hq:hq + 1],
               "dk": first["dk"][b, :, hq:hq + 1], "dv": first["dv"][b, :, 2 * hq:2 * hq + 2],
               "dg": first["dg"][b, :, 2 * hq:2 * hq + 2], "dbeta": first["dbeta"][b, :, 2 * hq:2 * hq + 2],
               "final_state": first["final_state"][b:b + 1, 2 * hq:2 * hq + 2]}
        check(got, ref, f"cfg1 slice b={b} hq={hq}")


def test_cfg2_full_size_varlen_with_states():
    w = make_workload("cfg2")  # 65,536 packed tokens, H = HV = 32, h0 per sequence
    first = run_gdn(w)
    again = run_gdn(w)
    for name in first:
        assert torch.equal(first[name], again[name]), name
    # the shortest and the longest document and one in between; the first, a middle and the last head
    lengths = [b - a for a, b in zip(w.cu_seqlens, w.cu_seqlens[1:])]
    shortest, longest = lengths.index(min(lengths)), lengths.index(max(lengths))
    other = next(n for n in range(len(lengths)) if n not in (shortest, longest))
    for n, h in ((shortest, 0), (other, 17), (longest, 31)):
        lo, hi = w.cu_seqlens[n], w.cu_seqlens[n + 1]
        ref = O.chunked_forward_backward(w.q[0, lo:hi, h:h + 1].float(), w.k[0, lo:hi, h:h + 1].float(),
                                         w.v[0, lo:hi, h:h + 1].float(), w.g[0, lo:hi, h:h + 1],
                                         w.beta[0, lo:hi, h:h + 1].float(), (hi - lo,),
                                         w.do[0, lo:hi, h:h + 1].float(), h0=w.h0[n:n + 1, h:h + 1],
                                         dht=w.dht[n:n + 1, h:h + 1], output_final_state=True)
        got = {name: first[name][0, lo:hi, h:h + 1] for name in NAMES}
        got["final_state"] = first["final_state"][n:n + 1, h:h + 1]
        got["dh0"] = first["dh0"][n:n + 1, h:h + 1]
        check(got, ref, f"cfg2 document {n} ({hi - lo} tokens) head {h}")


def test_cfg4_one_rank_slice_of_the_long_sequence():
    w = make_workload("cfg4")  # one 32,768-token sequence, H = HV = 32
    first = run_gdn(w)
    for h in (0, 13, 31):  # the first, a middle and the last head
        ref = O.chunked_forward_backward(w.q[0, :, h:h + 1].float(), w.k[0, :, h:h + 1].float(),
                                         w.v[0, :, h:h + 1].float(), w.g[0, :, h:h + 1], w.beta[0, :, h:h + 1].float(),
                                         (w.q.shape[1],), w.do[0, :, h:h + 1].float())
        check({name: first[name][0, :, h:h + 1] for name in NAMES}, ref, f"cfg4 slice head {h}")


def test_cfg3_kda_full_size():
    from miles_ext_kernels_b200.cake import kda

    w = make_workload("cfg3")  # one 4,096-token sequence per GPU, H = 32, per-channel gate [1, T, H, 128]
    dev = torch.device("cuda")
    T, H = w.q.shape[1], w.q.shape[2]
    g = w.g[0]
    assert g.shape == (T, H, 128)
    cu = torch.tensor((0, T), dtype=torch.int32, device=dev)

    def once():
        t = {n: getattr(w, n)[0].to(dev).requires_grad_(True) for n in ("q", "k", "v", "beta")}
        gd = g.to(dev).requires_grad_(True)
        o = kda.chunk_kda(t["q"], t["k"], t["v"], gd, t["beta"], cu)
        o.backward(w.do[0].to(dev))
        torch.cuda.synchronize()
        return {"o": o.detach(), "dq": t["q"].grad, "dk": t["k"].grad, "dv": t["v"].grad, "dg": gd.grad,
                "dbeta": t["beta"].grad}

    first, again = once(), once()
    for name in first:
        assert torch.equal(first[name], again[name]), name
    for h in (0, 9, 31):  # the first, a middle and the last head
        ref = K.chunked_forward_backward(w.q[0, :, h:h + 1].float(), w.k[0, :, h:h + 1].float(),
                                         w.v[0, :, h:h + 1].float(), g[:, h:h + 1], w.beta[0, :, h:h + 1].float(), (T,),
                                         w.do[0, :, h:h + 1].float())
        check({name: first[name][:, h:h + 1] for name in NAMES}, ref, f"cfg3 slice head {h}")
