"""The public entry ``cake.gdn.chunk_gated_delta_rule`` on a B200 against the CPU oracle.

Accuracy budgets are the reference's (reference: tests/cake/gdn/test_gdn_det_gpu.py:58-59, 213-223): per output
tensor, relative RMS error <= 1e-2 and largest absolute error <= 2e-2 x the largest reference magnitude, against the
FP64 token recurrence; the FP32 final state and dh0 are held to 8e-3 x their largest magnitude against the FP64
recurrence and to 1e-3 against the chunked FP32-state oracle (the reference's torch path).  Determinism is bitwise.
"""

from __future__ import annotations

import itertools
from pathlib import Path

import pytest
import torch

from gdn_cases import draw
from oracle import gdn_oracle as O

pytestmark = pytest.mark.gpu

NAMES = ("o", "dq", "dk", "dv", "dg", "dbeta")
REF_LAYOUT = (63, 130, 257, 450)


def _cu(seq_lens):
    return tuple(itertools.accumulate(seq_lens, initial=0))


def run(x, seq_lens, *, state=False, l2=True, route="host", views=False, batch=None, **kwargs):
    """One forward + backward through the public entry; outputs and gradients on the host."""
    from miles_ext_kernels_b200.cake import gdn

    dev = torch.device("cuda")
    T = sum(seq_lens)
    H, HV = x["q"].shape[1], x["v"].shape[1]
    lead = (1, T) if batch is None else (batch, T // batch)
    if views:  # miles' packed row: per key head its q, its k, then its value heads
        G = HV // H
        mixed = torch.cat([x["q"], x["k"], x["v"].reshape(T, H, G * 128)], dim=-1).reshape(*lead, -1).to(dev)
        mixed.requires_grad_(True)
        q, k, v = mixed.view(*lead, H, -1).split([128, 128, G * 128], dim=-1)
        v = v.reshape(*lead, HV, 128)
        assert not q.is_contiguous()
    else:
        q, k, v = (x[n].to(dev).reshape(*lead, *x[n].shape[1:]).requires_grad_(True) for n in ("q", "k", "v"))
    g = x["g"].to(dev).reshape(*lead, HV).requires_grad_(True)
    beta = x["beta"].to(dev).bfloat16().reshape(*lead, HV).requires_grad_(True)
    h0 = x["h0"].to(dev).requires_grad_(True) if state else None
    if batch is None:
        kwargs["cu_seqlens"] = torch.tensor(_cu(seq_lens), dtype=torch.int32, device=dev)
        if route == "host":
            kwargs["cu_seqlens_cpu"] = _cu(seq_lens)
    o, final = gdn.chunk_gated_delta_rule(q, k, v, g=g, beta=beta, initial_state=h0, output_final_state=state,
                                          use_qk_l2norm_in_kernel=l2, **kwargs)
    do = x["do"].to(dev).reshape(o.shape)
    if state:
        torch.autograd.backward([o, final], [do, x["dht"].to(dev)])
    else:
        o.backward(do)
    torch.cuda.synchronize()
    if views:
        dq, dk, dv = mixed.grad.view(*lead, H, -1).split([128, 128, (HV // H) * 128], dim=-1)
        dv = dv.reshape(*lead, HV, 128)
    else:
        dq, dk, dv = q.grad, k.grad, v.grad
    flat = lambda t: t.detach().reshape(T, *t.shape[2:]).cpu()  # noqa: E731
    out = {"o": flat(o), "dq": flat(dq), "dk": flat(dk), "dv": flat(dv), "dg": flat(g.grad), "dbeta": flat(beta.grad)}
    if state:
        out.update(final_state=final.detach().cpu(), dh0=h0.grad.cpu())
    return out


def assert_within(got, ref, what, names=NAMES):
    report = {n: O.within_budget(got[n].float(), ref[n]) for n in names}
    failed = [n for n, (ok, _) in report.items() if not ok]
    assert not failed, f"{what}: outside the accuracy budgets: {failed}; {report}"


def assert_same_bits(got, want, what):
    differing = [n for n in want if not torch.equal(got[n], want[n])]
    assert not differing, f"{what}: not the same bits: {differing}"


@pytest.mark.parametrize("heads", [(2, 6), (2, 4), (2, 2)], ids=["2x6", "2x4", "2x2"])
@pytest.mark.parametrize("state", [False, True], ids=["nostate", "state"])
def test_within_the_reference_budgets_of_the_fp64_recurrence(heads, state):
    x = draw(REF_LAYOUT, heads, seed=1, gate="weak", state=state)
    got = run(x, REF_LAYOUT, state=state)
    ref = O.recurrence_fp64(x["q"], x["k"], x["v"], x["g"], x["beta"], REF_LAYOUT, h0=x.get("h0"), do=x["do"],
                            dht=x.get("dht"), use_qk_l2norm=True, output_final_state=state)
    assert_within(got, ref, f"{heads} state={state}")
    if state:
        # fp32 state outputs, two bounds.  Against the FP64 recurrence: 8e-3 of the largest magnitude -- what a
        # path with the reference's BF16 rounding points (w, u, h_tape, v_new stored in BF16) can hold: the
        # reference's own CPU path, restated by the chunked oracle, is 2.4e-3 .. 6.1e-3 away from FP64 on these
        # inputs, so 1e-3 against FP64 is out of reach for it and for any implementation that matches it.  Against
        # the chunked oracle (the reference's torch path, rounding where the kernels round): 1e-3.
        chunked = O.chunked_forward_backward(x["q"], x["k"], x["v"], x["g"], x["beta"], REF_LAYOUT, x["do"].float(),
                                             h0=x["h0"], dht=x["dht"], use_qk_l2norm=True, output_final_state=True)
        for name in ("final_state", "dh0"):
            m64 = O.metrics(got[name], ref[name])
            assert m64["finite"] and m64["max_abs"] <= 8e-3 * m64["max_ref"] and m64["rel_rms"] <= 5e-3, (name, m64)
            m = O.metrics(got[name], chunked[name])
            assert m["finite"] and m["max_abs"] <= 1e-3 * m["max_ref"], (name, m)


def test_strong_gates_of_the_benchmark_generator():
    seq_lens = (257, 320)
    x = draw(seq_lens, (2, 4), seed=2, gate="strong", normalised=True)
    got = run(x, seq_lens, l2=False)
    ref = O.recurrence_fp64(x["q"], x["k"], x["v"], x["g"], x["beta"], seq_lens, do=x["do"])
    assert_within(got, ref, "strong gates")


@pytest.mark.parametrize("path", sorted((Path(__file__).parent / "golden").glob("gdn_fake_backend_*.pt")),
                         ids=lambda p: p.stem)
def test_against_the_reference_emulation_fixtures(path):
    record = torch.load(path)
    i = record["inputs"]
    x = {n: i[n][0] for n in ("q", "k", "v", "do")}
    x["g"], x["beta"] = i["g"][0], i["beta"][0].float()
    got = run(x, record["seq_lens"], l2=record["use_qk_l2norm"])
    want = {n: record["outputs"][n][0].float() for n in NAMES}
    assert_within(got, want, path.stem)


def test_repeats_bit_for_bit_and_views_give_contiguous_bits():
    x = draw(REF_LAYOUT, (2, 4), seed=4, state=True)
    first = run(x, REF_LAYOUT, state=True)
    again = run(x, REF_LAYOUT, state=True)
    assert_same_bits(again, first, "second run")
    views = run(x, REF_LAYOUT, state=True, views=True)
    assert_same_bits(views, first, "strided views of one packed row")


def test_device_boundaries_give_the_host_route_bits():
    x = draw(REF_LAYOUT, (2, 4), seed=5, state=True)
    host = run(x, REF_LAYOUT, state=True, route="host")
    device = run(x, REF_LAYOUT, state=True, route="device")
    assert_same_bits(device, host, "device-built chunk table")


def test_recomputed_state_gives_the_saved_backward_bits():
    import miles_ext_kernels_b200 as package

    x = draw(REF_LAYOUT, (2, 4), seed=6)
    saved = run(x, REF_LAYOUT)
    package.configure(cake_gdn_recompute_state=True)
    recomputed = run(x, REF_LAYOUT)
    assert_same_bits(recomputed, saved, "--cake-gdn-recompute-state")


def test_equal_length_batch():
    seq_lens = (256, 256, 256)
    x = draw(seq_lens, (2, 4), seed=7, state=True)
    got = run(x, seq_lens, state=True, batch=3)
    packed = run(x, seq_lens, state=True)
    assert_same_bits(got, packed, "[B, T] batch vs the same tokens packed")


def test_side_stream_and_pool_give_the_same_bits():
    import miles_ext_kernels_b200 as package

    x = draw(REF_LAYOUT, (2, 4), seed=8)
    want = run(x, REF_LAYOUT)
    package.configure(cake_workspace_pool_bytes=1 << 30)
    side = torch.cuda.Stream()
    for _ in range(2):
        with torch.cuda.stream(side):
            got = run(x, REF_LAYOUT)
        assert_same_bits(got, want, "side stream with the pool")
        assert_same_bits(run(x, REF_LAYOUT), want, "default stream with the pool")
    assert package.release() > 0


def test_a_call_without_tokens():
    from miles_ext_kernels_b200.cake import gdn

    dev = torch.device("cuda")
    q = torch.empty(1, 0, 2, 128, dtype=torch.bfloat16, device=dev, requires_grad=True)
    v = torch.empty(1, 0, 4, 128, dtype=torch.bfloat16, device=dev)
    g = torch.empty(1, 0, 4, device=dev)
    h0 = torch.randn(1, 4, 128, 128, device=dev)
    cu = torch.zeros(2, dtype=torch.int32, device=dev)
    o, final = gdn.chunk_gated_delta_rule(q, q, v, g, g, initial_state=h0, output_final_state=True, cu_seqlens=cu)
    assert o.shape == v.shape and torch.equal(final, h0)


def test_rejections_match_the_reference_messages():
    from miles_ext_kernels_b200.cake import gdn

    dev = torch.device("cuda")
    q = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16, device=dev)
    v = torch.zeros(1, 128, 4, 128, dtype=torch.bfloat16, device=dev)
    g = torch.zeros(1, 128, 4, device=dev)
    cu = torch.tensor([0, 128], dtype=torch.int32, device=dev)
    with pytest.raises(ValueError, match="must end at the 128 tokens of q; it ends at 127"):
        gdn.chunk_gated_delta_rule(q, q, v, g, g, cu_seqlens=cu, cu_seqlens_cpu=(0, 127))
    with pytest.raises(ValueError, match="one state per sequence"):
        gdn.chunk_gated_delta_rule(q, q, v, g, g, cu_seqlens=cu, initial_state=torch.zeros(2, 4, 128, 128, device=dev))
    with pytest.raises(ValueError, match="k must have q's shape"):
        gdn.chunk_gated_delta_rule(q, q[:, :64], v, g, g)
    with pytest.raises(NotImplementedError, match="chunk_size must be 64"):
        gdn.chunk_gated_delta_rule(q, q, v, g, g, chunk_size=32)
    with pytest.raises(NotImplementedError, match="use_gate_in_kernel"):
        gdn.chunk_gated_delta_rule(q, q, v, g, g, use_gate_in_kernel=True)
    with pytest.raises(NotImplementedError, match="bfloat16"):
        gdn.chunk_gated_delta_rule(q.float(), q.float(), v.float(), g, g)


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64], ids=["int32", "int64"])
def test_the_chunk_table_kernel_gives_the_torch_route_tables(dtype):
    """The device route's one-launch table kernel against the same tables built by torch integer ops on the host
    copy, pad chunks included: ragged, empty and single-token sequences, and more sequences than threads."""
    from miles_ext_kernels_b200.cake._impl.gdn import meta as meta_module

    gen = torch.Generator().manual_seed(3)
    layouts = [(64,), (1,), (63, 65, 0, 128, 1), (300, 0, 0, 724), tuple(int(n) for n in torch.randint(0, 200, (1500,), generator=gen))]
    for seq_lens in layouts:
        cu = torch.tensor([0, *torch.tensor(seq_lens).cumsum(0).tolist()], dtype=dtype)
        total = int(cu[-1])
        want = meta_module._from_device(cu, total)
        got = meta_module._from_device(cu.cuda(), total)
        assert (got.num_chunks, got.num_seqs, got.total_tokens, got.exact) == (want.num_chunks, want.num_seqs, total, False)
        for name in ("chunk_start", "chunk_len", "chunk_seq", "seq_chunk_start"):
            assert torch.equal(getattr(got, name).cpu(), getattr(want, name)), (seq_lens[:8], name)


def test_forward_and_backward_replay_from_a_cuda_graph():
    """The op is capturable: no host synchronisation, no allocation outside torch's capture-aware allocator, tensor
    maps travel as kernel parameters.  A replay on new inputs written into the captured buffers gives the bits of an
    eager call on those inputs."""
    import miles_ext_kernels_b200 as package
    from miles_ext_kernels_b200.cake import gdn

    dev = torch.device("cuda")
    seq_lens = (200, 312)
    cu = _cu(seq_lens)
    first, second = (draw(seq_lens, (2, 4), seed=s) for s in (41, 42))
    want = run(second, seq_lens)
    static = {n: first[n].to(dev).unsqueeze(0).clone() for n in ("q", "k", "v", "g", "do")}
    static["beta"] = first["beta"].to(dev).bfloat16().unsqueeze(0).clone()
    cu_dev = torch.tensor(cu, dtype=torch.int32, device=dev)

    def step():
        leaves = {n: static[n].detach().requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
        o, _ = gdn.chunk_gated_delta_rule(leaves["q"], leaves["k"], leaves["v"], g=leaves["g"], beta=leaves["beta"],
                                          cu_seqlens=cu_dev, cu_seqlens_cpu=cu, use_qk_l2norm_in_kernel=True)
        o.backward(static["do"])
        return [o.detach()] + [leaves[n].grad for n in ("q", "k", "v", "g", "beta")]

    package.configure(cake_workspace_pool_bytes=1 << 28)  # the pool is bypassed while capturing
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                step()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            outs = step()
        for n in ("q", "k", "v", "g", "do"):
            static[n].copy_(second[n].to(dev).unsqueeze(0))
        static["beta"].copy_(second["beta"].to(dev).bfloat16().unsqueeze(0))
        graph.replay()
        torch.cuda.synchronize()
    finally:
        package.configure()
    got = dict(zip(NAMES, (t[0].cpu() for t in outs)))
    assert_same_bits(got, {n: want[n] for n in NAMES}, "graph replay")


@pytest.mark.parametrize("l2", [True, False], ids=["l2norm", "plain"])
@pytest.mark.parametrize("split", ["packed_qkv_views", "torch_split"])
@pytest.mark.parametrize("segments", [0, 2], ids=["serial_scans", "segmented_scans"])
def test_views_of_one_packed_row_are_read_in_place_and_give_the_contiguous_bits(l2, split, segments):
    """q, k, v as the column slices [q heads | k heads | v heads] of one packed row: no copy on the way in (the
    kernels take the token stride), one packed gradient row on the way out, the bits of contiguous operands --
    also when the scans are cut into segments (the segments' extents keep the operands' strides)."""
    import miles_ext_kernels_b200 as package
    from miles_ext_kernels_b200.cake import gdn
    from miles_ext_kernels_b200.cake._impl.gdn import ops

    dev = torch.device("cuda")
    B, T, (H, HV) = 2, (2304 if segments else 448), (2, 4)
    seq_lens = (T,) * B
    x = draw(seq_lens, (H, HV), seed=51, normalised=not l2)
    package.configure(cake_gdn_scan_segments=segments)
    try:
        _packed_row_case(x, seq_lens, l2, split, B, T, H, HV, dev, gdn, ops)
    finally:
        package.configure()


def _packed_row_case(x, seq_lens, l2, split, B, T, H, HV, dev, gdn, ops):
    want = run(x, seq_lens, l2=l2, batch=B)
    row = torch.cat([x["q"].reshape(B * T, -1), x["k"].reshape(B * T, -1), x["v"].reshape(B * T, -1)], dim=-1)
    row = row.reshape(B, T, -1).to(dev).requires_grad_(True)
    if split == "packed_qkv_views":
        q, k, v = gdn.packed_qkv_views(row, H, HV)
    else:
        q, k, v = row.split([H * 128, H * 128, HV * 128], dim=-1)
        q, k, v = q.unflatten(-1, (H, 128)), k.unflatten(-1, (H, 128)), v.unflatten(-1, (HV, 128))
    assert not q.is_contiguous() and ops._rows(q).data_ptr() == q.data_ptr()  # read where it lies
    assert ops._rows(v).data_ptr() == v.data_ptr() and ops._tile_one_row(ops._rows(q), ops._rows(k), ops._rows(v))
    g = x["g"].to(dev).reshape(B, T, HV).requires_grad_(True)
    beta = x["beta"].to(dev).bfloat16().reshape(B, T, HV).requires_grad_(True)
    o, _ = gdn.chunk_gated_delta_rule(q, k, v, g=g, beta=beta, use_qk_l2norm_in_kernel=l2)
    o.backward(x["do"].to(dev).reshape(o.shape))
    torch.cuda.synchronize()
    flat = lambda t: t.detach().reshape(B * T, *t.shape[2:]).cpu()  # noqa: E731
    grad = flat(row.grad)
    got = {"o": flat(o), "dq": grad[:, : H * 128].reshape(-1, H, 128), "dk": grad[:, H * 128 : 2 * H * 128].reshape(-1, H, 128),
           "dv": grad[:, 2 * H * 128 :].reshape(-1, HV, 128), "dg": flat(g.grad), "dbeta": flat(beta.grad)}
    assert_same_bits(got, {n: want[n] for n in NAMES}, f"packed row, {split}")
    with pytest.raises(ValueError, match="columns"):
        gdn.packed_qkv_views(row[..., :-128], H, HV)


def test_the_tape_goes_through_autograd_saved_tensors():
    """Every tensor the backward reads is kept with ``save_for_backward``: an in-place write to an operand between
    forward and backward is caught by autograd's version check instead of giving silently wrong gradients, and a
    saved-tensor hook (what activation checkpointing and CPU offload use) sees the whole tape."""
    from miles_ext_kernels_b200.cake import gdn

    dev = torch.device("cuda")
    seq_lens = (70, 130)
    x = draw(seq_lens, (2, 4), seed=6, normalised=True)  # the call below does not normalise q / k itself
    cu = _cu(seq_lens)

    def call():
        t = {n: x[n].unsqueeze(0).to(dev).requires_grad_(True) for n in ("q", "k", "v", "g")}
        beta = x["beta"].unsqueeze(0).to(dev).bfloat16().requires_grad_(True)
        o, _ = gdn.chunk_gated_delta_rule(t["q"], t["k"], t["v"], g=t["g"], beta=beta,
                                          cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=dev), cu_seqlens_cpu=cu)
        return t, o

    t, o = call()
    with torch.no_grad():
        t["q"].mul_(2.0)
    # autograd words it in one of two ways, depending on whether the saved tensor is the operand or a view of it
    with pytest.raises(RuntimeError, match="modified (by an )?inplace"):
        o.backward(x["do"].unsqueeze(0).to(dev))

    seen = []

    def pack(tensor):
        seen.append(tensor.numel() * tensor.element_size())
        return tensor

    with torch.autograd.graph.saved_tensors_hooks(pack, lambda tensor: tensor):
        t, o = call()
    o.backward(x["do"].unsqueeze(0).to(dev))
    torch.cuda.synchronize()
    T, H, HV = sum(seq_lens), 2, 4
    chunks = sum(-(-n // 64) for n in seq_lens)
    # q, k, v, w, u, v_new rows; A, Aqk and the h tape per chunk; the gate and beta columns
    floor = 2 * T * H * 256 + 4 * T * HV * 256 + chunks * HV * (2 * 8192 + 32768) + 2 * T * HV * 4
    assert sum(seen) >= floor, (sum(seen), floor, seen)
    assert t["q"].grad is not None and torch.isfinite(t["q"].grad.float()).all()
