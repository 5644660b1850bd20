"""Packed causal depthwise conv1d + SiLU: the oracle against the reference's own FP64 outputs (CPU), the op's
argument surface (CPU), and the kernels against the oracle under the reference's gates -- y and dx within
``1e-3 + 2^-7 |ref|``, the weight gradient within ``5e-2 + 1e-4 |ref|`` (bf16 policy) or ``1e-3 + 2e-6 |ref|`` (fp32
policy; BF16 taps: one BF16 ulp) of the FP64 sum (GPU) (reference: tests/cake/conv1d/test_conv1d_gpu.py:40-260)."""

from __future__ import annotations

from pathlib import Path

import pytest
import torch

from oracle import conv1d_oracle as C

GOLDEN = sorted((Path(__file__).parent / "golden").glob("conv1d_reference_*.pt"))
Y_ATOL, Y_RTOL = 1e-3, 2**-7
DW_ATOL, DW_RTOL = 5e-2, 1e-4
DW_FP32G_ATOL, DW_FP32G_RTOL = 1e-3, 2e-6
PERF_FRACTIONS = (0.37, 0.29, 0.21)


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_the_oracle_reproduces_the_reference_fp64_outputs(path):
    rec = torch.load(path)
    got = C.reference(rec["x"], rec["w"], rec["cu"], rec["dy"], "fp32")
    assert torch.equal(got["y"], rec["y"]) and torch.equal(got["dx"], rec["dx"])
    assert C.outside(got["dw"], rec["dw"], atol=1e-12, rtol=1e-12) == 0
    rounded = C.reference(rec["x"], rec["w"], rec["cu"], rec["dy"], "bf16")  # the other policy stays within the gates
    assert C.outside(rounded["y"], rec["y"], atol=Y_ATOL, rtol=Y_RTOL) == 0
    assert C.outside(rounded["dx"], rec["dx"], atol=2e-2, rtol=2**-6) == 0


def test_the_op_declaration_and_its_checks():
    import miles_ext_kernels_b200 as package
    from miles_ext_kernels_b200 import cake
    from miles_ext_kernels_b200.cake import conv1d

    op = cake.op_spec("conv1d")
    assert op.variants == ("det", "fast") and op.selected_by == (("linear_attention_conv_backend", "cake"),)
    assert set(op.exports) == {"causal_conv1d", "causal_conv1d_kcp", "causal_conv1d_kcp_multi", "check_supported"}
    assert cake.option("conv1d", "cake_conv1d_silu_grad_preactivation") == "bf16"
    package.configure(cake_conv1d_silu_grad_preactivation="fp32")
    assert cake.option("conv1d", "cake_conv1d_silu_grad_preactivation") == "fp32"
    package.configure()
    with pytest.raises(ValueError, match="kernel size 4"):
        conv1d.check_supported(512, 3, "silu")
    with pytest.raises(ValueError, match="SiLU"):
        conv1d.check_supported(512, 4, "gelu")
    with pytest.raises(ValueError, match="without a bias"):
        conv1d.check_supported(512, 4, "silu", has_bias=True)
    with pytest.raises(ValueError, match="multiple of 8"):
        conv1d.check_supported(516, 4, "silu")
    with pytest.raises(TypeError, match="one tensor and its taps"):
        conv1d.causal_conv1d_kcp([torch.zeros(4, 8)], torch.zeros(8, 4), None)
    with pytest.raises(TypeError, match="sequences of tensors"):
        conv1d.causal_conv1d_kcp_multi(torch.zeros(4, 8), [torch.zeros(8, 4)], None)


def test_the_rows_a_cut_reaches_across():
    from miles_ext_kernels_b200.cake._impl.gdn.kcp import halo_rows

    cu = (0, 7, 9, 30, 40)  # cuts at 10, 20, 30 in a world of 4
    assert halo_rows(cu, 0, 4, 3) == (0, 3)   # tokens 10..12 of the third document follow
    assert halo_rows(cu, 1, 4, 3) == (1, 3)   # the third document began at 9: one row of history
    assert halo_rows(cu, 2, 4, 3) == (3, 0)   # a document ends at the cut
    assert halo_rows(cu, 3, 4, 3) == (0, 0)
    assert halo_rows((0, 11, 40), 0, 4, 3) == (0, 1)  # one token of the first document past the cut
    assert halo_rows((0, 40), 2, 4, 3) == (3, 3)


def _halo_rank(rank, world, port, out_dir):
    import os

    import torch.distributed as dist

    from miles_ext_kernels_b200.cake._impl.gdn.kcp import KcpContext

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ctx = KcpContext((0, 15, 20, 30), None, rank, world, "cpu")  # cuts at 10 (inside a document) and 20 (between two)
    rows = torch.arange(30 * 4, dtype=torch.float32).view(30, 4)[rank * 10:(rank + 1) * 10]
    exchange = ctx.halo_exchange()
    (prev,), (nxt,) = exchange.forward(rows[None, :3].clone(), rows[None, -3:].clone())  # one span per rank
    (back,) = exchange.backward(-rows[None, :3].clone())
    # the same rows through the all-gather exchange of the other layouts
    from miles_ext_kernels_b200.cake._impl.gdn.kcp import _GatherHalo

    (prev2,), (nxt2,) = _GatherHalo(ctx).forward(rows[None, :3].clone(), rows[None, -3:].clone())
    same = all((a is None and b is None) or torch.equal(a, b) for a, b in ((prev, prev2), (nxt, nxt2)))
    torch.save({"halo": ctx.halo, "prev": prev, "next": nxt, "back": back, "same": same}, f"{out_dir}/rank{rank}.pt")
    dist.barrier()
    dist.destroy_process_group()


def test_neighbours_exchange_rows_only_across_cut_documents(tmp_path):
    """World of 3 over gloo: rows cross the first cut in both directions, nothing crosses the second."""
    import socket

    import torch.multiprocessing as mp

    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    mp.spawn(_halo_rank, args=(3, port, str(tmp_path)), nprocs=3, join=True)
    full = torch.arange(30 * 4, dtype=torch.float32).view(30, 4)
    got = [torch.load(tmp_path / f"rank{r}.pt") for r in range(3)]
    assert [g["halo"] for g in got] == [(0, 3), (3, 0), (0, 0)] and all(g["same"] for g in got)
    assert got[0]["prev"] is None and torch.equal(got[0]["next"], full[10:13])
    assert torch.equal(got[0]["back"], -full[10:13])
    assert torch.equal(got[1]["prev"], full[7:10]) and got[1]["next"] is None and got[1]["back"] is None
    assert got[2]["prev"] is None and got[2]["next"] is None and got[2]["back"] is None


# (S, C, documents): documents of 1-3 tokens and empty ones, run boundaries, channel counts that are not multiples
# of a warp's 256 or of a block's 2048, and the framework's per-rank channel counts
CASES = (
    (5, 136, (2, 0, 3)),
    (63, 384, (1, 2, 3, 57)),
    (1000, 512, "perf"),
    (4097, 1280, (1000, 0, 3, 3094)),
    (4097, 2560, (1000, 0, 3, 3094)),
    (32771, 8192, (1, 2, 3, 0, 9000, 3, 23762)),
)


def doc_lengths(S, docs):
    if docs == "perf":
        lens = []
        for fraction in PERF_FRACTIONS:
            n = int(fraction * S)
            lens.append(n - 1 if n % 64 == 0 else n)
        return (*lens, S - sum(lens))
    assert sum(docs) == S
    return tuple(docs)


def inputs(S, channels, docs, taps):
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed((2033 * 1_000_003 + S * 7919 + channels * 31) % (2**31 - 1))
    x = torch.randn(1, S, channels, device=dev, generator=gen).bfloat16()
    w = (0.5 * torch.randn(channels, 4, device=dev, generator=gen)).to(taps)
    dy = torch.randn(1, S, channels, device=dev, generator=gen).bfloat16()
    lens = doc_lengths(S, docs)
    cu = torch.tensor([0, *torch.tensor(lens).cumsum(0).tolist()], dtype=torch.int32, device=dev)
    return x, w, cu, dy


def run(x, w, cu, dy, policy=None, weight_grad=True):
    from miles_ext_kernels_b200.cake.conv1d import causal_conv1d

    xi, wi = x.detach().requires_grad_(True), w.detach().requires_grad_(weight_grad)
    y = causal_conv1d(xi, wi, cu, silu_grad_preactivation=policy)
    assert y.dtype == torch.bfloat16 and y.shape == x.shape
    y.backward(dy)
    return {"y": y.detach(), "dx": xi.grad, "dw": wi.grad}


@pytest.mark.gpu
@pytest.mark.parametrize("taps", [torch.float32, torch.bfloat16], ids=["fp32_taps", "bf16_taps"])
@pytest.mark.parametrize("policy", ["bf16", "fp32"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: f"s{c[0]}_c{c[1]}")
def test_within_the_reference_gates_of_the_fp64_sums(case, policy, taps):
    S, channels, docs = case
    if S > 5000 and (taps == torch.bfloat16 or policy == "fp32"):
        pytest.skip("the large case runs once")
    x, w, cu, dy = inputs(S, channels, docs, taps)
    got = run(x, w, cu, dy, policy)
    ref = C.reference(x[0].cpu(), w.cpu(), cu.cpu(), dy[0].cpu(), policy)
    assert C.outside(got["y"][0].cpu(), ref["y"], atol=Y_ATOL, rtol=Y_RTOL) == 0
    assert C.outside(got["dx"][0].cpu(), ref["dx"], atol=Y_ATOL if policy == "fp32" else 2e-3, rtol=Y_RTOL) == 0
    atol, rtol = (DW_ATOL, DW_RTOL) if policy == "bf16" else (DW_FP32G_ATOL, DW_FP32G_RTOL)
    if taps == torch.bfloat16:
        atol, rtol = atol * (1 + 2**-8), 2**-7
    assert got["dw"].dtype == taps and C.outside(got["dw"].cpu(), ref["dw"], atol=atol, rtol=rtol) == 0
    again = run(x, w, cu, dy, policy)
    for name in got:
        assert torch.equal(got[name], again[name]), name  # fixed-order sums: the same bits
    assert run(x, w, cu, dy, policy, weight_grad=False)["dw"] is None


@pytest.mark.gpu
def test_one_document_without_boundaries_and_the_2d_form():
    from miles_ext_kernels_b200.cake.conv1d import causal_conv1d

    x, w, cu, dy = inputs(777, 256, (777,), torch.float32)
    with_cu = run(x, w, cu, dy)
    without = run(x, w, None, dy)
    flat = run(x[0], w, None, dy[0])
    for name in ("y", "dx", "dw"):
        assert torch.equal(with_cu[name], without[name]), name
        assert torch.equal(flat[name].view_as(without[name]), without[name]), name
    with pytest.raises(ValueError, match="one packed batch"):
        causal_conv1d(x.expand(2, -1, -1), w)
    with pytest.raises(ValueError, match="multiple of 8"):
        causal_conv1d(x[..., :100], w[:100])


def _cut_context(cu, rank, world, full_xs, full_dys, layout="contiguous"):
    """A rank's ``KcpContext`` whose neighbour exchange reads the undivided tensors (ranks emulated one after another
    on one GPU)."""
    from miles_ext_kernels_b200.cake._impl.gdn.kcp import KcpContext

    class Cut(KcpContext):
        exchanges = 0

        def rows(self, tensors, doc, at):
            """Rows ``at .. at + 3`` of document ``doc`` (zeros outside the batch)."""
            lo = cu[doc] + at
            out = torch.zeros(3, sum(t.shape[1] for t in tensors), dtype=tensors[0].dtype, device=tensors[0].device)
            a, b = max(lo, 0), min(lo + 3, tensors[0].shape[0])
            if b > a:
                out[a - lo : b - lo] = torch.cat([t[a:b] for t in tensors], dim=1)
            return out

        def halo_exchange(self):
            ctx = self

            class Loopback:
                def forward(self, first, last):
                    ctx.exchanges += 1
                    heads = [ctx.fragments[sp.first] for sp in ctx.plan.spans]
                    tails = [ctx.fragments[sp.last] for sp in ctx.plan.spans]
                    for i, (h, t) in enumerate(zip(heads, tails)):
                        assert torch.equal(first[i], ctx.rows(full_xs, h.doc, h.offset))
                        assert torch.equal(last[i], ctx.rows(full_xs, t.doc, t.end - 3))
                    prev = [None if sp.prev is None else ctx.rows(full_xs, h.doc, h.offset - 3)
                            for sp, h in zip(ctx.plan.spans, heads)]
                    nxt = [None if sp.next is None else ctx.rows(full_xs, t.doc, t.end)
                           for sp, t in zip(ctx.plan.spans, tails)]
                    return prev, nxt

                def backward(self, first):
                    tails = [ctx.fragments[sp.last] for sp in ctx.plan.spans]
                    return [None if sp.next is None else ctx.rows(full_dys, t.doc, t.end)
                            for sp, t in zip(ctx.plan.spans, tails)]

            return Loopback()

        def take(self, full):
            """This rank's tokens of an undivided ``[S, ...]`` tensor, in local order."""
            return torch.cat([full[cu[f.doc] + f.offset : cu[f.doc] + f.end] for f in self.fragments])

        def scatter(self, full, local):
            at = 0
            for f in self.fragments:
                full[cu[f.doc] + f.offset : cu[f.doc] + f.end] = local[at : at + f.length]
                at += f.length

    return Cut(cu, None, rank, world, "cuda", layout=layout)


@pytest.mark.gpu
@pytest.mark.parametrize("policy", ["bf16", "fp32"])
@pytest.mark.parametrize("world,lens,layout", [
    (2, (300, 724), "contiguous"), (4, (1, 2, 253, 1, 2, 509, 256), "contiguous"), (4, (1024,), "contiguous"),
    (8, (130, 126, 2, 766), "contiguous"), (2, (300, 724), "zigzag"), (4, (1, 2, 253, 1, 2, 509, 256), "zigzag"),
    (4, (1024,), "zigzag"), (2, (256, 64, 704), "zigzag_per_document"), (4, (512, 512), "zigzag_per_document"),
])
def test_the_cut_route_gives_the_bits_of_the_undivided_call(world, lens, layout, policy):
    """y and dx of every rank's tokens are the undivided call's; the ranks' weight-gradient partials add up to its
    weight gradient within the gate; two tensors through one exchange equal two calls."""
    import miles_ext_kernels_b200 as package
    from miles_ext_kernels_b200.cake.conv1d import causal_conv1d_kcp, causal_conv1d_kcp_multi

    S = sum(lens)
    x, w, cu, dy = inputs(S, 384, lens, torch.float32)
    x2, w2, _, dy2 = inputs(S, 136, lens, torch.bfloat16)
    package.configure(cake_conv1d_silu_grad_preactivation=policy)
    try:
        want, want2 = run(x, w, cu, dy, policy), run(x2, w2, cu, dy2, policy)
        cu_host = tuple(cu.tolist())
        got = {n: torch.zeros_like(x[0]) for n in ("y", "dx")} | {n: torch.zeros_like(x2[0]) for n in ("y2", "dx2")}
        dws = []
        for rank in range(world):
            ctx = _cut_context(cu_host, rank, world, [x[0], x2[0]], [dy[0], dy2[0]], layout)
            xa, xb = ctx.take(x[0]).requires_grad_(True), ctx.take(x2[0]).requires_grad_(True)
            wa, wb = w.clone().requires_grad_(True), w2.clone().requires_grad_(True)
            ya, yb = causal_conv1d_kcp_multi([xa, xb], [wa, wb], ctx)
            torch.autograd.backward([ya, yb], [ctx.take(dy[0]), ctx.take(dy2[0])])
            assert ctx.exchanges == 1 and wb.grad.dtype == torch.bfloat16
            for name, local in (("y", ya.detach()), ("dx", xa.grad), ("y2", yb.detach()), ("dx2", xb.grad)):
                ctx.scatter(got[name], local)
            dws.append(wa.grad.double())
            # one tensor on its own: the same bits, and a recompute handle skips the second exchange
            class Handle:
                entries = {}
            single = _cut_context(cu_host, rank, world, [x[0]], [dy[0]], layout)
            xs_ = single.take(x[0]).requires_grad_(True)
            y1 = causal_conv1d_kcp(xs_, w, single, recompute_handle=Handle)
            y1.backward(single.take(dy[0]))
            assert torch.equal(y1, ya) and torch.equal(xs_.grad, xa.grad)
            again = causal_conv1d_kcp(single.take(x[0]), w, single, recompute_handle=Handle)
            assert single.exchanges == 1 and torch.equal(again, ya)
        assert torch.equal(got["y"], want["y"][0]) and torch.equal(got["dx"], want["dx"][0])
        assert torch.equal(got["y2"], want2["y"][0]) and torch.equal(got["dx2"], want2["dx"][0])
        atol, rtol = (DW_ATOL, DW_RTOL) if policy == "bf16" else (DW_FP32G_ATOL, DW_FP32G_RTOL)
        assert C.outside(sum(dws).float().cpu(), want["dw"].double().cpu(), atol=atol, rtol=rtol) == 0
    finally:
        package.configure()
