"""The context-parallel layouts on ONE GPU: the ranks of a group run one after another and the all-gather of the
parallel state exchange is stood in for by the summaries the ranks published in an earlier pass (every rank's
publication depends on its own tokens only).  Against the undivided call on the same GPU, within the budgets of the
multi-GPU test (reference: tests/cake/gdn/test_gdn_kcp_gpu.py:404-634)."""

from __future__ import annotations

import pytest
import torch

from gdn_cases import draw

pytestmark = pytest.mark.gpu
HEADS = (2, 4)


class _Published(Exception):
    """A rank has handed over its summaries; the pass that collects them ends the rank's call here."""


def _emulated_context(cu, rank, world, layout, board):
    """A rank's context whose exchanges read and write ``board``: ``board[direction]`` is a list of the ranks'
    published summaries (``None``: not collected yet)."""
    from miles_ext_kernels_b200.cake._impl.gdn import kcp

    class Exchange(kcp._ParallelExchange):
        def _gather(self, local):
            direction = "backward" if self._reverse else "forward"
            slots = board[direction]
            if any(s is None for s in slots):
                slots[rank] = local.clone()
                raise _Published
            return torch.stack(slots)

        def forward_begin(self, *args):
            self._reverse = False
            return super().forward_begin(*args)

        def backward_begin(self, *args):
            self._reverse = True
            return super().backward_begin(*args)

        def kda_forward_state(self, *args):
            self._reverse = False
            return super().kda_forward_state(*args)

        def kda_backward_state(self, *args):
            self._reverse = True
            return super().kda_backward_state(*args)

    class Context(kcp.KcpContext):
        def exchange(self, mode="auto"):
            return Exchange(self)

    return Context(cu, None, rank, world, "cuda", layout=layout)


def _take(full, cu, fragments):
    return torch.cat([full[cu[f.doc] + f.offset : cu[f.doc] + f.end] for f in fragments])


@pytest.mark.parametrize("world,seq_lens,layout,gate", [
    (4, (6000, 2192), "zigzag", "weak"), (4, (6000, 2192), "zigzag", "strong"), (4, (6000, 2192), "contiguous", "weak"),
    (2, (3072, 1024), "zigzag_per_document", "weak"), (4, (2048, 4096, 2048), "zigzag_per_document", "weak"),
    (3, (1200, 3408), "zigzag", "weak"),
])
def test_layouts_against_the_undivided_call(world, seq_lens, layout, gate):
    from miles_ext_kernels_b200.cake import gdn
    from oracle import gdn_oracle as O

    dev = torch.device("cuda")
    x = draw(seq_lens, HEADS, seed=9, gate=gate)
    cu = (0, *torch.tensor(seq_lens).cumsum(0).tolist())
    board = {"forward": [None] * world, "backward": [None] * world}

    def run_rank(rank):
        ctx = _emulated_context(cu, rank, world, layout, board)
        mine = lambda t: _take(t, cu, ctx.fragments).unsqueeze(0).to(dev)  # noqa: E731
        leaves = {n: mine(x[n]).requires_grad_(True) for n in ("q", "k", "v", "g")}
        beta = mine(x["beta"]).bfloat16().requires_grad_(True)
        o = gdn.kcp_chunk_gated_delta_rule(leaves["q"], leaves["k"], leaves["v"], leaves["g"], beta, ctx,
                                           use_qk_l2norm_in_kernel=True)
        o.backward(mine(x["do"]))
        return ctx, {"o": o.detach()[0], **{f"d{n}": t.grad[0] for n, t in leaves.items()}, "dbeta": beta.grad[0]}

    for _ in range(2):  # the passes that collect the forward, then the backward summaries
        for rank in range(world):
            with pytest.raises(_Published):
                run_rank(rank)
    assert all(s is not None for s in board["forward"] + board["backward"])
    results = [run_rank(rank) for rank in range(world)]

    leaves = {n: x[n].unsqueeze(0).to(dev).requires_grad_(True) for n in ("q", "k", "v", "g")}
    beta = x["beta"].unsqueeze(0).to(dev).bfloat16().requires_grad_(True)
    o, _ = gdn.chunk_gated_delta_rule(leaves["q"], leaves["k"], leaves["v"], leaves["g"], beta,
                                      cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=dev), cu_seqlens_cpu=cu,
                                      use_qk_l2norm_in_kernel=True)
    o.backward(x["do"].unsqueeze(0).to(dev))
    want = {"o": o.detach()[0], **{f"d{n}": t.grad[0] for n, t in leaves.items()}, "dbeta": beta.grad[0]}
    for name, ref in want.items():
        got = torch.zeros_like(ref)
        for ctx, out in results:
            at = 0
            for f in ctx.fragments:
                got[cu[f.doc] + f.offset : cu[f.doc] + f.end] = out[name][at : at + f.length]
                at += f.length
        ok, m = O.within_budget(got.float().cpu(), ref.float().cpu(), rel_rms_max=6e-3, max_abs_rel=2e-2)
        assert ok, (name, m)


@pytest.mark.parametrize("world,seq_lens,layout", [
    (2, (1500, 548), "contiguous"), (4, (3000, 1096), "zigzag"), (2, (1024, 2048), "zigzag_per_document"),
])
def test_kda_layouts_against_the_undivided_call(world, seq_lens, layout):
    """The per-channel-decay variant through the same exchange: its fragments' summaries come from its own pre-scans
    (every summary exact, no warm-up rule)."""
    from miles_ext_kernels_b200.cake import kda
    from oracle import gdn_oracle as O
    from test_kda_gpu import NAMES, draw as draw_kda

    dev = torch.device("cuda")
    H = 2
    x = draw_kda(seq_lens, H, seed=61, gate="faint")
    cu = (0, *torch.tensor(seq_lens).cumsum(0).tolist())
    board = {"forward": [None] * world, "backward": [None] * world}

    def run_rank(rank):
        ctx = _emulated_context(cu, rank, world, layout, board)
        mine = lambda t: _take(t, cu, ctx.fragments).to(dev)  # noqa: E731
        leaves = {n: mine(x[n]).requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
        o = kda.chunk_kda_kcp(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], ctx)
        o.backward(mine(x["do"]))
        return ctx, {"o": o.detach(), **{f"d{n}": t.grad for n, t in leaves.items()}}

    for _ in range(2):
        for rank in range(world):
            with pytest.raises(_Published):
                run_rank(rank)
    results = [run_rank(rank) for rank in range(world)]
    leaves = {n: x[n].to(dev).requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
    o = kda.chunk_kda(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"],
                      torch.tensor(cu, dtype=torch.int32, device=dev))
    o.backward(x["do"].to(dev))
    want = {"o": o.detach(), **{f"d{n}": t.grad for n, t in leaves.items()}}
    for name in NAMES:
        ref = want[name]
        got = torch.zeros_like(ref)
        for ctx, out in results:
            at = 0
            for f in ctx.fragments:
                got[cu[f.doc] + f.offset : cu[f.doc] + f.end] = out[name][at : at + f.length]
                at += f.length
        ok, m = O.within_budget(got.float().cpu(), ref.float().cpu(), rel_rms_max=6e-3, max_abs_rel=2e-2)
        assert ok, (name, m)


def test_kda_light_save_mode_and_recompute_handle():
    """``save_mode="light"`` replays this rank's kernels in the backward from the states the forward received: the
    bits of the saved backward, and no second exchange.  Under activation checkpointing a recompute handle does the
    same for the region's replayed forward: the gather runs once per direction, not twice."""
    import torch.utils.checkpoint as checkpoint

    from miles_ext_kernels_b200.cake import kda
    from test_kda_gpu import NAMES, draw as draw_kda

    dev = torch.device("cuda")
    world, seq_lens, H = 2, (1500, 548), 2
    x = draw_kda(seq_lens, H, seed=62, gate="faint")
    cu = (0, *torch.tensor(seq_lens).cumsum(0).tolist())
    board = {"forward": [None] * world, "backward": [None] * world}
    gathers = []

    def run_rank(rank, count=False, **options):
        ctx = _emulated_context(cu, rank, world, "contiguous", board)
        if count:
            inner = ctx.exchange

            def counting(mode="auto"):
                exchange = inner(mode)
                gather = exchange._gather

                def counted(local):
                    gathers.append("backward" if exchange._reverse else "forward")
                    return gather(local)

                exchange._gather = counted
                return exchange

            ctx.exchange = counting
        mine = lambda t: _take(t, cu, ctx.fragments).to(dev)  # noqa: E731
        leaves = {n: mine(x[n]).requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
        if options.pop("checkpointed", False):
            o = checkpoint.checkpoint(lambda *t: kda.chunk_kda_kcp(*t, ctx, **options), *leaves.values(),
                                      use_reentrant=False)
        else:
            o = kda.chunk_kda_kcp(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], ctx, **options)
        o.backward(mine(x["do"]))
        return {"o": o.detach(), **{f"d{n}": t.grad for n, t in leaves.items()}}

    for _ in range(2):
        for rank in range(world):
            with pytest.raises(_Published):
                run_rank(rank)
    for rank in range(world):
        full = run_rank(rank)
        gathers.clear()
        light = run_rank(rank, count=True, save_mode="light")
        assert gathers == ["forward", "backward"], gathers
        for name in NAMES:
            assert torch.equal(light[name], full[name]), (rank, name)
        gathers.clear()
        replayed = run_rank(rank, count=True, checkpointed=True)
        assert gathers == ["forward", "forward", "backward"], gathers  # the replay exchanges again
        gathers.clear()
        handled = run_rank(rank, count=True, checkpointed=True, recompute_handle=kda.RecomputeHandle())
        assert gathers == ["forward", "backward"], gathers  # the replay binds what the forward received
        for name in NAMES:
            assert torch.equal(handled[name], full[name]) and torch.equal(replayed[name], full[name]), (rank, name)


def test_gdn_recompute_state_under_a_context_gives_the_saved_bits():
    """``--cake-gdn-recompute-state`` under a context (the reference's ``save_mode="light"``): the backward rebuilds
    w / u / h / v_new from the saved operands and the state that entered this rank, without a second exchange."""
    import miles_ext_kernels_b200 as package
    from miles_ext_kernels_b200.cake import gdn

    dev = torch.device("cuda")
    world, seq_lens = 2, (3000, 1096)
    x = draw(seq_lens, HEADS, seed=10, gate="weak")
    cu = (0, *torch.tensor(seq_lens).cumsum(0).tolist())
    board = {"forward": [None] * world, "backward": [None] * world}

    def run_rank(rank):
        ctx = _emulated_context(cu, rank, world, "contiguous", board)
        mine = lambda t: _take(t, cu, ctx.fragments).unsqueeze(0).to(dev)  # noqa: E731
        leaves = {n: mine(x[n]).requires_grad_(True) for n in ("q", "k", "v", "g")}
        beta = mine(x["beta"]).bfloat16().requires_grad_(True)
        o = gdn.kcp_chunk_gated_delta_rule(leaves["q"], leaves["k"], leaves["v"], leaves["g"], beta, ctx,
                                           use_qk_l2norm_in_kernel=True)
        o.backward(mine(x["do"]))
        return {"o": o.detach()[0], **{f"d{n}": t.grad[0] for n, t in leaves.items()}, "dbeta": beta.grad[0]}

    for _ in range(2):
        for rank in range(world):
            with pytest.raises(_Published):
                run_rank(rank)
    for rank in range(world):
        package.configure()
        saved = run_rank(rank)
        package.configure(cake_gdn_recompute_state=True)
        again = run_rank(rank)
        for name, want in saved.items():
            assert torch.equal(again[name], want), (rank, name)


def test_a_call_under_a_context_replays_from_a_cuda_graph():
    """Forward + backward under a context are capturable (the fragment plans, chain tables and fold spans are cached
    device tables; nothing is uploaded from a temporary inside the call): a replay on new inputs written into the
    captured buffers gives the bits of an eager call on those inputs.  The gather of the exchange is the stand-in of
    this file (the other rank's summaries are fixed tensors), so what is captured is everything but NCCL's kernel."""
    from miles_ext_kernels_b200.cake import gdn

    dev = torch.device("cuda")
    world, seq_lens = 2, (3000, 1096)
    cu = (0, *torch.tensor(seq_lens).cumsum(0).tolist())
    first, second = (draw(seq_lens, HEADS, seed=s, gate="weak") for s in (11, 12))
    board = {"forward": [None] * world, "backward": [None] * world}
    names = ("q", "k", "v", "g", "beta", "do")

    def shard(x, ctx):
        out = {n: _take(x[n], cu, ctx.fragments).unsqueeze(0).to(dev) for n in names}
        out["beta"] = out["beta"].bfloat16()
        return out

    def step(ctx, t):
        leaves = {n: t[n].detach().requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
        o = gdn.kcp_chunk_gated_delta_rule(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], ctx,
                                           use_qk_l2norm_in_kernel=True)
        o.backward(t["do"])
        return [o.detach()] + [leaves[n].grad for n in ("q", "k", "v", "g", "beta")]

    for _ in range(2):  # collect every rank's summaries of the first inputs
        for rank in range(world):
            ctx = _emulated_context(cu, rank, world, "contiguous", board)
            with pytest.raises(_Published):
                step(ctx, shard(first, ctx))
    for rank in range(world):
        ctx = _emulated_context(cu, rank, world, "contiguous", board)
        want = [t.clone() for t in step(ctx, shard(second, ctx))]
        static = {n: t.clone() for n, t in shard(first, ctx).items()}
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                step(ctx, static)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            outs = step(ctx, static)
        for n, t in shard(second, ctx).items():
            static[n].copy_(t)
        graph.replay()
        torch.cuda.synchronize()
        for got, ref in zip(outs, want):
            assert torch.equal(got, ref), rank
