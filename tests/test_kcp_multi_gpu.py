"""Context parallelism on 2 and 4 GPUs: one packed batch split into contiguous slices, the chunk state handed from
rank to rank (NCCL point to point) or folded from the ranks' affine summaries (one all-gather), against the same
batch on one GPU.  Child processes, one per GPU, with a bounded
process-group timeout so an unmatched transfer fails instead of hanging (reference: tests/cake/gdn/test_gdn_kcp_gpu.py:
404-634).  NVLS is switched off: nothing here needs in-switch reduction."""

from __future__ import annotations

import datetime
import os
import socket

import pytest
import torch

from gdn_cases import draw

pytestmark = pytest.mark.gpu

# "aligned": every rank boundary falls on a chunk boundary of its document, so the sequential hand-over cuts the same
# chunks as one GPU does and must give the same bits; "ragged": a boundary cuts a chunk, the runs chunk the document
# differently and agree within the budgets.  The parallel exchange (affine rank summaries, one all-gather) agrees
# within the budgets on either; with four ranks the first document crosses three of them, so a middle rank's
# transfer matrix takes part, and each rank's fragment is long enough (32 chunks) for a two-segment summary.
CASES = {
    # name: (world, seq_lens, exchange, gate)
    "2-aligned-sequential": (2, (320, 704), "sequential", "weak"),
    "2-ragged-sequential": (2, (300, 724), "sequential", "weak"),
    "2-long-parallel": (2, (3000, 1096), "parallel", "weak"),
    "4-long-parallel-weak": (4, (6000, 2192), "parallel", "weak"),
    "4-long-parallel-strong": (4, (6000, 2192), "parallel", "strong"),
    "4-long-sequential": (4, (6016, 2176), "sequential", "weak"),
    # the load-balanced layouts: rank r holds pieces r and 2 W - 1 - r (of the batch / of every document); a rank
    # publishes up to two summaries per direction and folds chains that pass through its own other piece
    "2-zigzag": (2, (3000, 1096), "auto", "weak", "zigzag"),
    "4-zigzag": (4, (6000, 2192), "auto", "weak", "zigzag"),
    "4-zigzag-strong-gate": (4, (6000, 2192), "auto", "strong", "zigzag"),
    "2-zigzag-per-document": (2, (3072, 1024), "auto", "weak", "zigzag_per_document"),
}
HEADS = (2, 4)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _take(full: torch.Tensor, cu, fragments) -> torch.Tensor:
    """A rank's tokens of an undivided ``[S, ...]`` tensor, in local order."""
    return torch.cat([full[cu[f.doc] + f.offset : cu[f.doc] + f.end] for f in fragments])


def _worker(rank: int, world: int, port: int, out_dir: str, seq_lens, exchange: str, gate: str,
            layout: str = "contiguous") -> None:
    import torch.distributed as dist

    import miles_ext_kernels_b200 as package
    from miles_ext_kernels_b200.cake import gdn

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120),
                            device_id=dev)
    package.configure(cake_gdn_kcp_exchange=exchange)
    x = draw(seq_lens, HEADS, seed=9, gate=gate)
    cu = (0, seq_lens[0], sum(seq_lens))
    ctx = gdn.build_kcp_context(cu, device=dev, layout=layout)
    mine = lambda t: _take(t, cu, ctx.fragments).unsqueeze(0).to(dev)  # noqa: E731
    leaves = {n: mine(x[n]).requires_grad_(True) for n in ("q", "k", "v", "g")}
    beta = mine(x["beta"]).bfloat16().requires_grad_(True)
    o = gdn.kcp_chunk_gated_delta_rule(leaves["q"], leaves["k"], leaves["v"], leaves["g"], beta, ctx,
                                       use_qk_l2norm_in_kernel=True)
    o.backward(mine(x["do"]))
    torch.cuda.synchronize()
    torch.save({"o": o.detach().cpu()[0], **{f"d{n}": t.grad.cpu()[0] for n, t in leaves.items()},
                "dbeta": beta.grad.cpu()[0], "fragments": [(f.doc, f.offset, f.length) for f in ctx.fragments]},
               f"{out_dir}/rank{rank}.pt")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("case", list(CASES))
def test_ranks_against_one_gpu(tmp_path, case):
    import torch.multiprocessing as mp

    from miles_ext_kernels_b200.cake import gdn
    from oracle import gdn_oracle as O

    world, seq_lens, exchange, gate, *rest = CASES[case]
    layout = rest[0] if rest else "contiguous"
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), seq_lens, exchange, gate, layout), nprocs=world,
             join=True)
    dev = torch.device("cuda", 0)
    x = draw(seq_lens, HEADS, seed=9, gate=gate)
    cu = (0, seq_lens[0], sum(seq_lens))
    leaves = {n: x[n].unsqueeze(0).to(dev).requires_grad_(True) for n in ("q", "k", "v", "g")}
    beta = x["beta"].unsqueeze(0).to(dev).bfloat16().requires_grad_(True)
    o, _ = gdn.chunk_gated_delta_rule(leaves["q"], leaves["k"], leaves["v"], leaves["g"], beta,
                                      cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=dev), cu_seqlens_cpu=cu,
                                      use_qk_l2norm_in_kernel=True)
    o.backward(x["do"].unsqueeze(0).to(dev))
    torch.cuda.synchronize()
    want = {"o": o.detach().cpu()[0], **{f"d{n}": t.grad.cpu()[0] for n, t in leaves.items()},
            "dbeta": beta.grad.cpu()[0]}
    parts = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    for name, ref in want.items():
        got = torch.zeros_like(ref)  # every rank's tokens back at their places in the batch
        for part in parts:
            at = 0
            for doc, offset, length in part["fragments"]:
                got[cu[doc] + offset : cu[doc] + offset + length] = part[name][at : at + length]
                at += length
        if case == "2-aligned-sequential":
            # the same chunks in the same order with the exact fp32 state at the boundary: the same bits
            assert torch.equal(got, ref), name
        else:
            ok, m = O.within_budget(got.float(), ref.float(), rel_rms_max=6e-3, max_abs_rel=2e-2)
            assert ok, (name, m)


def _conv_worker(rank: int, world: int, port: int, out_dir: str, lens, channels, layout) -> None:
    import torch.distributed as dist

    from miles_ext_kernels_b200.cake import gdn
    from miles_ext_kernels_b200.cake.conv1d import causal_conv1d_kcp_multi

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120),
                            device_id=dev)
    cu = (0, *torch.tensor(lens).cumsum(0).tolist())
    ctx = gdn.build_kcp_context(cu, device=dev, layout=layout)
    mine = lambda t: _take(t, cu, ctx.fragments).to(dev)  # noqa: E731
    full = _conv_inputs(sum(lens), channels)
    xs = [mine(full[f"x{i}"]).requires_grad_(True) for i in range(len(channels))]
    ws = [full[f"w{i}"].to(dev).requires_grad_(True) for i in range(len(channels))]
    ys = causal_conv1d_kcp_multi(xs, ws, ctx)
    torch.autograd.backward(list(ys), [mine(full[f"dy{i}"]) for i in range(len(channels))])
    torch.cuda.synchronize()
    out = {"fragments": [(f.doc, f.offset, f.length) for f in ctx.fragments]}
    for i in range(len(channels)):
        out.update({f"y{i}": ys[i].detach().cpu(), f"dx{i}": xs[i].grad.cpu(), f"dw{i}": ws[i].grad.cpu()})
    torch.save(out, f"{out_dir}/rank{rank}.pt")
    dist.barrier()
    dist.destroy_process_group()


def _conv_inputs(S, channels):
    gen = torch.Generator().manual_seed(77)
    out = {}
    for i, c in enumerate(channels):
        out[f"x{i}"] = torch.randn(S, c, generator=gen).bfloat16()
        out[f"w{i}"] = 0.5 * torch.randn(c, 4, generator=gen)
        out[f"dy{i}"] = torch.randn(S, c, generator=gen).bfloat16()
    return out


@pytest.mark.parametrize("world,lens,layout", [(2, (300, 724), "contiguous"),
                                               (4, (1, 2, 253, 1, 2, 509, 256), "contiguous"),
                                               (2, (300, 724), "zigzag"), (4, (1, 2, 253, 1, 2, 509, 256), "zigzag")])
def test_short_convolution_across_ranks(tmp_path, world, lens, layout):
    """The three rows across each cut travel between neighbours (one message per direction for the layer's
    tensors): y and dx are the bits of one GPU's call, the ranks' weight-gradient partials add up to its sum."""
    import torch.multiprocessing as mp

    from miles_ext_kernels_b200.cake.conv1d import causal_conv1d

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    channels = (384, 136)
    mp.spawn(_conv_worker, args=(world, _free_port(), str(tmp_path), lens, channels, layout), nprocs=world, join=True)
    dev = torch.device("cuda", 0)
    full = _conv_inputs(sum(lens), channels)
    cu_host = (0, *torch.tensor(lens).cumsum(0).tolist())
    cu = torch.tensor(cu_host, dtype=torch.int32, device=dev)
    parts = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]

    def whole(name, like):
        out = torch.zeros_like(like)
        for part in parts:
            at = 0
            for doc, offset, length in part["fragments"]:
                out[cu_host[doc] + offset : cu_host[doc] + offset + length] = part[name][at : at + length]
                at += length
        return out

    for i in range(len(channels)):
        x, w = full[f"x{i}"].to(dev).requires_grad_(True), full[f"w{i}"].to(dev).requires_grad_(True)
        y = causal_conv1d(x, w, cu)
        y.backward(full[f"dy{i}"].to(dev))
        assert torch.equal(whole(f"y{i}", y.detach().cpu()), y.detach().cpu())
        assert torch.equal(whole(f"dx{i}", x.grad.cpu()), x.grad.cpu())
        dw = sum(p[f"dw{i}"].double() for p in parts)
        assert torch.allclose(dw, w.grad.double().cpu(), atol=5e-2, rtol=1e-4)
