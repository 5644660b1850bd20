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
}
HEADS = (2, 4)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str, seq_lens, exchange: str, gate: str) -> None:
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
    ctx = gdn.build_kcp_context(cu, device=dev)
    lo = rank * ctx.num_tokens
    sl = slice(lo, lo + ctx.num_tokens)
    leaves = {n: x[n][sl].unsqueeze(0).to(dev).requires_grad_(True) for n in ("q", "k", "v", "g")}
    beta = x["beta"][sl].unsqueeze(0).to(dev).bfloat16().requires_grad_(True)
    o = gdn.kcp_chunk_gated_delta_rule(leaves["q"], leaves["k"], leaves["v"], leaves["g"], beta, ctx,
                                       use_qk_l2norm_in_kernel=True)
    o.backward(x["do"][sl].unsqueeze(0).to(dev))
    torch.cuda.synchronize()
    torch.save({"o": o.detach().cpu()[0], **{f"d{n}": t.grad.cpu()[0] for n, t in leaves.items()},
                "dbeta": beta.grad.cpu()[0]}, f"{out_dir}/rank{rank}.pt")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("case", list(CASES))
def test_ranks_against_one_gpu(tmp_path, case):
    import torch.multiprocessing as mp

    from miles_ext_kernels_b200.cake import gdn
    from oracle import gdn_oracle as O

    world, seq_lens, exchange, gate = CASES[case]
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), seq_lens, exchange, gate), nprocs=world, join=True)
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
        got = torch.cat([p[name] for p in parts], 0)
        if case == "2-aligned-sequential":
            # the same chunks in the same order with the exact fp32 state at the boundary: the same bits
            assert torch.equal(got, ref), name
        else:
            ok, m = O.within_budget(got.float(), ref.float(), rel_rms_max=6e-3, max_abs_rel=2e-2)
            assert ok, (name, m)
