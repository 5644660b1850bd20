"""Host logic of the GDN op on the CPU: chunk tables (host and device routes), entry checks, the context-parallel
partition, and a two-rank gloo run of the state hand-over (reference: tests/cake/gdn/test_gdn_host.py,
test_gdn_kcp_wiring.py)."""

from __future__ import annotations

import os
import socket

import pytest
import torch

from miles_ext_kernels_b200.cake._impl.gdn import kcp, ops
from miles_ext_kernels_b200.cake._impl.gdn import meta as M
from oracle import gdn_oracle as O


def test_host_tables_match_the_oracle_and_are_cached_per_layout():
    seq_lens = (1, 63, 64, 65, 130, 0, 7)
    cu = [0]
    for n in seq_lens:
        cu.append(cu[-1] + n)
    before = M.host_meta_builds()
    meta = M.chunk_meta(torch.tensor(cu), tuple(cu), 1, cu[-1], "cpu")
    again = M.chunk_meta(torch.tensor(cu), tuple(cu), 1, cu[-1], "cpu")
    assert again is meta and M.host_meta_builds() == before + 1
    table = O.chunk_table(seq_lens)
    assert tuple(meta.chunk_start.tolist()) == table.chunk_start
    assert tuple(meta.chunk_len.tolist()) == table.chunk_len
    assert tuple(meta.chunk_seq.tolist()) == table.chunk_seq
    assert tuple(meta.seq_chunk_start.tolist()) == table.seq_chunk_start
    assert meta.exact and meta.num_chunks == table.num_chunks and meta.num_seqs == len(seq_lens)


@pytest.mark.parametrize("seq_lens", [(1, 63, 64, 65, 130), (4096,), (0, 5, 0), (64, 64)])
def test_device_route_equals_host_route_on_the_real_chunks(seq_lens):
    cu = [0]
    for n in seq_lens:
        cu.append(cu[-1] + n)
    total = cu[-1]
    host = M.chunk_meta(torch.tensor(cu), tuple(cu), 1, total, "cpu")
    dev = M.chunk_meta(torch.tensor(cu, dtype=torch.int32), None, 1, total, "cpu")
    assert not dev.exact and dev.num_chunks >= host.num_chunks
    n = host.num_chunks
    assert dev.chunk_start[:n].tolist() == host.chunk_start.tolist()
    assert dev.chunk_len[:n].tolist() == host.chunk_len.tolist()
    assert dev.chunk_seq[:n].tolist() == host.chunk_seq.tolist()
    assert dev.seq_chunk_start.tolist() == host.seq_chunk_start.tolist()
    assert dev.chunk_len[n:].sum().item() == 0  # pad chunks are empty


def test_uneven_documents_are_walked_longest_first():
    cu = (0, 100, 1000, 1064, 5000, 5010)  # chunk counts 2, 15, 1, 62, 1
    meta = M.chunk_meta(torch.tensor(cu), cu, 1, cu[-1], "cpu")
    assert meta.seq_order.tolist() == [3, 1, 0, 2, 4] and meta.seq_order.dtype == torch.int32
    assert meta.seq_chunk_start.tolist() == [0, 2, 17, 18, 80, 81]
    even = M.chunk_meta(None, None, 3, 100, "cpu")
    assert even.seq_order is None  # nothing to balance


def test_equal_length_batches_and_boundary_errors():
    meta = M.chunk_meta(None, None, 3, 100, "cpu")
    assert meta.num_seqs == 3 and meta.chunk_len.tolist() == [64, 36] * 3
    with pytest.raises(ValueError, match="must end at the 128 tokens of q; it ends at 127"):
        M.chunk_meta(torch.tensor([0, 128]), (0, 127), 1, 128, "cpu")
    with pytest.raises(ValueError, match="must start at 0"):
        M.chunk_meta(torch.tensor([1, 128]), (1, 128), 1, 128, "cpu")
    with pytest.raises(ValueError, match="leading batch dimension of 1"):
        M.chunk_meta(torch.tensor([0, 128]), (0, 128), 2, 64, "cpu")


def test_entry_checks_on_metadata():
    q = torch.zeros(1, 8, 2, 128, dtype=torch.bfloat16)
    v = torch.zeros(1, 8, 4, 128, dtype=torch.bfloat16)
    g = torch.zeros(1, 8, 4)
    with pytest.raises(ValueError, match="q must be a CUDA tensor"):
        ops.chunk_gated_delta_rule(q, q, v, g, g)
    with pytest.raises(NotImplementedError, match="head dims must be 128"):
        ops.chunk_gated_delta_rule(q[..., :64], q[..., :64], v, g, g)
    with pytest.raises(NotImplementedError, match="q/k/v must be bfloat16"):
        ops.chunk_gated_delta_rule(q.float(), q, v, g, g)
    with pytest.raises(NotImplementedError, match="head_first=True is not supported"):
        ops.chunk_gated_delta_rule(q, q, v, g, g, head_first=True)
    with pytest.raises(TypeError, match="must be a KcpContext"):
        ops.chunk_gated_delta_rule(q, q, v, g, g, cp_context=object())
    ctx = kcp.KcpContext((0, 8), None, 0, 1, "cpu")
    with pytest.raises(ValueError, match="initial_state is not supported under context parallelism"):
        ops.chunk_gated_delta_rule(q, q, v, g, g, cp_context=ctx, initial_state=torch.zeros(1, 4, 128, 128))
    with pytest.raises(ValueError, match="output_final_state is not supported under context parallelism"):
        ops.chunk_gated_delta_rule(q, q, v, g, g, cp_context=ctx, output_final_state=True)
    with pytest.raises(TypeError):
        ops.kcp_chunk_gated_delta_rule(q, q, v, g, g, None)


def test_contiguous_partition_is_flas():
    cu = (0, 130, 320, 460, 512)  # four documents, 512 tokens
    for world in (1, 2, 4):
        part = 512 // world
        for rank in range(world):
            ctx = kcp.KcpContext(cu, None, rank, world, "cpu")
            lo, hi = rank * part, (rank + 1) * part
            want = tuple(sorted({min(max(b, lo), hi) - lo for b in cu}))
            assert ctx.cu_seqlens_cpu == want and ctx.num_tokens == part
            assert ctx.cu_seqlens.tolist() == list(want) and ctx.cu_seqlens.dtype == torch.int32
            assert ctx.continues_in == (lo not in cu) and ctx.continues_out == (hi not in cu)
            assert ctx.fla_compatible and ctx.layout == "contiguous"
    with pytest.raises(ValueError, match="divide by the world size"):
        kcp.KcpContext((0, 10), None, 0, 3, "cpu")
    zig = kcp.KcpContext(cu, None, 0, 2, "cpu", layout="zigzag")  # pieces 0 and 3 of four
    assert zig.cu_seqlens_cpu == (0, 128, 204, 256) and not zig.fla_compatible


def test_document_runs_across_ranks():
    from miles_ext_kernels_b200.cake._impl.gdn.kcp import document_run

    cu = (0, 6000, 8192)  # four ranks of 2,048 tokens: the first document crosses ranks 0..2, the second 2..3
    assert document_run(cu, 0, 4) == (0, 2)
    assert document_run(cu, 1, 4) == (0, 2)
    assert document_run(cu, 2, 4) == (0, 3)
    assert document_run(cu, 3, 4) == (2, 3)
    cu = (0, 2048, 4096, 8192)  # documents end on rank boundaries: nothing continues there
    assert document_run(cu, 0, 4) == (0, 0) and document_run(cu, 1, 4) == (1, 1)
    assert document_run(cu, 2, 4) == (2, 3) and document_run(cu, 3, 4) == (2, 3)


# ---- two ranks on gloo: the hand-over reproduces the single-rank recurrence -----------------------------------------
def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str) -> None:
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    cu = (0, 100, 256)  # the second document crosses the rank boundary at token 128
    gen = torch.Generator().manual_seed(7)
    T, H, HV = cu[-1], 1, 2
    q, k = torch.randn(T, H, 128, generator=gen), torch.randn(T, H, 128, generator=gen)
    v, do = torch.randn(T, HV, 128, generator=gen), torch.randn(T, HV, 128, generator=gen)
    g, beta = -0.2 * torch.rand(T, HV, generator=gen), torch.rand(T, HV, generator=gen)
    ctx = kcp.build_kcp_context(cu, device="cpu")
    assert ctx.rank == rank and ctx.world_size == world
    ex = ctx.exchange()
    lo = rank * ctx.num_tokens
    sl = slice(lo, lo + ctx.num_tokens)
    local = ctx.cu_seqlens_cpu
    lens = tuple(b - a for a, b in zip(local[:-1], local[1:]))
    # forward: receive, scan (the oracle stands in for the kernels on the CPU), send
    h0 = ex.incoming_state(len(lens), HV, "cpu")
    o, final, tape = O.chunked_forward(q[sl], k[sl], v[sl], g[sl], beta[sl], lens, h0=h0, use_qk_l2norm=True,
                                       rounding=None, output_final_state=True)
    ex.outgoing_state(final)
    # backward: receive the adjoint state from the next rank, scan in reverse, send to the previous rank
    dht = ex.incoming_adjoint(len(lens), HV, "cpu")
    grads = O.chunked_backward(tape, do[sl], dht=dht, rounding=None)
    ex.outgoing_adjoint(grads["dh0"])
    torch.save({"o": o, **{n: grads[n] for n in ("dq", "dk", "dv", "dg", "dbeta")}}, f"{out_dir}/rank{rank}.pt")
    if rank == 0:
        ref = O.chunked_forward_backward(q, k, v, g, beta, (100, 156), do, use_qk_l2norm=True, rounding=None)
        torch.save(ref, f"{out_dir}/ref.pt")
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_single_rank_result(tmp_path):
    import torch.multiprocessing as mp

    mp.spawn(_rank_main, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    ref = torch.load(tmp_path / "ref.pt")
    parts = [torch.load(tmp_path / f"rank{r}.pt") for r in range(2)]
    for name in ("o", "dq", "dk", "dv", "dg", "dbeta"):
        got = torch.cat([p[name] for p in parts], 0)
        m = O.metrics(got, ref[name])
        assert m["finite"] and m["max_abs"] <= 1e-5 * max(m["max_ref"], 1e-3), (name, m)


def test_config0_is_rejected_with_the_reference_messages():
    """The benchmark's configuration 0 (fp32, dk = dv = 64) is outside what the kernels serve, as it is outside what
    the reference's serve (reference: miles_ext_kernels/cake/_impl/gdn/ops.py:2307-2310): the entry point says so
    with the reference's exception class and words before it looks at anything else; only the oracles run it."""
    from miles_ext_kernels_b200.workloads import make_workload

    w = make_workload("cfg0")
    with pytest.raises(NotImplementedError, match="q/k/v must be bfloat16"):
        ops.chunk_gated_delta_rule(w.q, w.k, w.v, w.g, w.beta)
    with pytest.raises(NotImplementedError, match="head dims must be 128"):
        ops.chunk_gated_delta_rule(w.q.bfloat16(), w.k.bfloat16(), w.v.bfloat16(), w.g, w.beta.bfloat16())
