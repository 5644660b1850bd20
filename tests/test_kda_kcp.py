"""Context-parallel KDA: the partition and context on the host, the rank-ordered reduce of the gate parameters'
gradients on two gloo ranks (CPU), the boundary states of the kernels on one GPU (a document cut in two by hand), and
two ranks on two GPUs against the undivided batch (reference: tests/cake/kda/test_kda_kcp_gpu.py)."""

from __future__ import annotations

import datetime
import os
import socket

import pytest
import torch

NAMES = ("o", "dq", "dk", "dv", "dg", "dbeta")


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def draw(T, H, seed):
    gen = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(T, H, 128, generator=gen), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(T, H, 128, generator=gen), dim=-1)
    v = torch.randn(T, H, 128, generator=gen)
    beta = torch.sigmoid(torch.randn(T, H, generator=gen))
    g = -0.3 * torch.rand(T, H, 128, generator=gen)
    do = torch.randn(T, H, 128, generator=gen)
    return {"q": q.bfloat16(), "k": k.bfloat16(), "v": v.bfloat16(), "g": g, "beta": beta.bfloat16(),
            "do": do.bfloat16()}


# ---- host logic (CPU) ------------------------------------------------------------------------------------------------
def test_partition_and_context_on_the_host():
    from miles_ext_kernels_b200.cake import kda

    part = kda.partition_kcp(torch.tensor([0, 320, 1024]), 2)
    assert part.world_size == 2 and part.cu_seqlens_global == (0, 320, 1024) and part.layout == "contiguous"
    assert kda.partition_kcp((0, 320, 1024), 2) == part
    first = kda.build_context_kcp(part, object(), 0, "cpu")
    second = kda.build_context_kcp(part, object(), 1, "cpu", heads=(4, 64))
    assert first.cu_seqlens_cpu == (0, 320, 512) and not first.continues_in and first.continues_out
    assert second.cu_seqlens_cpu == (0, 512) and second.continues_in and not second.continues_out
    assert first.num_tokens == second.num_tokens == 512
    zig = kda.build_context_kcp(kda.partition_kcp((0, 320, 1024), 2, "zigzag"), object(), 0, "cpu")
    assert zig.layout == "zigzag" and zig.cu_seqlens_cpu == (0, 256, 512)  # pieces 0 and 3 of four
    table = kda.partition_kcp((0, 1024), 2, fragments=[[(0, 0, 512)], [(0, 512, 512)]])
    assert table.layout == "explicit" and kda.build_context_kcp(table, object(), 1, "cpu").continues_in
    with pytest.raises(ValueError, match="held by no rank"):
        kda.partition_kcp((0, 1024), 2, fragments=[[(0, 0, 512)], [(0, 512, 256)]])
    with pytest.raises(NotImplementedError, match="cut points"):
        kda.partition_kcp((0, 1024), 2, cut_points=(512,))
    with pytest.raises(ValueError, match="divide"):
        kda.partition_kcp((0, 1023), 2)
    with pytest.raises(ValueError, match="start at 0"):
        kda.partition_kcp((1, 1024), 2)
    with pytest.raises(ValueError, match="process group"):
        kda.build_context_kcp(part, None, 0, "cpu")
    with pytest.raises(TypeError, match="partition_kcp"):
        kda.build_context_kcp((0, 1024), None, 0, "cpu")
    with pytest.raises(ValueError, match="1 to 64 heads"):
        kda.build_context_kcp(part, object(), 0, "cpu", heads=65)
    one = kda.build_context_kcp(kda.partition_kcp((0, 64), 1), None, 0, "cpu")
    x = torch.zeros(1)
    with pytest.raises(TypeError, match="build_context_kcp"):
        kda.chunk_kda_kcp(x, x, torch.zeros(64, 2, 128), x, x, "not a context")
    with pytest.raises(NotImplementedError, match="boundary_mode"):
        kda.chunk_kda_kcp(x, x, torch.zeros(64, 2, 128), x, x, one, boundary_mode="replay")
    with pytest.raises(ValueError, match="save_mode"):
        kda.chunk_kda_kcp(x, x, torch.zeros(64, 2, 128), x, x, one, save_mode="medium")
    with pytest.raises(NotImplementedError, match="checkpoint_keep"):
        kda.chunk_kda_kcp(x, x, torch.zeros(64, 2, 128), x, x, one, checkpoint_keep="transfer")
    with pytest.raises(TypeError, match="RecomputeHandle"):
        kda.chunk_kda_kcp(x, x, torch.zeros(64, 2, 128), x, x, one, recompute_handle=object())
    with pytest.raises(ValueError, match="exchange"):
        kda.chunk_kda_kcp(x, x, torch.zeros(64, 2, 128), x, x, one, exchange="ring")


def _reduce_main(rank: int, world: int, port: int, out_dir: str) -> None:
    import torch.distributed as dist

    from miles_ext_kernels_b200.cake import kda

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    ctx = kda.build_context_kcp(kda.partition_kcp((0, 64 * world), world), dist.group.WORLD, rank, "cpu")
    gen = torch.Generator().manual_seed(100 + rank)
    da, db = torch.randn(4, generator=gen), torch.randn(4 * 128, generator=gen)
    total = kda.reduce_gate_param_grads_kcp(ctx, da, db)
    torch.save({"da": da, "db": db, "sum_a": total[0], "sum_b": total[1]}, f"{out_dir}/rank{rank}.pt")
    dist.barrier()
    dist.destroy_process_group()


def test_gate_parameter_gradients_sum_in_rank_order_on_every_rank(tmp_path):
    import torch.multiprocessing as mp

    mp.spawn(_reduce_main, args=(3, _free_port(), str(tmp_path)), nprocs=3, join=True)
    parts = [torch.load(tmp_path / f"rank{r}.pt") for r in range(3)]
    want_a = (parts[0]["da"] + parts[1]["da"]) + parts[2]["da"]
    want_b = (parts[0]["db"] + parts[1]["db"]) + parts[2]["db"]
    for p in parts:
        assert torch.equal(p["sum_a"], want_a) and torch.equal(p["sum_b"], want_b)


# ---- the kernels' boundary states on one GPU ---------------------------------------------------------------------------
def _single(x, cu, dev, **modes):
    from miles_ext_kernels_b200.cake import kda

    leaves = {n: x[n].to(dev).requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
    out = kda.chunk_kda(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"],
                        torch.tensor(cu, dtype=torch.int32, device=dev), **modes)
    out.backward(x["do"].to(dev))
    torch.cuda.synchronize()
    got = {"o": out.detach().cpu()}
    got.update({f"d{n}": leaves[n].grad.cpu() for n in ("q", "k", "v", "g", "beta")})
    return got


@pytest.mark.gpu
@pytest.mark.parametrize("cut", [512, 300], ids=["aligned", "ragged"])
def test_a_document_cut_in_two_by_hand_reproduces_the_undivided_run(cut):
    """What two ranks do, in one process: slice A keeps its final state, slice B starts from it; backward, B hands
    its initial-state gradient to A as the adjoint of A's final state."""
    from miles_ext_kernels_b200.cake._impl.kda import ops
    from oracle import gdn_oracle as O

    dev = torch.device("cuda")
    T, H = 1024, 3
    x = draw(T, H, 21)
    want = _single(x, (0, T), dev)
    with torch.no_grad():
        halves, saved = [], []
        state = None
        for lo, hi in ((0, cut), (cut, T)):
            t = {n: x[n][lo:hi].to(dev).contiguous() for n in ("q", "k", "v", "g")}
            beta32 = x["beta"][lo:hi].to(dev).float().contiguous()
            cu = torch.tensor((0, hi - lo), dtype=torch.int32, device=dev)
            o, s, final = ops._forward(t["q"], t["k"], t["v"], t["g"], beta32, cu, ops.DEFAULT_SCALE, False,
                                       cu_seqlens_cpu=(0, hi - lo), h0=state, want_final=hi < T)
            state = final
            halves.append(o)
            saved.append((s, t["v"], beta32))
        grads = [None, None]
        adjoint = None
        for part in (1, 0):
            lo, hi = ((0, cut), (cut, T))[part]
            s, v3, beta32 = saved[part]
            out = ops._backward(s, v3, beta32, x["do"][lo:hi].to(dev).contiguous(), dht=adjoint, want_dh0=part == 1)
            grads[part], adjoint = out[:5], out[5]
        torch.cuda.synchronize()
    got = {"o": torch.cat(halves).cpu()}
    for i, name in enumerate(("dq", "dk", "dv", "dg", "dbeta")):
        got[name] = torch.cat([grads[0][i], grads[1][i]]).cpu()
    got["dbeta"] = got["dbeta"].to(torch.bfloat16)  # the public entry returns it in beta's dtype
    for name in NAMES:
        ref = want[name].float()
        have = got[name].float()
        if cut % 64 == 0:
            assert torch.equal(have, ref), name  # the same chunks, the exact fp32 state at the cut: the same bits
        else:
            ok, m = O.within_budget(have, ref, rel_rms_max=6e-3, max_abs_rel=2e-2)
            assert ok, (name, m)


@pytest.mark.gpu
def test_a_one_rank_context_gives_the_bits_of_chunk_kda():
    from miles_ext_kernels_b200.cake import kda

    dev = torch.device("cuda")
    cu = (0, 200, 264, 640)
    x = draw(cu[-1], 2, 22)
    want = _single(x, cu, dev, use_qk_l2norm_in_kernel=True)
    ctx = kda.build_context_kcp(kda.partition_kcp(cu, 1), None, 0, dev)
    leaves = {n: x[n].to(dev).requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
    out = kda.chunk_kda_kcp(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], ctx,
                            use_qk_l2norm_in_kernel=True)
    out.backward(x["do"].to(dev))
    torch.cuda.synchronize()
    assert torch.equal(out.detach().cpu(), want["o"])
    for n in ("q", "k", "v", "g", "beta"):
        assert torch.equal(leaves[n].grad.cpu(), want[f"d{n}"]), n
    o2, saved = kda.chunk_kda_fwd_kcp(x["q"].to(dev), x["k"].to(dev), x["v"].to(dev), x["g"].to(dev),
                                      x["beta"].to(dev), ctx, use_qk_l2norm_in_kernel=True)
    grads = kda.chunk_kda_bwd_kcp(x["q"].to(dev), x["k"].to(dev), x["v"].to(dev), x["g"].to(dev), x["beta"].to(dev),
                                  ctx, x["do"].to(dev), saved=saved, use_qk_l2norm_in_kernel=True)
    assert torch.equal(o2.cpu(), want["o"])
    for got, name in zip(grads, ("dq", "dk", "dv", "dbeta", "dg")):
        assert torch.equal(got.cpu(), want[name]), name
    with pytest.raises(ValueError, match="tokens of its slice"):
        kda.chunk_kda_kcp(leaves["q"][:64], leaves["k"][:64], leaves["v"][:64], leaves["g"][:64],
                          leaves["beta"][:64], ctx)


# ---- two ranks on two GPUs ---------------------------------------------------------------------------------------------
LAYOUTS = {"aligned": (320, 704), "ragged": (300, 724)}


def _worker(rank: int, world: int, port: int, out_dir: str, seq_lens) -> None:
    import torch.distributed as dist

    from miles_ext_kernels_b200.cake import kda

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120),
                            device_id=dev)
    H = 2
    x = draw(sum(seq_lens), H, 23)
    gen = torch.Generator().manual_seed(7)
    a_log = (torch.rand(H, generator=gen) * 1.5).to(dev).requires_grad_(True)
    dt_bias = (0.5 * torch.randn(H * 128, generator=gen)).to(dev).requires_grad_(True)
    cu = (0, seq_lens[0], sum(seq_lens))
    ctx = kda.build_context_kcp(kda.partition_kcp(cu, world), dist.group.WORLD, rank, dev)
    sl = slice(rank * ctx.num_tokens, (rank + 1) * ctx.num_tokens)
    leaves = {n: x[n][sl].to(dev).requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
    raw = (10.0 * leaves["g"].detach()).bfloat16().requires_grad_(True)  # a raw gate: activated in the op
    out = kda.chunk_kda_kcp(leaves["q"], leaves["k"], leaves["v"], raw, leaves["beta"], ctx, use_gate_in_kernel=True,
                            A_log=a_log, dt_bias=dt_bias, use_qk_l2norm_in_kernel=True)
    out.backward(x["do"][sl].to(dev))
    da, db = kda.reduce_gate_param_grads_kcp(ctx, a_log.grad, dt_bias.grad)
    torch.cuda.synchronize()
    torch.save({"o": out.detach().cpu(), "dq": leaves["q"].grad.cpu(), "dk": leaves["k"].grad.cpu(),
                "dv": leaves["v"].grad.cpu(), "dg": raw.grad.cpu(), "dbeta": leaves["beta"].grad.cpu(),
                "dA_log": da.cpu(), "ddt_bias": db.cpu()}, f"{out_dir}/rank{rank}.pt")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("layout", list(LAYOUTS))
def test_two_ranks_against_one_gpu(tmp_path, layout):
    import torch.multiprocessing as mp

    from miles_ext_kernels_b200.cake import kda
    from oracle import gdn_oracle as O

    seq_lens = LAYOUTS[layout]
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), seq_lens), nprocs=2, join=True)
    dev = torch.device("cuda", 0)
    H = 2
    x = draw(sum(seq_lens), H, 23)
    gen = torch.Generator().manual_seed(7)
    a_log = (torch.rand(H, generator=gen) * 1.5).to(dev).requires_grad_(True)
    dt_bias = (0.5 * torch.randn(H * 128, generator=gen)).to(dev).requires_grad_(True)
    cu = (0, seq_lens[0], sum(seq_lens))
    leaves = {n: x[n].to(dev).requires_grad_(True) for n in ("q", "k", "v", "g", "beta")}
    raw = (10.0 * leaves["g"].detach()).bfloat16().requires_grad_(True)
    out = kda.chunk_kda(leaves["q"], leaves["k"], leaves["v"], raw, leaves["beta"],
                        torch.tensor(cu, dtype=torch.int32, device=dev), use_gate_in_kernel=True, A_log=a_log,
                        dt_bias=dt_bias, use_qk_l2norm_in_kernel=True)
    out.backward(x["do"].to(dev))
    torch.cuda.synchronize()
    want = {"o": out.detach().cpu(), "dq": leaves["q"].grad.cpu(), "dk": leaves["k"].grad.cpu(),
            "dv": leaves["v"].grad.cpu(), "dg": raw.grad.cpu(), "dbeta": leaves["beta"].grad.cpu()}
    parts = [torch.load(tmp_path / f"rank{r}.pt") for r in range(2)]
    for name, ref in want.items():
        got = torch.cat([p[name] for p in parts], 0)
        if layout == "aligned":
            assert torch.equal(got, ref), name
        else:
            ok, m = O.within_budget(got.float(), ref.float(), rel_rms_max=6e-3, max_abs_rel=2e-2)
            assert ok, (name, m)
    # the parameter gradients: the same bits on both ranks, and the single-GPU sums within fp32 reassociation
    for name, ref in (("dA_log", a_log.grad.cpu()), ("ddt_bias", dt_bias.grad.cpu())):
        assert torch.equal(parts[0][name], parts[1][name]), name
        ok, m = O.within_budget(parts[0][name].float(), ref.float(), rel_rms_max=6e-3, max_abs_rel=2e-2)
        assert ok, (name, m)
