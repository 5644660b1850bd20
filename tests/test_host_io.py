"""The host-memory pipeline: how a call is cut into parts (CPU) and that the parts' results are the bits of the
undivided call (GPU)."""

import pytest
import torch

from miles_ext_kernels_b200 import host_io


def test_batch_parts_cover_the_rows_once():
    for batch in (1, 3, 4, 7):
        for n in (None, 1, 2, 5, 16):
            parts = host_io.batch_parts(batch, n)
            rows = [r for p in parts for r in range(p.rows.start, p.rows.stop)]
            assert rows == list(range(batch))
            assert all(p.cu_seqlens is None and p.tokens == slice(None) for p in parts)
    with pytest.raises(ValueError):
        host_io.batch_parts(0)


def test_packed_parts_keep_sequences_whole():
    cu = (0, 100, 100, 420, 900, 1000, 4096)
    for n in (1, 2, 3, 6, 12):
        parts = host_io.packed_parts(cu, n)
        assert len(parts) <= n
        assert parts[0].tokens.start == 0 and parts[-1].tokens.stop == cu[-1]
        assert parts[0].seqs.start == 0 and parts[-1].seqs.stop == len(cu) - 1
        for a, b in zip(parts, parts[1:]):
            assert a.tokens.stop == b.tokens.start and a.seqs.stop == b.seqs.start
        for p in parts:
            assert p.cu_seqlens[0] == 0 and p.cu_seqlens[-1] == p.tokens.stop - p.tokens.start
            assert tuple(x + p.tokens.start for x in p.cu_seqlens) == cu[p.seqs.start:p.seqs.stop + 1]
    with pytest.raises(ValueError):
        host_io.packed_parts((1, 5), 2)


def _inputs(B, T, H, HV, seed):
    gen = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(B, T, H, 128, generator=gen), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(B, T, H, 128, generator=gen), dim=-1)
    v = torch.randn(B, T, HV, 128, generator=gen)
    g = -torch.nn.functional.softplus(torch.randn(B, T, HV, generator=gen))
    beta = torch.sigmoid(torch.randn(B, T, HV, generator=gen))
    do = torch.randn(B, T, HV, 128, generator=gen)
    low = torch.bfloat16
    return {"q": q.to(low), "k": k.to(low), "v": v.to(low), "g": g, "beta": beta.to(low), "do": do.to(low)}


@pytest.mark.gpu
@pytest.mark.parametrize("packed", [False, True], ids=["batch", "packed"])
def test_pipeline_lands_the_bits_of_the_undivided_call(packed):
    from miles_ext_kernels_b200.cake import gdn

    device = torch.device("cuda")
    H, HV = 2, 4
    if packed:
        cu = (0, 300, 364, 1000, 1500, 2048)
        host = _inputs(1, cu[-1], H, HV, 11)
        num_seqs = len(cu) - 1
        parts = host_io.packed_parts(cu, 3)
    else:
        cu = None
        host = _inputs(3, 512, H, HV, 12)
        num_seqs = 3
        parts = host_io.batch_parts(3)
    gen = torch.Generator().manual_seed(5)
    host["h0"] = 0.1 * torch.randn(num_seqs, HV, 128, 128, generator=gen)
    host = {n: t.pin_memory() for n, t in host.items()}

    def step(t, cu_cpu):
        q, k, v, g, beta, h0 = (t[n].detach().requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0"))
        cu_dev = None if cu_cpu is None else torch.tensor(cu_cpu, dtype=torch.int32, device=device)
        o, final = gdn.chunk_gated_delta_rule(q, k, v, g=g, beta=beta, initial_state=h0, output_final_state=True,
                                              cu_seqlens=cu_dev, cu_seqlens_cpu=cu_cpu)
        o.backward(t["do"])
        return [o, q.grad, k.grad, v.grad, g.grad, beta.grad, h0.grad, final]

    want = step({n: t.to(device) for n, t in host.items()}, cu)
    pipe = host_io.HostPipeline(device, parts, per_token=("q", "k", "v", "g", "beta", "do"))
    total = (host["q"].shape[0], host["q"].shape[1], num_seqs)
    for _ in range(2):  # the second call reuses the staging and landing buffers
        got = pipe.run(host, lambda part, t: step(t, part.cu_seqlens), range(6), total)
        torch.cuda.synchronize()
        for i, (a, b) in enumerate(zip(got, want)):
            assert a.is_pinned() and torch.equal(a, b.detach().cpu()), i
    with pytest.raises(ValueError, match="pinned"):
        pipe.run({n: t.clone() for n, t in host.items()}, lambda part, t: step(t, part.cu_seqlens), range(6), total)
