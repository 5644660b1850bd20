"""Seeded inputs of the GDN tests, packed ``[T, heads, 128]``, drawn on the host."""

from __future__ import annotations

import math

import torch


def draw(seq_lens, heads, *, seed=0, gate="weak", state=False, normalised=False, dim=128):
    """q, k (bf16; L2-normalised per head when ``normalised``), v, do (bf16), g (fp32), beta (fp32 holding bf16
    values), and h0 / dht (fp32) when ``state``."""
    H, HV = heads
    T = sum(seq_lens)
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(T, H, dim, generator=gen)
    k = torch.randn(T, H, dim, generator=gen)
    if normalised:
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6)
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    v = torch.randn(T, HV, dim, generator=gen)
    beta = torch.sigmoid(torch.randn(T, HV, generator=gen))
    a = torch.randn(T, HV, generator=gen)
    u = torch.rand(T, HV, generator=gen)
    if gate == "weak":
        g = -0.5 * u
    elif gate == "strong":
        g = -torch.nn.functional.softplus(a) * torch.exp(u * math.log(16.0))
    else:
        raise ValueError(gate)
    do = torch.randn(T, HV, dim, generator=gen)
    out = {
        "q": q.bfloat16(), "k": k.bfloat16(), "v": v.bfloat16(), "g": g, "beta": beta.bfloat16().float(),
        "do": do.bfloat16(),
    }
    if state:
        out["h0"] = 0.1 * torch.randn(len(seq_lens), HV, dim, dim, generator=gen)
        out["dht"] = 0.1 * torch.randn(len(seq_lens), HV, dim, dim, generator=gen)
    return out


def to_token_major(x_c, table):
    """Oracle chunk-major ``[NC, heads, 64, ...]`` -> packed ``[T, heads, ...]``."""
    rows = []
    for c, length in enumerate(table.chunk_len):
        rows.append(x_c[c].transpose(0, 1)[:length])
    return torch.cat(rows, 0)
