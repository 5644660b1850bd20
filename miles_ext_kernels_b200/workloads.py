"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configurations of the
gated-delta-rule path.  Inputs are drawn on the host from one ``torch.Generator`` per configuration, in a fixed
order, in FP32, then cast: ``q, k ~ N(0, 1)`` L2-normalised per head, ``v ~ N(0, 1)``, ``beta = sigmoid(N(0, 1))``,
``g = -softplus(N(0, 1)) * exp(U(0, ln 16))`` per token and head, ``dO ~ N(0, 1)``, and where a configuration says so
``h0 ~ 0.02 N(0, 1)`` per sequence.

No dataset or public benchmark is involved: the reference measures this path on synthetic tensors too.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

__all__ = ["CONFIGS", "Workload", "make_workload", "flops_per_token", "bytes_per_token"]


@dataclass(frozen=True)
class Config:
    name: str
    op: str  # "gdn" or "kda"
    seed: int
    batch: int  # leading dimension of the call (1 when packed)
    seq_lens: tuple[int, ...]  # per sequence (packed) or the common length repeated `batch` times
    num_qk_heads: int
    num_v_heads: int
    head_dim: int = 128
    dtype: str = "bf16"
    initial_state: bool = False
    final_state: bool = False
    packed: bool = False
    description: str = ""


def _varlen_lengths(total: int, lo: int, hi: int, seed: int) -> tuple[int, ...]:
    gen = torch.Generator().manual_seed(seed)
    lens: list[int] = []
    while sum(lens) < total:
        lens.append(int(torch.randint(lo, hi + 1, (1,), generator=gen)))
    lens[-1] -= sum(lens) - total
    return tuple(lens)


CONFIGS = {
    "cfg0": Config("cfg0", "gdn", 0, 1, (256,), 4, 4, head_dim=64, dtype="fp32",
                   description="CPU plumbing: B=1, T=256, H=HV=4, dk=dv=64, fp32, zero initial state"),
    "cfg1": Config("cfg1", "gdn", 1, 4, (8192,) * 4, 16, 32, final_state=True,
                   description="GDN fwd+bwd, bf16, fp32 state, GVA heads: B=4, T=8192, H_qk=16, H_v=32, d=128"),
    "cfg2": Config("cfg2", "gdn", 2, 1, _varlen_lengths(65536, 256, 8192, 2), 32, 32, initial_state=True,
                   final_state=True, packed=True,
                   description="GDN varlen packed: 65,536 tokens, lengths U[256, 8192], H=32, d=128, h0 ~ N(0, 0.02)"),
    "cfg3": Config("cfg3", "kda", 3, 1, (4096,), 32, 32, packed=True,
                   description="KDA per-channel decay: one T=4096 sequence per GPU (B=8 over 8 GPUs), H=32, d=128"),
    "cfg4": Config("cfg4", "gdn", 4, 1, (32768,), 32, 32, packed=True,
                   description="long-context GDN: one rank's 32,768-token slice of a T=262,144 sequence, H=32, d=128"),
}


@dataclass
class Workload:
    """Host tensors of one configuration (pinned when CUDA is available) in the call's shapes ``[B, T, heads, ...]``."""

    config: Config
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    g: torch.Tensor
    beta: torch.Tensor
    do: torch.Tensor
    h0: torch.Tensor | None = None
    dht: torch.Tensor | None = None
    cu_seqlens: tuple[int, ...] | None = None
    extra: dict = field(default_factory=dict)

    @property
    def num_tokens(self) -> int:
        return self.q.shape[0] * self.q.shape[1]


def make_workload(name: str, *, tokens: int | None = None, heads: tuple[int, int] | None = None,
                  seed: int | None = None) -> Workload:
    """The workload of configuration ``name``; ``tokens`` / ``heads`` cut it down to a bounded sample of the same
    distributions (used by the CPU baseline and by small parity cases); ``seed`` replaces the configuration's own
    (ranks that each hold their own piece of a sharded workload draw different values)."""
    cfg = CONFIGS[name]
    H, HV = heads or (cfg.num_qk_heads, cfg.num_v_heads)
    d = cfg.head_dim
    seq_lens = list(cfg.seq_lens)
    if tokens is not None:
        if cfg.packed:
            kept, total = [], 0
            for length in seq_lens:
                take = min(length, tokens - total)
                if take <= 0:
                    break
                kept.append(take)
                total += take
            seq_lens = kept
        else:
            seq_lens = [max(1, tokens // cfg.batch)] * cfg.batch
    if cfg.packed:
        B, T = 1, sum(seq_lens)
    else:
        B, T = cfg.batch, seq_lens[0]
    gen = torch.Generator().manual_seed(cfg.seed if seed is None else seed)
    q = torch.randn(B, T, H, d, generator=gen)
    k = torch.randn(B, T, H, d, generator=gen)
    v = torch.randn(B, T, HV, d, generator=gen)
    beta = torch.sigmoid(torch.randn(B, T, HV, generator=gen))
    a = torch.randn(B, T, HV, generator=gen)
    u = torch.rand(B, T, HV, generator=gen)
    g = -torch.nn.functional.softplus(a) * torch.exp(u * math.log(16.0))
    do = torch.randn(B, T, HV, d, generator=gen)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6)
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    num_seqs = len(seq_lens) if cfg.packed else B
    h0 = 0.02 * torch.randn(num_seqs, HV, d, d, generator=gen) if cfg.initial_state else None
    dht = torch.randn(num_seqs, HV, d, d, generator=gen) if cfg.initial_state else None
    if cfg.op == "kda":  # per-key-channel gate: g [B, T, H, d] = -softplus(N(0, 1)) exp(A_log), A_log ~ U(0, ln 16)
        a_log = torch.rand(H, generator=gen) * math.log(16.0)
        g = -torch.nn.functional.softplus(torch.randn(B, T, H, d, generator=gen)) * torch.exp(a_log)[None, None, :, None]
    low = torch.bfloat16 if cfg.dtype == "bf16" else torch.float32
    cu = None
    if cfg.packed:
        cu, at = [0], 0
        for length in seq_lens:
            at += length
            cu.append(at)
        cu = tuple(cu)
    work = Workload(cfg, q.to(low), k.to(low), v.to(low), g, beta.to(low), do.to(low), h0, dht, cu)
    if torch.cuda.is_available():
        for name_ in ("q", "k", "v", "g", "beta", "do", "h0", "dht"):
            t = getattr(work, name_)
            if t is not None:
                setattr(work, name_, t.pin_memory())
    return work


# --------------------------------------------------------------------------------------------------------------------
# roofline arithmetic (per token; C = 64, d = 128)
# --------------------------------------------------------------------------------------------------------------------
def flops_per_token(num_v_heads: int, chunk: int = 64, d: int = 128) -> float:
    """Algorithmic FLOPs of forward + backward per token: every dense chunk contraction counted as ``2 m n k``
    (no triangular discount), per (chunk, value head), divided by the chunk's tokens."""
    c2d, cd2, c3 = 2 * chunk * chunk * d, 2 * chunk * d * d, 2 * chunk**3
    forward = c2d + c3 / 3 + 2 * c2d + 3 * cd2 + 2 * c2d
    backward = 12 * c2d + 6 * cd2 + 2 * c3
    return (forward + backward) / chunk * num_v_heads


def bytes_per_token(num_qk_heads: int, num_v_heads: int, d: int = 128, op: str = "gdn") -> float:
    """Compulsory HBM bytes of forward + backward per token: the forward reads q, k, v, g, beta and writes o; the
    backward reads q, k, v, g, beta, dO and writes dq, dk, dv, dg, dbeta (bf16 = 2 B, g fp32, beta bf16)."""
    row = 2 * d
    if op == "kda":  # g and dg are [., d] fp32 per head
        return num_v_heads * (3 * 2 * row + 5 * row + 3 * 2 + 3 * 4 * d)
    return 3 * (2 * num_qk_heads * row) + 5 * (num_v_heads * row) + 3 * (num_v_heads * 6)
