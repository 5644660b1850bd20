"""CPU oracle of KDA (the gated delta rule with a per-key-channel decay).  TEST INFRASTRUCTURE ONLY (see
``oracle/__init__.py``).

* :func:`recurrence_fp64` -- the exact per-document token recurrence with autograd, zero initial state (reference:
  tests/cake/kda/_reference.py:102-142): ``S = S * exp(g_t)[:, None]; S = S + (beta_t k_t) (x) (v_t - k_t^T S);
  o_t = scale q_t^T S``; optional raw gate ``g = lb * sigmoid(exp(A_log)(raw + dt_bias))`` (reference: :86-99) and
  in-op q / k L2 norm.
* :func:`chunked_forward` / :func:`chunked_backward` -- the chunked algorithm (chunk 64) the CUDA kernels implement,
  stage by stage, with their BF16 rounding points: the model for the stage-level parity tests.

Parity pinned: ``tests/golden/kda_reference_*.pt`` hold outputs of the reference's own FP64 oracle
(``tests/golden/make_kda_golden.py``); ``tests/test_oracle_kda.py`` checks both restatements against them.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .gdn_oracle import BF16, CHUNK, F32, F64, L2NORM_EPS, ChunkTable, _gather, _rounder, chunk_table
from .gdn_oracle import l2norm_forward, l2norm_pullback

LOWER_BOUND = -5.0


def raw_gate(raw, A_log, dt_bias, lower_bound=LOWER_BOUND, dtype=F32):
    """``lower_bound * sigmoid(exp(A_log)[h] * (raw + dt_bias[h]))`` for ``raw [..., H, D]``."""
    H, D = raw.shape[-2], raw.shape[-1]
    a = torch.exp(A_log.to(dtype)).reshape(H, 1)
    return lower_bound * torch.sigmoid(a * (raw.to(dtype) + dt_bias.to(dtype).reshape(H, D)))


def recurrence_fp64(q, k, v, g, beta, seq_lens, *, scale=None, do=None, use_qk_l2norm=False, A_log=None,
                    dt_bias=None, lower_bound=LOWER_BOUND, dtype=F64):
    """q, k, v, g ``[T, H, D]``; beta ``[T, H]``.  With ``A_log`` / ``dt_bias`` the gate ``g`` is raw.  Returns
    ``{o}`` and, with ``do``, ``{dq, dk, dv, dg, dbeta[, dA_log, ddt_bias]}`` in ``dtype``."""
    want = do is not None
    leaf = lambda t: t.detach().to(dtype).requires_grad_(want)  # noqa: E731
    q_, k_, v_, g_, b_ = (leaf(t) for t in (q, k, v, g, beta))
    params = []
    gate = g_
    if A_log is not None:
        a_, d_ = leaf(A_log), leaf(dt_bias)
        params = [a_, d_]
        gate = raw_gate(g_, a_, d_, lower_bound, dtype)
    T, H, D = q_.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    qf, kf = q_, k_
    if use_qk_l2norm:
        qf = qf / torch.sqrt((qf * qf).sum(-1, keepdim=True) + L2NORM_EPS)
        kf = kf / torch.sqrt((kf * kf).sum(-1, keepdim=True) + L2NORM_EPS)
    outs = []
    at = 0
    for length in seq_lens:
        S = torch.zeros(H, D, v_.shape[-1], dtype=dtype)
        for t in range(at, at + length):
            S = S * torch.exp(gate[t])[:, :, None]
            pred = torch.einsum("hk,hkv->hv", kf[t], S)
            S = S + torch.einsum("hk,hv->hkv", b_[t][:, None] * kf[t], v_[t] - pred)
            outs.append(scale * torch.einsum("hk,hkv->hv", qf[t], S))
        at += length
    o = torch.stack(outs) if outs else torch.zeros_like(v_)
    result = {"o": o.detach()}
    if want:
        grads = torch.autograd.grad(o, [q_, k_, v_, g_, b_, *params], do.to(dtype))
        result.update(dq=grads[0], dk=grads[1], dv=grads[2], dg=grads[3], dbeta=grads[4])
        if params:
            result.update(dA_log=grads[5], ddt_bias=grads[6])
    return result


@dataclass
class KdaTape:
    table: ChunkTable
    index: torch.Tensor
    mask: torch.Tensor
    scale: float
    q: torch.Tensor  # [NC, H, 64, D] normalised rows
    k: torch.Tensor
    v: torch.Tensor
    beta: torch.Tensor  # [NC, H, 64]
    G: torch.Tensor  # [NC, H, 64, D] chunk-local cumulative gate (natural log)
    qg: torch.Tensor  # rounded q e^G
    kg: torch.Tensor  # rounded k e^G
    kr: torch.Tensor  # rounded k e^{G_L - G}
    A: torch.Tensor
    Aqk: torch.Tensor
    w: torch.Tensor
    u: torch.Tensor
    h: torch.Tensor
    v_new: torch.Tensor
    q_raw: torch.Tensor | None = None
    k_raw: torch.Tensor | None = None
    q_rstd: torch.Tensor | None = None
    k_rstd: torch.Tensor | None = None


def _pair_decay(G):
    """``e^{G_i - G_j}`` per channel for ``i >= j`` (zero above the diagonal): ``[..., 64, 64, D]``."""
    diff = G[..., :, None, :] - G[..., None, :, :]
    lower = torch.ones(G.shape[-2], G.shape[-2], dtype=torch.bool).tril()[..., None]
    return torch.where(lower, diff, torch.full_like(diff, float("-inf"))).exp()


def chunked_forward(q, k, v, g, beta, seq_lens, *, scale=None, use_qk_l2norm=False, rounding="bf16"):
    """Forward of chunked KDA.  Returns ``(o [T, H, D] fp32 holding rounded values, tape)``."""
    rnd = _rounder(rounding)
    T, H, D = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    table = chunk_table(seq_lens)
    NC = table.num_chunks
    starts = torch.tensor(table.chunk_start, dtype=torch.long)
    lens = torch.tensor(table.chunk_len, dtype=torch.long)
    offs = torch.arange(CHUNK)
    mask = (offs[None, :] < lens[:, None]).to(F32)
    index = (starts[:, None] + offs[None, :]).clamp(max=max(T - 1, 0))
    q_raw = k_raw = q_rstd = k_rstd = None
    qn, kn = q.to(F32), k.to(F32)
    if use_qk_l2norm:
        q_raw, k_raw = qn, kn
        qn, q_rstd = l2norm_forward(qn, rnd)
        kn, k_rstd = l2norm_forward(kn, rnd)
    qc = _gather(qn, index, mask).permute(0, 2, 1, 3)  # [NC, H, 64, D]
    kc = _gather(kn, index, mask).permute(0, 2, 1, 3)
    vc = _gather(v, index, mask).permute(0, 2, 1, 3)
    gc = _gather(g, index, mask).permute(0, 2, 1, 3)
    bc = _gather(beta, index, mask).permute(0, 2, 1)
    G = torch.cumsum(gc, dim=2)
    GL = G[:, :, -1:, :]
    qg, kg, kr = rnd(qc * G.exp()), rnd(kc * G.exp()), rnd(kc * (GL - G).exp())
    E = _pair_decay(G)  # [NC, H, 64, 64, D]
    Sqk = torch.einsum("chid,chjd,chijd->chij", qc, kc, E)
    Skk = torch.einsum("chid,chjd,chijd->chij", kc, kc, E)
    Aqk = rnd((scale * Sqk).tril())
    L = (bc[..., None] * Skk).tril(-1)
    eye = torch.eye(CHUNK, dtype=F32)
    A = rnd(torch.linalg.solve_triangular(eye + L, eye.expand_as(L), upper=False, unitriangular=True))
    kb = rnd(kg * bc[..., None])
    vb = rnd(vc * bc[..., None])
    w, u = rnd(torch.matmul(A, kb)), rnd(torch.matmul(A, vb))
    gamma = GL[:, :, 0, :].exp()  # [NC, H, D]
    h_tape = torch.zeros(NC, H, D, v.shape[-1], dtype=F32)
    v_new = torch.zeros(NC, H, CHUNK, v.shape[-1], dtype=F32)
    for n in range(len(seq_lens)):
        h = torch.zeros(H, D, v.shape[-1], dtype=F32)
        for c in range(table.seq_chunk_start[n], table.seq_chunk_start[n + 1]):
            hb = rnd(h)
            h_tape[c] = hb
            b_v = u[c] - torch.matmul(w[c], hb)
            v_new[c] = rnd(b_v)
            h = gamma[c][..., None] * h + torch.matmul(kr[c].transpose(-1, -2), rnd(b_v))
    o_c = rnd(scale * torch.matmul(qg, h_tape) + torch.matmul(Aqk, v_new))
    o = torch.zeros(T, H, v.shape[-1], dtype=F32)
    valid = mask.bool()
    o[index[valid]] = o_c.permute(0, 2, 1, 3)[valid]
    tape = KdaTape(table, index, mask, float(scale), qc, kc, vc, bc, G, qg, kg, kr, A, Aqk, w, u, h_tape, v_new,
                   q_raw, k_raw, q_rstd, k_rstd)
    return o, tape


def chunked_backward(t: KdaTape, do, *, rounding="bf16", round_grads=True):
    """Backward of chunked KDA: ``{dq, dk, dv [T, H, D]; dg [T, H, D]; dbeta [T, H]}`` (fp32)."""
    rnd = _rounder(rounding)
    out_rnd = rnd if round_grads else (lambda x: x)
    NC, H, D = t.q.shape[0], t.q.shape[1], t.q.shape[3]
    scale = t.scale
    G = t.G
    GL = G[:, :, -1:, :]
    gamma = GL[:, :, 0, :].exp()
    doc = _gather(do, t.index, t.mask).permute(0, 2, 1, 3)
    do_s = rnd(scale * doc)
    dv_intra = rnd(torch.matmul(t.Aqk.transpose(-1, -2), doc))
    dh_tape = torch.zeros_like(t.h)
    dv_new = torch.zeros_like(t.v_new)
    for n in range(len(t.table.seq_chunk_start) - 1):
        dh = torch.zeros(H, D, t.v.shape[-1], dtype=F32)
        for c in reversed(range(t.table.seq_chunk_start[n], t.table.seq_chunk_start[n + 1])):
            dhb = rnd(dh)
            dh_tape[c] = dhb
            dvb_ = rnd(dv_intra[c] + torch.matmul(t.kr[c], dhb))
            dv_new[c] = dvb_
            dh = (gamma[c][..., None] * dh + torch.matmul(t.qg[c].transpose(-1, -2), do_s[c])
                  - torch.matmul(t.w[c].transpose(-1, -2), dvb_))
    h, dh = t.h, dh_tape
    vn, dvn, bet = t.v_new, dv_new, t.beta
    E = _pair_decay(G)
    eG, eR = G.exp(), (GL - G).exp()
    # contractions on tensor cores in the kernels
    dqg = torch.matmul(do_s, h.transpose(-1, -2))  # d(q e^G)
    dkr = torch.matmul(vn, dh.transpose(-1, -2))  # d(k e^{G_L - G})
    dw = rnd(-torch.matmul(dvn, h.transpose(-1, -2)))
    At = t.A.transpose(-1, -2)
    dkgb = torch.matmul(At, dw)  # d(beta k e^G)
    dvb = torch.matmul(At, dvn)
    kb, vb = rnd(t.kg * bet[..., None]), rnd(t.v * bet[..., None])
    dA = rnd(torch.matmul(dw, kb.transpose(-1, -2)) + torch.matmul(dvn, vb.transpose(-1, -2)))
    dL = rnd(-torch.matmul(rnd(torch.matmul(At, dA)), At).tril(-1))
    M1 = scale * torch.matmul(doc, vn.transpose(-1, -2)).tril()  # d(q k decay) from Aqk
    M2 = dL  # gradient of L_ij = beta_i S_kk_ij
    # pairwise decayed contractions (CUDA cores in the kernels)
    RQ = torch.einsum("chij,chjd,chijd->chid", M1, t.k, E)
    CK = torch.einsum("chij,chid,chijd->chjd", M1, t.q, E)
    RK1 = torch.einsum("chij,chjd,chijd->chid", M2, t.k, E)  # without beta_i
    CL = torch.einsum("chij,chid,chijd->chjd", M2 * bet[..., None], t.k, E)
    RK = bet[..., None] * RK1
    dkg = bet[..., None] * dkgb
    dq_c = RQ + dqg * eG
    dk_c = CK + RK + CL + dkr * eR + dkg * eG
    dG = t.q * RQ - t.k * CK + t.k * RK - t.k * CL + dqg * t.qg + dkg * t.kg - dkr * t.kr
    chunk_end = (dkr * t.kr).sum(2) + gamma * (dh * h).sum(-1)  # [NC, H, D]: credited to the chunk's last token
    lens = torch.tensor(t.table.chunk_len, dtype=torch.long)
    part = dG * t.mask[:, None, :, None]
    part[torch.arange(NC), :, lens - 1, :] += chunk_end
    dg_c = torch.flip(torch.cumsum(torch.flip(part, [2]), 2), [2])
    dbeta = (dkgb * t.kg).sum(-1) + (dvb * t.v).sum(-1) + (RK1 * t.k).sum(-1)
    dv_c = out_rnd(dvb * bet[..., None])

    T = do.shape[0]
    valid = t.mask.bool()
    tok = t.index[valid]

    def scatter(x_c, width=None):
        out = torch.zeros((T, H) if width is None else (T, H, width), dtype=F32)
        moved = x_c.permute(0, 2, 1) if width is None else x_c.permute(0, 2, 1, 3)
        out[tok] = moved[valid]
        return out

    dq, dk = scatter(dq_c, D), scatter(dk_c, D)
    if t.q_raw is not None:
        dq = l2norm_pullback(t.q_raw, t.q_rstd, dq)
        dk = l2norm_pullback(t.k_raw, t.k_rstd, dk)
    return {"dq": out_rnd(dq), "dk": out_rnd(dk), "dv": scatter(dv_c, t.v.shape[-1]), "dg": scatter(dg_c, D),
            "dbeta": scatter(dbeta * t.mask[:, None, :]), "dh_tape": dh_tape, "dv_new": dv_new,
            "aux": {"dqg": dqg, "dkr": dkr, "dkg": dkg, "M1": M1, "M2": M2}}


def chunked_forward_backward(q, k, v, g, beta, seq_lens, do, *, scale=None, use_qk_l2norm=False, rounding="bf16"):
    o, tape = chunked_forward(q, k, v, g, beta, seq_lens, scale=scale, use_qk_l2norm=use_qk_l2norm, rounding=rounding)
    grads = chunked_backward(tape, do, rounding=rounding)
    return {"o": o, **{n: grads[n] for n in ("dq", "dk", "dv", "dg", "dbeta")}}
