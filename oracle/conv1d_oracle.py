"""CPU oracle of the packed causal depthwise conv1d + SiLU (TEST INFRASTRUCTURE: only tests, the smoke check and the
benchmark's CPU baseline may import it; the product path never does).

``pre[t, c] = sum_{k<4} w[c, k] x[t - 3 + k, c]`` inside token ``t``'s document; ``y = bf16(pre sigmoid(pre))``;
``dpre = dy silu'(p)``; ``dx[t] = sum_k w[c, k] dpre[t + 3 - k]``; ``dw[c, k] = sum_t dpre[t] x[t - 3 + k]``.
Two policies for ``p``: ``"fp32"`` -- everything in FP64, one rounding (reference:
tests/cake/conv1d/_kcp.py:290-326; pinned by ``tests/golden/conv1d_reference_*.pt``, outputs of that function run
on the CPU) -- and ``"bf16"`` -- FP32 preactivation, SiLU' at its BF16 rounding, as flash-linear-attention does
(reference: tests/cake/conv1d/test_conv1d_gpu.py:112-160, restated; that module needs a GPU to import).
"""

from __future__ import annotations

import torch

WIDTH = 4


def _shift(v: torch.Tensor, doc: torch.Tensor, d: int) -> torch.Tensor:
    """``out[t] = v[t - d]`` (``d > 0``) or ``v[t + |d|]`` (``d < 0``) inside token ``t``'s document, else 0."""
    out = torch.zeros_like(v)
    n = abs(d)
    if d == 0:
        return v.clone()
    if n >= v.shape[0]:
        return out
    if d > 0:
        out[n:] = torch.where((doc[n:] == doc[:-n]).unsqueeze(1), v[:-n], torch.zeros_like(v[:-n]))
    else:
        out[:-n] = torch.where((doc[:-n] == doc[n:]).unsqueeze(1), v[n:], torch.zeros_like(v[n:]))
    return out


def reference(x: torch.Tensor, w: torch.Tensor, cu, dy: torch.Tensor, policy: str = "fp32") -> dict:
    """``y, dx`` (BF16, one rounding each) and ``dw`` (FP64 ``[C, 4]``) of ``x, dy [S, C]`` BF16, taps ``w [C, 4]`` and
    the document offsets ``cu``."""
    S = x.shape[0]
    cu = torch.as_tensor(cu)
    doc = torch.bucketize(torch.arange(S), cu[1:].long(), right=True)
    if policy == "fp32":
        xf, wf = x.double(), w.double()
    elif policy == "bf16":
        xf, wf = x.float(), w.float()
    else:
        raise ValueError(policy)
    taps_inputs = [_shift(xf, doc, WIDTH - 1 - k) for k in range(WIDTH)]
    pre = torch.zeros_like(xf)
    for k in range(WIDTH):
        pre = pre + wf[:, k] * taps_inputs[k]
    y = (pre * torch.sigmoid(pre)).bfloat16()
    p = pre if policy == "fp32" else pre.bfloat16().float()
    s = torch.sigmoid(p)
    dpre = dy.to(xf.dtype) * (s * (1.0 + p * (1.0 - s)))
    dx = torch.zeros_like(dpre)
    for k in range(WIDTH):
        dx = dx + wf[:, k] * _shift(dpre, doc, -(WIDTH - 1 - k))
    dw = torch.stack([(dpre.double() * taps_inputs[k].double()).sum(0) for k in range(WIDTH)], dim=1)
    return {"y": y, "dx": dx.bfloat16(), "dw": dw}


def outside(actual: torch.Tensor, expected: torch.Tensor, *, atol: float, rtol: float) -> int:
    """Elements of ``actual`` outside ``atol + rtol * |expected|`` (non-finite ones count)."""
    a, b = actual.detach().double().reshape(-1), expected.detach().double().reshape(-1)
    bad = ~torch.isfinite(a) | ((a - b).abs() > atol + rtol * b.abs())
    return int(bad.sum())
