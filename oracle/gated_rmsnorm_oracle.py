"""CPU oracle of the SiLU-gated RMSNorm (TEST INFRASTRUCTURE: only tests, the smoke check and the benchmark's CPU
baseline may import it; the product path never does).

FP64 forward and closed-form backward from the BF16 inputs, and the accuracy gates of the reference's GPU tests
(reference: tests/cake/gated_rmsnorm/inputs.py:75-95, tests/cake/gated_rmsnorm/test_gated_rmsnorm_gpu.py:30-75).
Pinned by ``tests/golden/gated_rmsnorm_reference_*.pt``: outputs of the reference's own ``fp64_reference`` on seeded
CPU inputs (``tests/golden/make_gated_rmsnorm_golden.py``).
"""

from __future__ import annotations

import torch

D = 128
BF16_RTOL = 2.0**-7  # one BF16 ulp relative to the value
DW_MAG_TOL = 2.0**-20  # the FP32 accumulation term of the weight-gradient bound, relative to sum |terms|


def fp64_reference(dy: torch.Tensor, x: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> dict:
    """``y, dx, dz, dw`` and ``mag`` (the sum of ``|terms|`` of each weight-gradient column), all FP64."""
    xd, zd, wd, gd = x.double(), z.double(), w.double(), dy.double()
    rstd = 1.0 / torch.sqrt(xd.square().mean(dim=-1, keepdim=True) + eps)
    n = xd * rstd
    s = torch.sigmoid(zd)
    silu = zd * s
    a = gd * silu
    dn = a * wd
    terms = (a * n).reshape(-1, D)
    return {
        "y": n * wd * silu,
        "dx": rstd * dn - xd * rstd**3 * (dn * xd).mean(dim=-1, keepdim=True),
        "dz": gd * n * wd * s * (1.0 + zd * (1.0 - s)),
        "dw": terms.sum(dim=0),
        "mag": terms.abs().sum(dim=0),
    }


def bf16_misses(got: torch.Tensor, want: torch.Tensor) -> int:
    """Elements of ``got`` beyond one BF16 ulp of ``want`` plus a floor of 1/64 ulp of its largest magnitude."""
    want = want.double()
    floor = want.abs().max().item() * BF16_RTOL / 64
    return int(((got.double() - want).abs() > want.abs() * BF16_RTOL + floor).sum())


def dw_misses(dw: torch.Tensor, want: torch.Tensor, mag: torch.Tensor, rtol_of: torch.Tensor | None = None) -> int:
    """Columns with ``|dw - want| > |rtol_of| * 2^-7 + sum|terms| * 2^-20`` (``rtol_of`` defaults to ``want``)."""
    rtol_of = want if rtol_of is None else rtol_of
    return int(((dw.double() - want).abs() > rtol_of.abs() * BF16_RTOL + mag * DW_MAG_TOL).sum())
