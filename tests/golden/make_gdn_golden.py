"""Generate ``gdn_fake_backend_*.pt``: inputs and outputs of the REFERENCE's own torch emulation of the GDN path.

Run once, in a container that has the reference checked out (it is not needed to run the tests)::

    PYTHONPATH=<reference root>:<reference root>/tests python tests/golden/make_gdn_golden.py

The call is the reference's public entry point ``miles_ext_kernels.cake.gdn.chunk_gated_delta_rule`` with a one-rank
CPU ``KcpContext`` and the packages' emulation backend selected (``ops.KCP_OPTIONS = {"backend": "fake"}``), exactly
as the reference's own test drives it (reference: tests/cake/gdn/test_gdn_kcp_wiring.py:410-444).  Inputs are drawn
from a seeded CPU generator; everything is stored as it came back (bf16 / fp32).
"""

from __future__ import annotations

import itertools
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
HEAD_DIM = 128

CASES = {
    # name: (seq_lens, (H, HV), seed, use_qk_l2norm, gate)
    "weak_gva": ((130, 63, 77), (2, 4), 11, True, "weak"),
    "weak_mha": ((64, 200), (2, 2), 12, False, "weak"),
    "strong_gva": ((257, 31), (1, 2), 13, True, "strong"),
}


def draw(seq_lens, heads, seed, l2norm, gate):
    H, HV = heads
    T = sum(seq_lens)
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(1, T, H, HEAD_DIM, generator=gen)
    k = torch.randn(1, T, H, HEAD_DIM, generator=gen)
    if not l2norm:
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6)
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    v = torch.randn(1, T, HV, HEAD_DIM, generator=gen)
    beta = torch.sigmoid(torch.randn(1, T, HV, generator=gen))
    a = torch.randn(1, T, HV, generator=gen)
    u = torch.rand(1, T, HV, generator=gen)
    if gate == "weak":
        g = -0.5 * u
    else:
        g = -torch.nn.functional.softplus(a) * torch.exp(u * torch.log(torch.tensor(16.0)))
    do = torch.randn(1, T, HV, HEAD_DIM, generator=gen)
    return {"q": q.bfloat16(), "k": k.bfloat16(), "v": v.bfloat16(), "g": g, "beta": beta.bfloat16(),
            "do": do.bfloat16()}


def main() -> None:
    from miles_ext_kernels import cake
    from miles_ext_kernels.cake._impl.gdn import ops
    from miles_ext_kernels.cake._impl.gdn.kcp import KcpContext

    ops.KCP_OPTIONS = {"backend": "fake"}
    cake.configure(cake_gdn_variant="det")
    for name, (seq_lens, heads, seed, l2norm, gate) in CASES.items():
        inputs = draw(seq_lens, heads, seed, l2norm, gate)
        cu = tuple(itertools.accumulate(seq_lens, initial=0))
        ctx = KcpContext(cu, None, 0, 1, torch.device("cpu"), 4, "contiguous", None)
        leaves = {n: t.detach().clone().requires_grad_(True) for n, t in inputs.items() if n != "do"}
        out, _ = ops.chunk_gated_delta_rule(
            **{n: leaves[n] for n in ("q", "k", "v", "g", "beta")}, use_qk_l2norm_in_kernel=l2norm, cp_context=ctx
        )
        out.backward(inputs["do"])
        record = {
            "seq_lens": seq_lens, "heads": heads, "seed": seed, "use_qk_l2norm": l2norm, "gate": gate,
            "inputs": inputs,
            "outputs": {"o": out.detach(), **{f"d{n}": t.grad for n, t in leaves.items()}},
        }
        torch.save(record, HERE / f"gdn_fake_backend_{name}.pt")
        print(name, {n: (tuple(t.shape), str(t.dtype)) for n, t in record["outputs"].items()})


if __name__ == "__main__":
    sys.exit(main())
