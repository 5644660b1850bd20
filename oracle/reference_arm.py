"""The reference's own CPU implementation of the GDN path, run from ``oracle/_ref/`` (made by ``oracle/make_ref.py``).

Test infrastructure: only ``tests/``, the smoke check and the CPU legs of ``bench.py`` import this module; the product
never does.  The call is the reference's public entry point with its emulation backend selected and a one-rank CPU
``KcpContext`` (reference: tests/cake/gdn/test_gdn_kcp_wiring.py:410-444; semantics
miles_ext_kernels/cake/_vendor/cake_gdn_det_train_kcp/cake_fake_backend.py:173-640).  Limits of that path: head
dims 128, bf16 q / k / v, packed ``[1, T, ...]`` operands with the context's boundaries, no initial and no final
state (the context-parallel contract).
"""

from __future__ import annotations

import sys
from pathlib import Path

import torch

REF_ROOT = Path(__file__).resolve().parent / "_ref"

_entry = None


def available() -> bool:
    return (REF_ROOT / "miles_ext_kernels" / "cake" / "_impl" / "gdn" / "ops.py").is_file()


def _load():
    global _entry
    if _entry is None:
        if not available():
            raise RuntimeError("oracle/_ref is absent: run `python oracle/make_ref.py <reference checkout>` first")
        if str(REF_ROOT) not in sys.path:
            sys.path.insert(0, str(REF_ROOT))
        from miles_ext_kernels import cake
        from miles_ext_kernels.cake._impl.gdn import ops
        from miles_ext_kernels.cake._impl.gdn.kcp import KcpContext

        ops.KCP_OPTIONS = {"backend": "fake"}
        cake.configure(cake_gdn_variant="det")
        _entry = (ops, KcpContext)
    return _entry


def forward_backward(q, k, v, g, beta, do, cu_seqlens, use_qk_l2norm: bool = False, scale=None) -> dict:
    """q, k ``[T, H, 128]`` bf16, v, do ``[T, HV, 128]`` bf16, g ``[T, HV]`` fp32, beta ``[T, HV]`` bf16, ``cu_seqlens`` a
    tuple of ints.  Returns ``{"o", "dq", "dk", "dv", "dg", "dbeta"}`` as the reference's CPU path gives them."""
    ops, KcpContext = _load()
    context = KcpContext(tuple(int(b) for b in cu_seqlens), None, 0, 1, torch.device("cpu"), 4, "contiguous", None)
    leaves = {n: t.detach().clone().unsqueeze(0).requires_grad_(True)
              for n, t in dict(q=q, k=k, v=v, g=g, beta=beta).items()}
    out, _ = ops.chunk_gated_delta_rule(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], scale=scale,
                                        use_qk_l2norm_in_kernel=use_qk_l2norm, cp_context=context)
    out.backward(do.unsqueeze(0))
    return {"o": out.detach()[0], **{f"d{n}": t.grad[0] for n, t in leaves.items()}}
