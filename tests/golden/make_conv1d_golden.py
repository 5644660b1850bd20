"""Writes ``conv1d_reference_*.pt``: seeded BF16 inputs and the outputs of the REFERENCE's own FP64 restatement of
the short convolution, ``reference`` / ``dweight_partial`` of tests/cake/conv1d/_kcp.py, imported from the reference
tree and run on the CPU.  Run where the reference is mounted:

    python tests/golden/make_conv1d_golden.py /path/to/reference
"""

import importlib.util
import sys
from pathlib import Path

import torch

CASES = {"s63_c384": (63, 384, (1, 2, 3, 57)), "s200_c136": (200, 136, (2, 0, 3, 120, 75))}


def main(reference_root: str) -> None:
    path = Path(reference_root) / "tests" / "cake" / "conv1d" / "_kcp.py"
    spec = importlib.util.spec_from_file_location("reference_conv1d_kcp", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    out_dir = Path(__file__).parent
    for name, (S, C, docs) in CASES.items():
        gen = torch.Generator().manual_seed(S * 7919 + C * 31)
        x = torch.randn(S, C, generator=gen).bfloat16()
        w = 0.5 * torch.randn(C, 4, generator=gen)
        dy = torch.randn(S, C, generator=gen).bfloat16()
        cu = [0]
        for n in docs:
            cu.append(cu[-1] + n)
        y, dx, dpre, taps_inputs = module.reference(x, w, cu, dy)
        dw = module.dweight_partial(dpre, taps_inputs, torch.arange(S))
        torch.save({"x": x, "w": w, "dy": dy, "cu": cu, "y": y, "dx": dx, "dw": dw}, out_dir / f"conv1d_reference_{name}.pt")
        print(name, tuple(y.shape), tuple(dw.shape))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(f"usage: python {sys.argv[0]} <reference root>")
    main(sys.argv[1])
