"""Writes ``gated_rmsnorm_reference_*.pt``: seeded BF16 inputs in the layer's layout (the gate a column slice of the
fused input projection) and the outputs of the REFERENCE's own FP64 closed form, ``fp64_reference`` of
tests/cake/gated_rmsnorm/inputs.py, imported from the reference tree and run on the CPU.  Run where the reference is
mounted:

    python tests/golden/make_gated_rmsnorm_golden.py /path/to/reference
"""

import importlib.util
import sys
from pathlib import Path

import torch

CASES = {"t7_hk6_hv12": (7, 6, 12, 0), "t9_hk8_hv16_extra8": (9, 8, 16, 8)}


def main(reference_root: str) -> None:
    path = Path(reference_root) / "tests" / "cake" / "gated_rmsnorm" / "inputs.py"
    spec = importlib.util.spec_from_file_location("reference_gated_rmsnorm_inputs", path)
    inputs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(inputs)
    out_dir = Path(__file__).parent
    for name, (tokens, hk, hv, extra) in CASES.items():
        gen = torch.Generator().manual_seed(tokens * 131 + hv)
        x = torch.randn(tokens, hv, 128, generator=gen).bfloat16()
        projection = torch.randn(tokens, inputs.projection_width(hk, hv, extra), generator=gen).bfloat16()
        start = (2 * hk + hv) * 128
        z = projection[:, start : start + hv * 128].unflatten(-1, (hv, 128))
        dy = torch.randn(tokens, hv, 128, generator=gen).bfloat16()
        w = (1.0 + 0.5 * torch.randn(128, generator=gen)).bfloat16()
        ref = inputs.fp64_reference(dy, x, z, w)
        torch.save({"x": x, "projection": projection, "z_start": start, "dy": dy, "w": w,
                    "heads": (hk, hv), "ref": {k: v.clone() for k, v in ref.items()}},
                   out_dir / f"gated_rmsnorm_reference_{name}.pt")
        print(name, {k: tuple(v.shape) for k, v in ref.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(f"usage: python {sys.argv[0]} <reference root>")
    main(sys.argv[1])
