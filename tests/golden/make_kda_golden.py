"""Generate ``kda_reference_*.pt``: inputs and outputs of the REFERENCE's own exact FP64 KDA oracle.

Run once in a container that has the reference checked out::

    PYTHONPATH=<reference root>/tests python tests/golden/make_kda_golden.py

Inputs come from the reference's seeded generator ``make_raw_inputs`` (reference: tests/cake/kda/_reference.py:45-83),
outputs from ``kda_exact_with_grads`` (activated gate, :136-142) and ``kda_exact_raw_with_grads`` (raw gate with
``A_log`` / ``dt_bias``, :145-157).
"""

from __future__ import annotations

from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
CASES = {"two_docs": ((100, 60), 2, 31), "one_doc": ((137,), 1, 32)}


def main() -> None:
    from cake.kda import _reference as R

    for name, (lengths, H, seed) in CASES.items():
        x = R.make_raw_inputs(lengths, H, "cpu", seed=seed)
        scale = 128**-0.5
        g = R.raw_gate(x["g"], x["A_log"], x["dt_bias"]).float()
        o, grads = R.kda_exact_with_grads(x["q"], x["k"], x["v"], g, x["beta"], x["dout"], x["cu_seqlens"], scale)
        o_raw, grads_raw = R.kda_exact_raw_with_grads(x["q"], x["k"], x["v"], x["g"], x["beta"], x["A_log"],
                                                      x["dt_bias"], x["dout"], x["cu_seqlens"], scale)
        record = {"lengths": lengths, "H": H, "seed": seed, "scale": scale, "inputs": x, "g_activated": g,
                  "activated": {"o": o.float(), **{n: t.float() for n, t in grads.items()}},
                  "raw": {"o": o_raw.float(), **{n: t.float() for n, t in grads_raw.items()}}}
        torch.save(record, HERE / f"kda_reference_{name}.pt")
        print(name, {n: tuple(t.shape) for n, t in record["raw"].items()})


if __name__ == "__main__":
    main()
