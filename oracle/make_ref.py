"""Recipe for ``oracle/_ref/``: the reference's own CPU implementation of the GDN path, as it lies in a checkout.

    python oracle/make_ref.py [<reference root>]        (default: the MILES_EXT_KERNELS_REFERENCE variable, else DEFAULT_ROOT)

The reference is Python: its torch emulation of the nine GDN programs (``cake_fake_backend.py`` of the deterministic
context-parallel package) runs on the host through the public entry point ``chunk_gated_delta_rule(...,
cp_context=<one-rank CPU KcpContext>)`` with ``KCP_OPTIONS = {"backend": "fake"}`` (reference:
tests/cake/gdn/test_gdn_kcp_wiring.py:410-444).  "Building" it means importing that path once from the checkout,
listing the files the call actually loaded (modules and the data files they read), and copying exactly those, unchanged and with their directory
structure, into ``oracle/_ref/`` -- which is ignored by git (no reference source enters this repository's history)
but travels with the working tree to a machine that has no checkout.  ``oracle/reference_arm.py`` imports it from
there.  Test infrastructure: only tests, the smoke check and the CPU legs of ``bench.py`` use it.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

DEFAULT_ROOT = "/root/reference"  # where the build machine mounts the checkout
HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"

_TRACE = r"""
import sys, torch
root = sys.argv[1]
opened = set()
def audit(event, args):  # data files (registries, manifests) the modules read at import or call time
    if event == "open" and isinstance(args[0], str) and args[0].startswith(root) and "w" not in (args[1] or "r"):
        opened.add(args[0])
sys.addaudithook(audit)
from miles_ext_kernels import cake
from miles_ext_kernels.cake._impl.gdn import ops
from miles_ext_kernels.cake._impl.gdn.kcp import KcpContext
from miles_ext_kernels.cake import kda  # noqa: F401  (the op spec only; its implementation needs a GPU)
ops.KCP_OPTIONS = {"backend": "fake"}
cake.configure(cake_gdn_variant="det")
T, H, HV = 128, 1, 2
gen = torch.Generator().manual_seed(0)
leaf = lambda *s: torch.randn(*s, generator=gen).bfloat16().requires_grad_(True)
q, k, v = leaf(1, T, H, 128), leaf(1, T, H, 128), leaf(1, T, HV, 128)
g = (-0.5 * torch.rand(1, T, HV, generator=gen)).requires_grad_(True)
beta = torch.rand(1, T, HV, generator=gen).bfloat16().requires_grad_(True)
ctx = KcpContext((0, 70, T), None, 0, 1, torch.device("cpu"), 4, "contiguous", None)
out, _ = ops.chunk_gated_delta_rule(q, k, v, g, beta, use_qk_l2norm_in_kernel=True, cp_context=ctx)
out.backward(torch.ones_like(out))
for m in list(sys.modules.values()):
    f = getattr(m, "__file__", None)
    if f and f.startswith(root):
        opened.add(f)
print("\n".join(sorted(f for f in opened if "__pycache__" not in f)))
"""


def main(argv: list[str]) -> int:
    root = Path(argv[1] if len(argv) > 1 else os.environ.get("MILES_EXT_KERNELS_REFERENCE", DEFAULT_ROOT)).resolve()
    if not (root / "miles_ext_kernels" / "cake").is_dir():
        print(f"make_ref: no reference checkout at {root}; oracle/_ref is left as it is", file=sys.stderr)
        return 1
    env = dict(os.environ, PYTHONPATH=str(root), PYTHONDONTWRITEBYTECODE="1", CUDA_VISIBLE_DEVICES="")
    listing = subprocess.run([sys.executable, "-c", _TRACE, str(root) + os.sep], env=env, cwd="/tmp", text=True,
                             capture_output=True)
    if listing.returncode != 0:
        print(listing.stderr[-2000:], file=sys.stderr)
        return listing.returncode
    files = sorted({Path(line) for line in listing.stdout.splitlines() if line.startswith(str(root))})
    if TARGET.exists():
        shutil.rmtree(TARGET)
    for src in files:
        dst = TARGET / src.relative_to(root)
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(src, dst)
    licence = root / "LICENSE"
    if licence.is_file():
        shutil.copyfile(licence, TARGET / "LICENSE")
    (TARGET / "SOURCE.txt").write_text(
        "Unmodified files of radixark/miles-ext-kernels, copied by oracle/make_ref.py from a local checkout: the\n"
        "modules its CPU (torch emulation) path of chunk_gated_delta_rule loads.  Not part of this repository's "
        "history.\n")
    total = sum(f.stat().st_size for f in files)
    print(f"oracle/_ref: {len(files)} files, {total / 1e6:.1f} MB")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
