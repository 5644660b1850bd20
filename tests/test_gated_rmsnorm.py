"""SiLU-gated RMSNorm: the oracle against the reference's own FP64 outputs (CPU), the op's argument surface (CPU),
and the kernels against the oracle under the reference's gates -- y, dx, dz within one BF16 ulp of FP64, the weight
gradient within ``|dw| 2^-7 + sum|terms| 2^-20`` -- with the gate read in place or copied (GPU)
(reference: tests/cake/gated_rmsnorm/test_gated_rmsnorm_gpu.py:30-135, test_arguments.py)."""

from __future__ import annotations

from pathlib import Path

import pytest
import torch

from oracle import gated_rmsnorm_oracle as R

GOLDEN = sorted((Path(__file__).parent / "golden").glob("gated_rmsnorm_reference_*.pt"))
DETECT = 1.02  # every gate must reject an output 2 % off


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_the_oracle_reproduces_the_reference_fp64_outputs(path):
    rec = torch.load(path)
    hv = rec["heads"][1]
    z = rec["projection"][:, rec["z_start"] : rec["z_start"] + hv * 128].unflatten(-1, (hv, 128))
    got = R.fp64_reference(rec["dy"], rec["x"], z, rec["w"])
    for name, want in rec["ref"].items():
        assert torch.equal(got[name], want), name


def test_the_op_declaration_and_its_checks():
    import miles_ext_kernels_b200 as package
    from miles_ext_kernels_b200 import cake
    from miles_ext_kernels_b200.cake import gated_rmsnorm

    assert "gated_rmsnorm" in cake.OPS
    op = cake.op_spec("gated_rmsnorm")
    assert op.variants == ("det", "fast") and set(op.exports) == {"check_supported", "rmsnorm_silu_gate"}
    assert op.selected_by == (("linear_attention_output_norm_backend", "cake"),)
    package.configure(cake_gated_rmsnorm_variant="fast")
    assert cake.variant("gated_rmsnorm") == "fast"
    package.configure()
    with pytest.raises(ValueError, match="SiLU"):
        gated_rmsnorm.check_supported(128, "swish", torch.bfloat16)
    with pytest.raises(ValueError, match="rows of 128"):
        gated_rmsnorm.check_supported(64, "silu", torch.bfloat16)
    with pytest.raises(ValueError, match="no bias"):
        gated_rmsnorm.check_supported(128, "silu", torch.bfloat16, has_bias=True)
    with pytest.raises(ValueError, match="BF16 weight"):
        gated_rmsnorm.check_supported(128, "silu", torch.float32)


# (key heads, value heads, extra projection columns): the projection width 2 Hk 128 + 2 Hv 128 + 2 Hv (+ extra) is
# the gate's token stride -- a multiple of 8 elements (read in place) or not (copied once)
LAYOUTS = ((6, 12, 0), (6, 12, 6), (8, 16, 0), (16, 32, 8), (16, 32, 3))
TOKENS = (1, 7, 1031, 32771)


def make(tokens, hk, hv, extra, seed=0):
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(((seed * 1_000_003 + tokens) * 131 + hv) * 17 + extra)
    randn = lambda *shape: torch.randn(*shape, device=dev, generator=gen).bfloat16()  # noqa: E731
    width = -(-(2 * hk * 128 + 2 * hv * 128 + 2 * hv) // 8) * 8 + extra
    x = randn(tokens, hv, 128)
    projection = randn(tokens, width)
    start = (2 * hk + hv) * 128
    z = projection[:, start : start + hv * 128].unflatten(-1, (hv, 128))
    dy = randn(tokens, hv, 128)
    w = (1.0 + 0.5 * torch.randn(128, device=dev, generator=gen)).bfloat16()
    return x, z, w, dy


def run(x, z, w, dy, weight_grad=True):
    from miles_ext_kernels_b200.cake.gated_rmsnorm import rmsnorm_silu_gate

    xi, zi = (t.detach().requires_grad_() for t in (x, z))
    wi = w.detach().requires_grad_(weight_grad)
    y = rmsnorm_silu_gate(xi, zi, wi, 1e-6)
    assert y.dtype == torch.bfloat16 and y.shape == x.shape
    y.backward(dy)
    assert xi.grad.dtype == zi.grad.dtype == torch.bfloat16
    if weight_grad:
        assert wi.grad.dtype == torch.bfloat16 and wi.grad.shape == (128,)
    return {"y": y.detach(), "dx": xi.grad, "dz": zi.grad, "dw": wi.grad}


def assert_accurate(got, ref, what):
    for name in ("y", "dx", "dz"):
        assert R.bf16_misses(got[name].cpu(), ref[name]) == 0, f"{what} {name}: beyond one BF16 ulp of FP64"
        assert R.bf16_misses(got[name].cpu().double() * DETECT, ref[name]) > 0, f"{what} {name}: gate too loose"
    assert R.dw_misses(got["dw"].cpu(), ref["dw"], ref["mag"]) == 0, f"{what} dw: beyond the bound"
    assert R.dw_misses(got["dw"].cpu().double() * DETECT, ref["dw"], ref["mag"]) > 0, f"{what} dw: gate too loose"


@pytest.mark.gpu
@pytest.mark.parametrize("layout", LAYOUTS, ids=lambda l: "hk{}_hv{}_x{}".format(*l))
@pytest.mark.parametrize("tokens", TOKENS)
def test_within_one_bf16_ulp_of_fp64_with_the_gate_in_place_or_copied(tokens, layout):
    from miles_ext_kernels_b200.cake._impl.gated_rmsnorm import ops

    x, z, w, dy = make(tokens, *layout)
    view = ops._rows_view(z, "z")[0]
    assert (view.data_ptr() == z.data_ptr()) == (z.stride(0) % 8 == 0)
    got = run(x, z, w, dy)
    ref = R.fp64_reference(dy.cpu(), x.cpu(), z.cpu(), w.cpu())
    assert_accurate(got, ref, f"{tokens} tokens, {layout}")
    again = run(x, z, w, dy)
    for name in got:
        assert torch.equal(got[name], again[name]), name  # fixed-order sums: the same bits
    flat = run(x.reshape(-1, 128), z.reshape(-1, 128), w, dy.reshape(-1, 128))  # [T * H, 128] rows
    for name in ("y", "dx", "dz"):
        assert torch.equal(flat[name].view(x.shape), got[name]), name
    assert run(x, z, w, dy, weight_grad=False)["dw"] is None


@pytest.mark.gpu
def test_gradients_of_a_head_split_sum_to_the_whole():
    x, z, w, dy = make(1031, 8, 16, 0)
    whole = run(x, z, w, dy)
    halves = [run(x[:, s], z[:, s], w, dy[:, s]) for s in (slice(0, 8), slice(8, 16))]
    ref = R.fp64_reference(dy.cpu(), x.cpu(), z.cpu(), w.cpu())
    summed = halves[0]["dw"].cpu().double() + halves[1]["dw"].cpu().double()
    bound = halves[0]["dw"].cpu().double().abs() + halves[1]["dw"].cpu().double().abs()
    assert R.dw_misses(summed, ref["dw"], ref["mag"], rtol_of=bound) == 0
    for name in ("y", "dx", "dz"):
        assert torch.equal(torch.cat([h[name] for h in halves], dim=1), whole[name]), name
