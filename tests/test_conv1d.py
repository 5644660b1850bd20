"""Packed causal depthwise conv1d + SiLU: the oracle against the reference's own FP64 outputs (CPU), the op's
argument surface (CPU), and the kernels against the oracle under the reference's gates -- y and dx within
``1e-3 + 2^-7 |ref|``, the weight gradient within ``5e-2 + 1e-4 |ref|`` (bf16 policy) or ``1e-3 + 2e-6 |ref|`` (fp32
policy; BF16 taps: one BF16 ulp) of the FP64 sum (GPU) (reference: tests/cake/conv1d/test_conv1d_gpu.py:40-260)."""

from __future__ import annotations

from pathlib import Path

import pytest
import torch

from oracle import conv1d_oracle as C

GOLDEN = sorted((Path(__file__).parent / "golden").glob("conv1d_reference_*.pt"))
Y_ATOL, Y_RTOL = 1e-3, 2**-7
DW_ATOL, DW_RTOL = 5e-2, 1e-4
DW_FP32G_ATOL, DW_FP32G_RTOL = 1e-3, 2e-6
PERF_FRACTIONS = (0.37, 0.29, 0.21)


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_the_oracle_reproduces_the_reference_fp64_outputs(path):
    rec = torch.load(path)
    got = C.reference(rec["x"], rec["w"], rec["cu"], rec["dy"], "fp32")
    assert torch.equal(got["y"], rec["y"]) and torch.equal(got["dx"], rec["dx"])
    assert C.outside(got["dw"], rec["dw"], atol=1e-12, rtol=1e-12) == 0
    rounded = C.reference(rec["x"], rec["w"], rec["cu"], rec["dy"], "bf16")  # the other policy stays within the gates
    assert C.outside(rounded["y"], rec["y"], atol=Y_ATOL, rtol=Y_RTOL) == 0
    assert C.outside(rounded["dx"], rec["dx"], atol=2e-2, rtol=2**-6) == 0


def test_the_op_declaration_and_its_checks():
    import miles_ext_kernels_b200 as package
    from miles_ext_kernels_b200 import cake
    from miles_ext_kernels_b200.cake import conv1d

    op = cake.op_spec("conv1d")
    assert op.variants == ("det", "fast") and op.selected_by == (("linear_attention_conv_backend", "cake"),)
    assert set(op.exports) == {"causal_conv1d", "causal_conv1d_kcp", "causal_conv1d_kcp_multi", "check_supported"}
    assert cake.option("conv1d", "cake_conv1d_silu_grad_preactivation") == "bf16"
    package.configure(cake_conv1d_silu_grad_preactivation="fp32")
    assert cake.option("conv1d", "cake_conv1d_silu_grad_preactivation") == "fp32"
    package.configure()
    with pytest.raises(ValueError, match="kernel size 4"):
        conv1d.check_supported(512, 3, "silu")
    with pytest.raises(ValueError, match="SiLU"):
        conv1d.check_supported(512, 4, "gelu")
    with pytest.raises(ValueError, match="without a bias"):
        conv1d.check_supported(512, 4, "silu", has_bias=True)
    with pytest.raises(ValueError, match="multiple of 8"):
        conv1d.check_supported(516, 4, "silu")
    with pytest.raises(NotImplementedError):
        conv1d.causal_conv1d_kcp(None, None, None)


# (S, C, documents): documents of 1-3 tokens and empty ones, run boundaries, channel counts that are not multiples
# of a warp's 256 or of a block's 2048, and the framework's per-rank channel counts
CASES = (
    (5, 136, (2, 0, 3)),
    (63, 384, (1, 2, 3, 57)),
    (1000, 512, "perf"),
    (4097, 1280, (1000, 0, 3, 3094)),
    (4097, 2560, (1000, 0, 3, 3094)),
    (32771, 8192, (1, 2, 3, 0, 9000, 3, 23762)),
)


def doc_lengths(S, docs):
    if docs == "perf":
        lens = []
        for fraction in PERF_FRACTIONS:
            n = int(fraction * S)
            lens.append(n - 1 if n % 64 == 0 else n)
        return (*lens, S - sum(lens))
    assert sum(docs) == S
    return tuple(docs)


def inputs(S, channels, docs, taps):
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed((2033 * 1_000_003 + S * 7919 + channels * 31) % (2**31 - 1))
    x = torch.randn(1, S, channels, device=dev, generator=gen).bfloat16()
    w = (0.5 * torch.randn(channels, 4, device=dev, generator=gen)).to(taps)
    dy = torch.randn(1, S, channels, device=dev, generator=gen).bfloat16()
    lens = doc_lengths(S, docs)
    cu = torch.tensor([0, *torch.tensor(lens).cumsum(0).tolist()], dtype=torch.int32, device=dev)
    return x, w, cu, dy


def run(x, w, cu, dy, policy=None, weight_grad=True):
    from miles_ext_kernels_b200.cake.conv1d import causal_conv1d

    xi, wi = x.detach().requires_grad_(True), w.detach().requires_grad_(weight_grad)
    y = causal_conv1d(xi, wi, cu, silu_grad_preactivation=policy)
    assert y.dtype == torch.bfloat16 and y.shape == x.shape
    y.backward(dy)
    return {"y": y.detach(), "dx": xi.grad, "dw": wi.grad}


@pytest.mark.gpu
@pytest.mark.parametrize("taps", [torch.float32, torch.bfloat16], ids=["fp32_taps", "bf16_taps"])
@pytest.mark.parametrize("policy", ["bf16", "fp32"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: f"s{c[0]}_c{c[1]}")
def test_within_the_reference_gates_of_the_fp64_sums(case, policy, taps):
    S, channels, docs = case
    if S > 5000 and (taps == torch.bfloat16 or policy == "fp32"):
        pytest.skip("the large case runs once")
    x, w, cu, dy = inputs(S, channels, docs, taps)
    got = run(x, w, cu, dy, policy)
    ref = C.reference(x[0].cpu(), w.cpu(), cu.cpu(), dy[0].cpu(), policy)
    assert C.outside(got["y"][0].cpu(), ref["y"], atol=Y_ATOL, rtol=Y_RTOL) == 0
    assert C.outside(got["dx"][0].cpu(), ref["dx"], atol=Y_ATOL if policy == "fp32" else 2e-3, rtol=Y_RTOL) == 0
    atol, rtol = (DW_ATOL, DW_RTOL) if policy == "bf16" else (DW_FP32G_ATOL, DW_FP32G_RTOL)
    if taps == torch.bfloat16:
        atol, rtol = atol * (1 + 2**-8), 2**-7
    assert got["dw"].dtype == taps and C.outside(got["dw"].cpu(), ref["dw"], atol=atol, rtol=rtol) == 0
    again = run(x, w, cu, dy, policy)
    for name in got:
        assert torch.equal(got[name], again[name]), name  # fixed-order sums: the same bits
    assert run(x, w, cu, dy, policy, weight_grad=False)["dw"] is None


@pytest.mark.gpu
def test_one_document_without_boundaries_and_the_2d_form():
    from miles_ext_kernels_b200.cake.conv1d import causal_conv1d

    x, w, cu, dy = inputs(777, 256, (777,), torch.float32)
    with_cu = run(x, w, cu, dy)
    without = run(x, w, None, dy)
    flat = run(x[0], w, None, dy[0])
    for name in ("y", "dx", "dw"):
        assert torch.equal(with_cu[name], without[name]), name
        assert torch.equal(flat[name].view_as(without[name]), without[name]), name
    with pytest.raises(ValueError, match="one packed batch"):
        causal_conv1d(x.expand(2, -1, -1), w)
    with pytest.raises(ValueError, match="multiple of 8"):
        causal_conv1d(x[..., :100], w[:100])
