"""The allocation-free forward entry point (``mek_gdn_forward_static``) against the regular forward stages.

Some hosts of this library may not allocate device memory once they are set up (a server with a fixed memory plan, a
plain C runtime without an allocator): for them the library keeps the forward's intermediates in a fixed device
array of its own.  The test drives the entry point through the C ABI twice in a row (the second call finds the
previous call's contents in the shared array) and expects the bits of the regular path both times.  It runs last so
that a failure here cannot hide another test's result; it also passes on its own in a fresh process.
"""

from __future__ import annotations

import math

import pytest
import torch

from gdn_cases import draw

pytestmark = pytest.mark.gpu


def _forward_both(seq_lens, heads, seed, state):
    from miles_ext_kernels_b200.cake._impl.gdn import meta as M
    from miles_ext_kernels_b200.cake._impl.gdn import native, stages

    dev = torch.device("cuda")
    x = {n: t.to(dev) for n, t in draw(seq_lens, heads, seed=seed, state=state, normalised=True).items()}
    cu = [0]
    for n in seq_lens:
        cu.append(cu[-1] + n)
    meta = M.chunk_meta(torch.tensor(cu, dtype=torch.int32, device=dev), tuple(cu), 1, cu[-1], dev)
    scale = 1.0 / math.sqrt(128)
    o_ref, final_ref, tape, _ = stages.forward(x["q"], x["k"], x["v"], x["g"], x["beta"], meta, scale, x.get("h0"), state,
                                            False)
    o = torch.full_like(o_ref, float("nan"))
    final = torch.full_like(final_ref, float("nan")) if state else None
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    dims = stages.dims_of(meta, heads[0], heads[1], scale)
    native.launch("gdn_forward_static", dims, x["q"], x["k"], x["v"], x["beta"], x["g"], x.get("h0"), o, final, status,
                  device=dev)
    torch.cuda.synchronize()
    stages.check_status(status)
    stages.check_status(tape.status)
    return (o, final), (o_ref, final_ref)


def test_two_calls_in_a_row_give_the_regular_forward_bits():
    for seq_lens, heads, seed, state in (((63, 130, 257), (2, 4), 21, True), ((200, 64), (1, 2), 22, False)):
        (o, final), (o_ref, final_ref) = _forward_both(seq_lens, heads, seed, state)
        assert torch.equal(o, o_ref)
        if state:
            assert torch.equal(final, final_ref)


def test_calls_at_the_limits_of_the_fixed_scratch():
    """One sequence of 2,048 tokens on four value heads fills the 8,192 token-heads; 68 ragged documents on two
    value heads fill the 256 chunk-heads (sixty of 65 tokens, two chunks each, and eight of one token)."""
    for seq_lens, heads, seed, state in (((2048,), (2, 4), 23, True), ((65,) * 60 + (1,) * 8, (1, 2), 24, False)):
        chunks = sum(-(-n // 64) for n in seq_lens)
        assert sum(seq_lens) * heads[1] <= 8192 and chunks * heads[1] <= 256
        assert sum(seq_lens) * heads[1] == 8192 or chunks * heads[1] == 256
        (o, final), (o_ref, final_ref) = _forward_both(seq_lens, heads, seed, state)
        assert torch.equal(o, o_ref)
        if state:
            assert torch.equal(final, final_ref)


def test_null_operands_are_rejected():
    from miles_ext_kernels_b200.cake._impl.gdn import meta as M
    from miles_ext_kernels_b200.cake._impl.gdn import native, stages

    dev = torch.device("cuda")
    meta = M.chunk_meta(None, None, 1, 64, dev)
    dims = stages.dims_of(meta, 1, 1, 1.0)
    z = torch.zeros(64 * 128, dtype=torch.bfloat16, device=dev)
    f = torch.zeros(64, device=dev)
    st = torch.zeros(1, dtype=torch.int32, device=dev)
    with pytest.raises(ValueError, match="must not be null"):
        native.launch("gdn_forward_static", dims, z, z, z, f, f, None, None, None, st, device=dev)
    with pytest.raises(ValueError, match="must not be null"):
        native.launch("gdn_forward_static", dims, z, z, z, f, f, None, z, None, None, device=dev)


def test_a_call_beyond_the_fixed_scratch_is_rejected():
    from miles_ext_kernels_b200.cake._impl.gdn import meta as M
    from miles_ext_kernels_b200.cake._impl.gdn import native, stages

    dev = torch.device("cuda")
    T, H, HV = 4096, 4, 4  # 16384 token-heads: twice the limit
    meta = M.chunk_meta(None, None, 1, T, dev)
    dims = stages.dims_of(meta, H, HV, 1.0)
    z = torch.zeros(1, device=dev)
    with pytest.raises(ValueError, match="does not fit the fixed scratch"):
        native.launch("gdn_forward_static", dims, z, z, z, z, z, None, z, None, z, device=dev)
