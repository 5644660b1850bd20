"""The tensor-core building block against a CPU matmul: every operand role the kernels use (K-major and MN-major
tiles in the 128-byte swizzled block layout, M = 64 and M = 128, negated A), through the C ABI."""

from __future__ import annotations

import ctypes

import numpy as np
import pytest

from umma_images import (
    bf16_round,
    desc_template,
    idesc,
    kmajor_offsets,
    lane_of_row,
    mnmajor_offsets,
    tile_image,
)

torch = pytest.importorskip("torch")

CASES = {
    # name: (M, N, K, a_mn, b_mn, neg_a)
    "k_k_m128_n64_k64": (128, 64, 64, False, False, False),
    "k_k_m128_n128_k128": (128, 128, 128, False, False, False),
    "k_k_m64_n64_k128": (64, 64, 128, False, False, False),
    "k_mn_m64_n128_k64": (64, 128, 64, False, True, False),
    "k_mn_m64_n128_k128": (64, 128, 128, False, True, False),
    "mn_mn_m128_n128_k64": (128, 128, 64, True, True, False),
    "mn_mn_m128_n64_k64_neg": (128, 64, 64, True, True, True),
    "mn_k_m64_n128_k64": (64, 128, 64, True, False, False),
    "k_k_m64_n256_k64": (64, 256, 64, False, False, False),
}


def run_case(lib, m, n, k, a_mn, b_mn, neg_a, seed=0, d_lane=0):
    rng = np.random.default_rng(seed)
    a = bf16_round(rng.standard_normal((m, k)).astype(np.float32))
    b = bf16_round(rng.standard_normal((n, k)).astype(np.float32))
    # K-major: the tile is [rows = M or N, cols = K].  MN-major: the tile is [rows = K, cols = M or N].
    a_img, a_stride = tile_image(a.T.copy() if a_mn else a)
    b_img, b_stride = tile_image(b.T.copy() if b_mn else b)
    a_off = mnmajor_offsets(k) if a_mn else kmajor_offsets(k, a_stride)
    b_off = mnmajor_offsets(k) if b_mn else kmajor_offsets(k, b_stride)
    a_desc = desc_template(a_stride if a_mn else 16)
    b_desc = desc_template(b_stride if b_mn else 16)
    dev = torch.device("cuda")
    t = lambda x, dt: torch.from_numpy(np.ascontiguousarray(x)).to(dev, dt)  # noqa: E731
    a_d, b_d = t(a_img, torch.uint8), t(b_img, torch.uint8)
    ao, bo = t(np.array(a_off, np.int32), torch.int32), t(np.array(b_off, np.int32), torch.int32)
    out = torch.zeros(128, n, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    p = lambda x: ctypes.c_void_p(x.data_ptr())  # noqa: E731
    rc = lib.mek_selftest_umma(
        p(a_d), a_img.size, p(b_d), b_img.size, ctypes.c_uint64(a_desc), ctypes.c_uint64(b_desc), p(ao), p(bo),
        len(a_off), ctypes.c_uint32(idesc(m, n, a_mn, b_mn, neg_a)), n, d_lane, 0, p(out), p(status),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
    )
    lib.check(rc)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "the MMA wait ran out"
    want = (a.astype(np.float64) @ b.astype(np.float64).T) * (-1.0 if neg_a else 1.0)
    lanes = [lane_of_row(m, r) + d_lane for r in range(m)]
    got = out.cpu().numpy()[lanes]
    return got, want


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CASES))
def test_umma_operand_layouts(name):
    from miles_ext_kernels_b200.cake._runtime import loader

    lib = loader.load_library()
    got, want = run_case(lib, *CASES[name])
    err = np.abs(got - want).max()
    assert err <= 1e-3 * max(1.0, np.abs(want).max()), f"{name}: max error {err}"


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["k_k_m64_n64_k128", "k_mn_m64_n128_k64", "mn_k_m64_n128_k64"])
def test_m64_accumulator_in_the_upper_half_lanes(name):
    """An M = 64 accumulator placed at lane 16 of each quadrant: rows 16 q + r land in lanes 32 q + 16 + r."""
    from miles_ext_kernels_b200.cake._runtime import loader

    lib = loader.load_library()
    got, want = run_case(lib, *CASES[name], d_lane=16)
    err = np.abs(got - want).max()
    assert err <= 1e-3 * max(1.0, np.abs(want).max()), f"{name}: max error {err}"


@pytest.mark.gpu
def test_a_wait_that_nothing_satisfies_runs_out_and_reports_it():
    """Failure detection without a fault: no MMA is issued, so no arrival ever reaches the barrier; the kernel's wait
    gives up after its one-second limit, writes the status word and exits cleanly; the context stays usable."""
    import time

    from miles_ext_kernels_b200.cake._runtime import loader

    lib = loader.load_library()
    dev = torch.device("cuda")
    img = torch.zeros(1024, dtype=torch.uint8, device=dev)
    off = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.zeros(128, 16, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    p = lambda x: ctypes.c_void_p(x.data_ptr())  # noqa: E731
    torch.cuda.synchronize()
    begin = time.perf_counter()
    rc = lib.mek_selftest_umma(p(img), 1024, p(img), 1024, ctypes.c_uint64(desc_template(16)),
                               ctypes.c_uint64(desc_template(16)), p(off), p(off), 0,
                               ctypes.c_uint32(idesc(64, 16, False, False)), 16, 0, 0, p(out), p(status),
                               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    lib.check(rc)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - begin
    assert int(status.item()) == 1 and 0.5 < elapsed < 10.0
    got, want = run_case(lib, *CASES["k_k_m128_n64_k64"])  # the context still works
    assert np.abs(got - want).max() <= 1e-3 * np.abs(want).max()


@pytest.mark.gpu
@pytest.mark.parametrize("box_rows,x,y", [(64, 0, 0), (64, 64, 37), (128, 128, 256), (64, 192, 480), (64, 0, 500)])
def test_tma_box_lands_in_the_operand_layout(box_rows, x, y):
    """A TMA box is, byte for byte, the swizzled 64-column block the tensor-core operands use; rows past the
    matrix's end arrive as zeros."""
    from miles_ext_kernels_b200.cake._runtime import loader

    lib = loader.load_library()
    rows, cols = 512, 256
    rng = np.random.default_rng(box_rows + x + y)
    src = bf16_round(rng.standard_normal((rows, cols)).astype(np.float32))
    dev = torch.device("cuda")
    src_dev = torch.from_numpy(src).to(dev).to(torch.bfloat16).contiguous()
    out = torch.zeros(box_rows * 128, dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    lib.check(lib.mek_selftest_tma(p(src_dev), ctypes.c_int64(rows), ctypes.c_int64(cols), box_rows, x, y, p(out),
                                   p(status), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    box = np.zeros((box_rows, 64), dtype=np.float32)
    live = max(0, min(box_rows, rows - y))
    box[:live] = src[y:y + live, x:x + 64]
    want, _ = tile_image(box)
    assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k,neg_a,d_lane", [(64, 32, 32, False, 0), (64, 32, 32, True, 16), (64, 64, 64, False, 0),
                                                (128, 64, 32, False, 0)])
def test_tf32_operands_in_the_swizzled_layout(m, n, k, neg_a, d_lane):
    """kind::tf32 with K-major fp32 operands (blocks of 32 columns = 128 bytes, the same 16-byte-chunk swizzle, K = 8
    per instruction): what the WY kernel's blocked triangular inverse relies on."""
    from miles_ext_kernels_b200.cake._runtime import loader
    from umma_images import idesc_tf32, kmajor_offsets_f32, tile_image_f32

    lib = loader.load_library()
    rng = np.random.default_rng(m + n + k)
    a = bf16_round(rng.standard_normal((m, k)).astype(np.float32))  # exact in tf32
    b = bf16_round(rng.standard_normal((n, k)).astype(np.float32))
    a_img, a_stride = tile_image_f32(a)
    b_img, b_stride = tile_image_f32(b)
    a_off, b_off = kmajor_offsets_f32(k, a_stride), kmajor_offsets_f32(k, b_stride)
    dev = torch.device("cuda")
    a_d, b_d = torch.from_numpy(a_img.copy()).to(dev), torch.from_numpy(b_img.copy()).to(dev)
    ao = torch.tensor(a_off, dtype=torch.int32, device=dev)
    bo = torch.tensor(b_off, dtype=torch.int32, device=dev)
    ncols = max(16, n)
    out = torch.zeros(128, ncols, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    p = lambda x: ctypes.c_void_p(x.data_ptr())  # noqa: E731
    rc = lib.mek_selftest_umma(p(a_d), a_img.size, p(b_d), b_img.size, ctypes.c_uint64(desc_template(16)),
                               ctypes.c_uint64(desc_template(16)), p(ao), p(bo), len(a_off),
                               ctypes.c_uint32(idesc_tf32(m, n, neg_a)), ncols, d_lane, 1, p(out), p(status),
                               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    lib.check(rc)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = (a.astype(np.float64) @ b.astype(np.float64).T) * (-1.0 if neg_a else 1.0)
    lanes = np.array([lane_of_row(m, r) + d_lane for r in range(m)])
    got = out.cpu().numpy()[lanes][:, :n]
    assert np.abs(got - want).max() <= 1e-4 * np.abs(want).max()


@pytest.mark.gpu
def test_two_accumulators_keep_the_tensor_core_busier_than_one():
    """The measurement behind the kernels' issue order: instructions into one accumulator wait for one another, so a
    thread that alternates between two accumulators, or two issuing threads, finish the same instructions sooner; and
    one M = 128, N = 128 instruction does the work of four M = 64, N = 64 ones in less than their time."""
    from miles_ext_kernels_b200.cake._runtime import loader

    lib = loader.load_library()
    dev = torch.device("cuda")
    cycles = torch.zeros(1, dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def per_instruction(m, n, issuers, interleave, count=64):
        for c in (8, count):  # a short run first: instruction cache, clocks
            lib.check(lib.mek_selftest_umma_rate(m, n, 0, 1, 128, c, issuers, interleave,
                                                 ctypes.c_void_p(cycles.data_ptr()),
                                                 ctypes.c_void_p(status.data_ptr()),
                                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
            torch.cuda.synchronize()
            assert int(status.item()) == 0
        chains = 2 if (issuers == 2 or interleave) else 1
        return int(cycles.item()) / (count * 8 * chains)

    one = per_instruction(64, 64, 1, 0)
    alternating = per_instruction(64, 64, 1, 1)
    two_threads = per_instruction(64, 64, 2, 0)
    big = per_instruction(128, 128, 2, 0)
    assert alternating < 0.8 * one and two_threads < 0.8 * one, (one, alternating, two_threads)
    assert big < 0.6 * 4 * two_threads, (big, two_threads)  # four small ones' work in under 60 % of their time
    with pytest.raises(NotImplementedError):
        lib.check(lib.mek_selftest_umma_rate(96, 64, 0, 0, 128, 8, 1, 0, None, None, None))
