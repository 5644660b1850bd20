"""Host-side model of the shared-memory operand layout the kernels use (128-byte swizzled 64-column blocks) and of
the tcgen05 descriptors that read it, for the tensor-core self-test."""

from __future__ import annotations

import numpy as np

BLOCK_COLS = 64
SBO = 1024


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (round to nearest even), as uint16."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16)


def bf16_round(x: np.ndarray) -> np.ndarray:
    return (bf16_bits(x).astype(np.uint32) << 16).view(np.float32)


def tile_image(tile: np.ndarray, block_stride: int | None = None) -> tuple[np.ndarray, int]:
    """The bytes of a [rows, cols] tile (cols a multiple of 64) as the kernels lay it out: one block per 64 columns,
    row r's 16-byte chunk c at ``r * 128 + ((c ^ (r & 7)) << 4)``.  Returns ``(uint8 image, block_stride)``."""
    rows, cols = tile.shape
    assert cols % BLOCK_COLS == 0 and rows % 8 == 0
    blocks = cols // BLOCK_COLS
    stride = rows * 128 if block_stride is None else block_stride
    assert stride % 1024 == 0 and stride >= rows * 128
    bits = bf16_bits(tile).reshape(rows, cols)
    image = np.zeros(blocks * stride // 2, dtype=np.uint16)
    for b in range(blocks):
        for r in range(rows):
            for c in range(8):
                dst = (b * stride + r * 128 + ((c ^ (r & 7)) << 4)) // 2
                image[dst : dst + 8] = bits[r, b * 64 + c * 8 : b * 64 + c * 8 + 8]
    return image.view(np.uint8), stride


def desc_template(lbo: int, sbo: int = SBO) -> int:
    """Shared-memory descriptor without a start address: SWIZZLE_128B, sm_100 version bit."""
    return (((lbo >> 4) & 0x3FFF) << 16) | (((sbo >> 4) & 0x3FFF) << 32) | (1 << 46) | (2 << 61)


def idesc(m: int, n: int, a_mn: bool, b_mn: bool, neg_a: bool = False) -> int:
    return (
        (1 << 4) | (1 << 7) | (1 << 10) | (int(neg_a) << 13) | (int(a_mn) << 15) | (int(b_mn) << 16)
        | ((n >> 3) << 17) | ((m >> 4) << 24)
    )


def kmajor_offsets(kdim: int, block_stride: int) -> list[int]:
    """Start-address offsets of each K = 16 instruction when the contraction runs along the tile's columns."""
    return [(k0 // 64) * block_stride + (k0 % 64) * 2 for k0 in range(0, kdim, 16)]


def mnmajor_offsets(kdim: int) -> list[int]:
    """... when the contraction runs along the tile's rows."""
    return [k0 * 128 for k0 in range(0, kdim, 16)]


def lane_of_row(m_rows: int, row: int) -> int:
    """Tensor-memory lane that holds accumulator row ``row`` for an M = 128 or M = 64 instruction."""
    return row if m_rows == 128 else (row % 16) + 32 * (row // 16)


def tile_image_f32(tile: np.ndarray) -> tuple[np.ndarray, int]:
    """The bytes of a [rows, cols] fp32 tile (cols a multiple of 32) in the same swizzled layout: one block per 32
    columns (128 bytes per row), row r's 16-byte chunk c (4 floats) at ``r * 128 + ((c ^ (r & 7)) << 4)``."""
    rows, cols = tile.shape
    assert cols % 32 == 0 and rows % 8 == 0
    blocks, stride = cols // 32, rows * 128
    words = np.ascontiguousarray(tile, dtype=np.float32).view(np.uint32)
    image = np.zeros(blocks * stride // 4, dtype=np.uint32)
    for b in range(blocks):
        for r in range(rows):
            for c in range(8):
                dst = (b * stride + r * 128 + ((c ^ (r & 7)) << 4)) // 4
                image[dst : dst + 4] = words[r, b * 32 + c * 4 : b * 32 + c * 4 + 4]
    return image.view(np.uint8), stride


def idesc_tf32(m: int, n: int, neg_a: bool = False) -> int:
    return (1 << 4) | (2 << 7) | (2 << 10) | (int(neg_a) << 13) | ((n >> 3) << 17) | ((m >> 4) << 24)


def kmajor_offsets_f32(kdim: int, block_stride: int) -> list[int]:
    """Start-address offsets of each K = 8 tf32 instruction when the contraction runs along the tile's columns."""
    return [(k0 // 32) * block_stride + (k0 % 32) * 4 for k0 in range(0, kdim, 8)]
