"""The shared-memory operand images the kernels use agree with the layout Frisk's inference
selects for 16-bit MMA operands: the 128-byte-swizzle canonical image whose byte address is
a ^ (((a >> 7) & 7) << 4) on 1024-byte aligned tiles
(lib/Dialect/Frisk/Target/SM90/SM90MmaLayoutProof.cpp:198-212,
benchmark/layout/execution/attention_tile_mma.py:117-136).  The kernel side is restated from
frisk_b200/csrc/ptx.cuh: what TMA writes with 128B swizzle and what the UMMA descriptors
(SBO = 1024, k-slice advance of 32 bytes, MN-major block strides) read."""
import numpy as np


def reference_swizzled_offset(a):
    """The reference's canonical address map for swizzle 128."""
    return a ^ (((a >> 7) & 7) << 4)


def tma_sw128_offset(row, byte_in_row):
    """Byte offset TMA gives element (row, byte) of a [rows][128 B] box: the 16-byte chunk index
    is XORed with the row index modulo 8."""
    chunk = (byte_in_row >> 4) ^ (row & 7)
    return row * 128 + (chunk << 4) + (byte_in_row & 15)


def umma_kmajor_offset(row, k_elem, elem_bytes=2):
    """Where the K-major SW128 descriptor of ptx.cuh finds element (row, k): 8-row groups are
    SBO = 1024 bytes apart, rows 128 bytes apart, the k16 slice is selected by advancing the
    start address by 32 bytes, and the hardware applies the same XOR on address bits 4-6."""
    linear = (row // 8) * 1024 + (row % 8) * 128 + k_elem * elem_bytes
    return reference_swizzled_offset(linear)


def test_tma_image_equals_reference_formula():
    for rows in (64, 128, 256):
        r = np.repeat(np.arange(rows), 128)
        b = np.tile(np.arange(128), rows)
        dense = r * 128 + b
        assert np.array_equal(tma_sw128_offset(r, b), reference_swizzled_offset(dense))


def test_descriptor_walk_equals_tma_image():
    # every (row, k) of a 128 x 64 tile of 16-bit elements, for all four k16 slices
    for row in range(128):
        for k in range(64):
            assert umma_kmajor_offset(row, k) == tma_sw128_offset(row, 2 * k)


def test_mn_major_blocks():
    # MN-major tile [k rows][64 mn elements]: one k row is one 128-byte line, 8-row atoms are
    # 1024 bytes (SBO) apart, the next 64 mn elements start a new box (LBO = rows*128 bytes),
    # a k16 slice advances 2048 bytes.  Same XOR inside every 1024-byte atom.
    rows = 64
    for k in range(rows):
        for mn in range(128):
            box, within = divmod(mn, 64)
            tma = box * rows * 128 + tma_sw128_offset(k, 2 * within)
            linear = box * rows * 128 + (k // 16) * 2048 + ((k % 16) // 8) * 1024 + (k % 8) * 128 + 2 * within
            assert reference_swizzled_offset(linear) == tma


def test_reference_d64_tile_offsets():
    # the reference's own 64x64 fp16 tile: row-major halves -> swizzled 16-bit offsets
    # (attention_tile_mma.py: shared_offsets_64x64 uses the same XOR on the byte address)
    r, c = np.divmod(np.arange(64 * 64), 64)
    a = (r * 64 + c) * 2
    sw = reference_swizzled_offset(a)
    assert len(set(sw.tolist())) == 64 * 64 and sw.max() < 8192
    assert np.array_equal(sw, tma_sw128_offset(r, 2 * c))
