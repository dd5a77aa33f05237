"""The work partition of the persistent GEMV kernels (host arithmetic, no GPU).

Units are (64-row block, 1 KB index chunk), block-major.  Whatever the shape, the CTA ranges must
tile [0, total) in order; a range boundary inside a block falls on a multiple of 8 chunks and never
leaves a piece shorter than 8 chunks; the fix-up enumerates at most 128 contributors per block.
"""
import ctypes as C

import numpy as np
import pytest

from prism_engine_b200 import _lib

SHAPES = [  # (rows, k) of decode GEMVs: 0.5B, 7B, 72B, tensor-parallel shards, odd sizes
    (1152, 896), (896, 896), (4864, 896), (896, 4864), (151936, 896),
    (4608, 3584), (3584, 3584), (18944, 3584), (3584, 18944), (152064, 3584),
    (10240, 8192), (8192, 8192), (29568, 8192), (8192, 29568), (152064, 8192),
    (1280, 8192), (8192, 1024), (3696, 8192), (8192, 3712), (64, 32), (72, 40 * 32), (640, 29568), (20000, 512),
]


def partition(n_blocks, n_chunks, slots, stream_chunks=64, min_chunks=8):
    L = _lib.load()
    g = C.c_uint32()
    assert L.prism_cuda_gemv_partition(n_blocks, n_chunks, slots, stream_chunks, min_chunks, C.byref(g), None, 0) == 0
    b = (C.c_uint32 * (g.value + 1))()
    assert L.prism_cuda_gemv_partition(n_blocks, n_chunks, slots, stream_chunks, min_chunks, C.byref(g), b, g.value + 1) == 0
    return np.array(b[:], dtype=np.int64)


@pytest.mark.parametrize("slots", [148, 444, 74, 37, 18])
@pytest.mark.parametrize("rows,k", SHAPES)
@pytest.mark.parametrize("swiglu", [False, True])
def test_ranges_tile_the_matrix(rows, k, slots, swiglu):
    n_chunks = k // 32
    n_hb = (rows + 63) // 64 * 2
    n_blocks = n_hb if swiglu else n_hb // 2
    total = n_blocks * n_chunks
    b = partition(n_blocks, n_chunks, slots)
    assert b[0] == 0 and b[-1] == total and np.all(np.diff(b) >= 0)
    sizes = np.diff(b)
    assert sizes.max() <= max(total // max(len(sizes), 1) + n_chunks, n_chunks) + 8
    # boundaries inside a block: multiples of 8 chunks, no piece under 8 chunks on either side
    inner = b[(b % n_chunks) != 0]
    assert np.all((inner % n_chunks) % 8 == 0)
    assert np.all(n_chunks - (inner % n_chunks) >= 8)
    # contributors per block
    first_blk = b[:-1] // n_chunks
    last_blk = (np.maximum(b[1:], b[:-1] + 1) - 1) // n_chunks
    nonempty = sizes > 0
    contrib = np.zeros(n_blocks + 1, dtype=np.int64)
    for f, l in zip(first_blk[nonempty], last_blk[nonempty]):
        contrib[f:l + 1] += 1
    assert contrib[:n_blocks].min() >= 1 and contrib.max() <= 128


def test_small_matrices_get_one_segment_per_cta():
    # fewer than 64 chunks per CTA slot: every block cut into equal parts, a CTA stays inside one block
    for rows, k in [(896, 896), (3584, 3584), (8192, 1024)]:
        n_chunks, n_blocks = k // 32, (rows + 63) // 64
        b = partition(n_blocks, n_chunks, 148)
        for lo, hi in zip(b[:-1], b[1:]):
            if hi > lo:
                assert lo // n_chunks == (hi - 1) // n_chunks


def test_bad_arguments_are_refused():
    L = _lib.load()
    g = C.c_uint32()
    assert L.prism_cuda_gemv_partition(0, 4, 148, 64, 8, C.byref(g), None, 0) != 0
    assert L.prism_cuda_gemv_partition(4, 4, 148, 64, 8, None, None, 0) != 0
    small = (C.c_uint32 * 2)()
    assert L.prism_cuda_gemv_partition(128, 256, 148, 64, 8, C.byref(g), small, 2) != 0


def test_whole_blocks_when_a_matrix_has_fewer_blocks_than_ctas():
    """The warp-specialised GEMV uses one CTA per block -- and the partition then cuts no block -- when the
    matrix has fewer blocks than CTA slots but enough of them, and rows that are not too long."""
    L = _lib.load()
    ctas = L.prism_cuda_gemv_partition_ctas
    # 72B o and down projections on 148 SMs: 128 blocks
    assert ctas(128, 256, 148, 1024, 50) == 128 and ctas(128, 924, 148, 1024, 50) == 128
    # more blocks than slots, or rows too long, or switched off: every slot
    assert ctas(160, 256, 148, 1024, 50) == 148
    assert ctas(128, 2000, 148, 1024, 50) == 148
    assert ctas(128, 256, 148, 0, 50) == 148
    # the fill threshold: 116 blocks are 78 per 100 slots, 73 are 49
    assert ctas(116, 256, 148, 1024, 50) == 116 and ctas(116, 256, 148, 1024, 85) == 148
    assert ctas(73, 256, 148, 1024, 50) == 148 and ctas(74, 256, 148, 1024, 50) == 74
    for n_blocks, n_chunks in ((128, 256), (128, 924), (116, 256), (80, 256)):
        g = ctas(n_blocks, n_chunks, 148, 1024, 50)
        b = partition(n_blocks, n_chunks, g)
        assert len(b) == n_blocks + 1 and np.all(b % n_chunks == 0) and np.all(np.diff(b) == n_chunks)
