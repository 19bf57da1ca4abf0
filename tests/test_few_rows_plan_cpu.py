"""The few-row kernel's plan, checked without a GPU: every shared-memory read of the consumer loop
stays inside its stage and inside the activation rows, every weight byte of a row is multiplied
exactly once and only from bytes a copy has brought, copies are 16-byte aligned, and the plan fits
the shared memory of an SM. The loop mirrored here is the kernel's (thread (g, q) of warp (wn, wk),
step s: weight piece at (wn * 8 + g) * pitch + wk * slice + q * 16 + s * 64 of the stage, activation
piece at the same K position)."""
import ctypes
import itertools

import pytest

from libwaifu_b200 import flint as F

SHAPES = [(1, 16384, 3072), (16, 1184, 4104), (9, 72, 12288), (5, 4096, 80), (2, 264, 80), (4, 72, 3088), (2, 8, 16),
          (4, 1184, 592), (3, 4096, 12288), (1, 3072, 3072), (16, 264, 3072), (5, 8, 16), (1, 16384, 2048), (2, 264, 72),
          (8, 640, 8208), (1, 64, 528), (3, 64, 1040), (2, 64, 4112), (7, 64, 6160), (1, 18432, 3072), (2, 136, 4112),
          (3, 72, 8208), (1, 151936, 4096), (16, 16384, 3072), (4, 8, 16384), (1, 8, 24), (2, 40, 2056)]


def plan(m, n, k, wbytes, xbytes, residual):
    L = F.lib()
    L.fl_sm100_few_rows_plan.argtypes = [ctypes.c_int32] * 6 + [ctypes.POINTER(ctypes.c_int32)]
    L.fl_sm100_few_rows_plan.restype = ctypes.c_int32
    out = (ctypes.c_int32 * 16)()
    F.check(L.fl_sm100_few_rows_plan(m, n, k, wbytes, xbytes, int(residual), out))
    return list(out)


@pytest.mark.parametrize("wbytes,xbytes", [(1, 1), (1, 2), (2, 2)])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_plan_invariants(m, n, k, wbytes, xbytes):
    if (k * wbytes) % 16:
        pytest.skip("rows are whole 16-byte pieces")
    p = plan(m, n, k, wbytes, xbytes, True)
    ctas, rows, wk, k_chunks, chunk, slc, k_pad, pitch_w, stride, stages, one_copy, pitch_x, x_bytes, ep, grid, smem = p
    if ctas == 0:
        assert not any(p)
        return
    kb = k * wbytes
    assert ctas in (1, 2) and rows * wk == 64 and stages >= 3
    assert chunk % (64 * wk) == 0 and slc * wk == chunk and slc % 64 == 0 and slc <= 512
    assert (k_chunks - 1) * chunk < kb <= k_chunks * chunk == k_pad
    assert smem * ctas + 1024 * ctas <= 233472 and smem <= 232448 - 128
    assert pitch_w % 16 == 0 and stride % 128 == 0 and x_bytes % 128 == 0 and x_bytes >= m * pitch_x
    if one_copy:
        assert k_chunks == 1 and pitch_w == kb
    # activation rows hold every K position a step can touch
    x_elems = k_pad // wbytes
    assert pitch_x >= x_elems * xbytes
    steps = slc // 64
    covered = bytearray(kb)
    for kc in range(k_chunks):
        k0 = kc * chunk
        brought = min(chunk, kb - k0)  # bytes of a channel the stage's copies bring
        assert brought > 0 and brought % 16 == 0 and k0 % 16 == 0
        for w, s, q in itertools.product(range(wk), range(steps), range(4)):
            off = w * slc + q * 16 + s * 64
            assert (rows - 1) * pitch_w + off + 16 <= stride, "a weight read leaves the stage"
            kbyte = k0 + off
            x_off = (kbyte // wbytes) * xbytes
            x_len = 16 // wbytes * xbytes
            assert x_off + x_len <= pitch_x, "an activation read leaves its row"
            if kbyte < kb:
                assert off + 16 <= brought, "a K position inside the row is read from bytes no copy brought"
                for b in range(16):
                    covered[kbyte + b] += 1
            else:
                assert kbyte + 16 <= k_pad  # past k: the activation is zero there
    assert all(c == 1 for c in covered), "a weight byte is multiplied twice or never"
    # the epilogue staging covers the channels of the busiest CTA
    units = -(-n // rows)
    assert grid == min(units, 148 * ctas) or grid <= units
    assert ep >= -(-units // grid) * rows * 8


def test_refused_shapes_report_zero():
    assert not any(plan(17, 64, 64, 1, 1, False))   # more than 16 rows
    assert not any(plan(1, 60, 64, 1, 1, False))    # channels not a multiple of 8
    assert not any(plan(16, 64, 16384, 1, 2, False))  # 16 rows of 32 KB do not fit beside a ring


def route(entry, m, n, k):
    L = F.lib()
    L.fl_sm100_few_rows_route.argtypes = [ctypes.c_int32] * 4
    L.fl_sm100_few_rows_route.restype = ctypes.c_int32
    return L.fl_sm100_few_rows_route(entry, m, n, k)


def test_few_row_routes():
    """Which kernel a few-row product takes, at the shapes the thresholds were measured on: the
    reference's decode shape and its neighbours go to the tensor-core few-row kernels, narrow or
    shallow weights stay with the mma.sync kernel, more rows than a kernel takes go to the tile
    kernel."""
    TILE, MMA_SYNC, TENSOR = 0, 1, 2
    # fl_fp8_matmul, half rows (docs/fp8.md:225-244 is 1 x 16384 x 3072)
    assert route(0, 1, 16384, 3072) == TENSOR and route(0, 16, 16384, 3072) == TENSOR
    assert route(0, 1, 8192, 3072) == TENSOR and route(0, 1, 6144, 3072) == MMA_SYNC and route(0, 2, 6144, 3072) == TENSOR
    assert route(0, 4, 3072, 3072) == MMA_SYNC and route(0, 8, 3072, 3072) == TENSOR
    assert route(0, 1, 8192, 1024) == MMA_SYNC and route(0, 1, 16384, 1024) == TENSOR
    assert route(0, 17, 3072, 2048) == TENSOR and route(0, 64, 16384, 12288) == TENSOR
    assert route(0, 17, 2048, 3072) == TILE and route(0, 65, 16384, 3072) == TILE and route(0, 32, 8192, 1024) == TILE
    # fl_fp8_linear: rows quantised per token
    assert route(1, 1, 16384, 3072) == TENSOR and route(1, 2, 18432, 3072) == TENSOR and route(1, 32, 3072, 3072) == TENSOR
    assert route(1, 1, 3072, 3072) == MMA_SYNC and route(1, 4, 3072, 3072) == TENSOR and route(1, 4, 3072, 1024) == MMA_SYNC
    assert route(1, 33, 16384, 3072) == TILE and route(1, 5, 2048, 3072) == TILE
    # fl_matmul on 16-bit operands
    assert route(2, 1, 16384, 3072) == TENSOR and route(2, 1, 8192, 3072) == MMA_SYNC and route(2, 4, 6144, 3072) == TENSOR
    assert route(2, 8, 3072, 3072) == TENSOR and route(2, 64, 3072, 3072) == TENSOR and route(2, 64, 3072, 12288) == TILE
    assert route(2, 64, 16384, 12288) == TENSOR and route(2, 16, 3072, 1024) == MMA_SYNC and route(2, 17, 3072, 1024) == TILE
    assert route(3, 1, 8, 8) == -1 and route(0, 0, 8, 8) == -1
