"""Runs every TMA kernel variant on the CPU (tests/emu/kdw_emu.cu executes the kernels' own scheduler,
thread mapping and step functions) and checks the result against the oracle."""
import numpy as np
import pytest

from oracle import dwconv_oracle as o

FPROP_CS = None
WGRAD_CS = None


def _variants(lib, kind):
    n = getattr(lib, f'kdw_{kind}_variants')()
    return [(v, getattr(lib, f'kdw_{kind}_variant_channels')(v)) for v in range(1, n + 1)]


def _inputs(seed, N, C, H, W, D):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((N, H, W, D, C)).astype(np.float16)
    g = rng.standard_normal((N, H, W, D, C)).astype(np.float16)
    w = ((rng.random((3, 3, 3, C)) * 2 - 1) / np.sqrt(27)).astype(np.float16)
    return x, g, w


SHAPES = [
    # N, C, H, W, D, grid
    (1, 8, 5, 7, 13, 3),
    (2, 16, 4, 9, 5, 7),
    (1, 64, 3, 10, 9, 296),
    (1, 8, 16, 16, 8, 5),
    (1, 32, 2, 2, 2, 4),
    (3, 8, 1, 1, 1, 2),
    (1, 16, 7, 17, 3, 1),
    (1, 128, 2, 3, 11, 11),
    (1, 8, 9, 3, 70, 6),
    # many columns, few CTAs: whole-column rounds followed by a split remainder
    (1, 8, 5, 40, 70, 4),
    (2, 16, 3, 20, 40, 5),
    (1, 32, 4, 17, 33, 7),
]


@pytest.mark.parametrize('shape', SHAPES, ids=[str(s) for s in SHAPES])
def test_emulated_fprop(kdw_lib, kdw_emu, shape):
    N, C, H, W, D, grid = shape
    x, _, w = _inputs(11, N, C, H, W, D)
    y_exact = o.fprop_exact(x, w).astype(np.float32)
    for v, cs in _variants(kdw_lib, 'fprop'):
        if C % cs:
            continue
        for mode in (0, 1):  # KDW_ACC_F32, KDW_ACC_F16
            y = np.full_like(x, np.nan)
            r = kdw_emu.emu_fprop(v, x.ctypes.data, w.ctypes.data, y.ctypes.data, N, C, H, W, D, H, 0, H, 0, mode, grid)
            if r == -1:
                continue  # tensor-core variants (warp-level mma) are not emulated on the CPU
            assert r > 0
            assert np.isfinite(y).all(), f'variant {v}: output not fully written'
            assert np.allclose(y.astype(np.float32), y_exact, rtol=1e-3, atol=1e-2), f'variant {v} mode={mode}'
            if mode == 0:
                assert o.allclose_two_stage(y, y_exact, rtol_strict=1e-4, atol_strict=1e-3, rtol_narrow=1e-3,
                                            atol_narrow=2e-3), f'variant {v}'


@pytest.mark.parametrize('shape', SHAPES, ids=[str(s) for s in SHAPES])
def test_emulated_wgrad(kdw_lib, kdw_emu, shape):
    N, C, H, W, D, grid = shape
    x, g, _ = _inputs(12, N, C, H, W, D)
    dw_exact = o.wgrad_exact(x, g)
    for v, cs in _variants(kdw_lib, 'wgrad'):
        if C % cs:
            continue
        dw = np.zeros((3, 3, 3, C), np.float32)
        r = kdw_emu.emu_wgrad(v, x.ctypes.data, g.ctypes.data, dw.ctypes.data, N, C, H, W, D, H, 0, H, 0, grid)
        if r == -1:
            continue  # tensor-core variants (warp-level mma) are not emulated on the CPU
        assert r > 0
        err = np.abs(dw - dw_exact).max()
        scale = np.abs(dw_exact).max() + 1.0
        assert err <= 2e-3 * scale, f'variant {v}: {err} vs scale {scale}'


def test_emulated_plane_ranges(kdw_lib, kdw_emu):
    """The H-sharded entry points: planes [h_begin, h_end) of a volume that carries halo planes."""
    N, C, H, W, D = 1, 8, 9, 6, 5
    x, g, w = _inputs(13, N, C, H, W, D)
    y_exact = o.fprop_exact(x, w).astype(np.float32)
    for (hb, he) in [(0, 4), (4, 9), (3, 4), (1, 8)]:
        # y holds only the owned planes: plane h -> y plane h - hb
        y = np.full((N, he - hb, W, D, C), np.nan, np.float16)
        r = kdw_emu.emu_fprop(1, x.ctypes.data, w.ctypes.data, y.ctypes.data, N, C, H, W, D, he - hb, hb, he, hb, 0, 3)
        assert r > 0 and np.isfinite(y).all()
        assert np.allclose(y.astype(np.float32), y_exact[:, hb:he], rtol=1e-3, atol=1e-2)
        # weight gradient of the owned grad planes, grad stored without halo
        gs = np.ascontiguousarray(g[:, hb:he])
        dw = np.zeros((3, 3, 3, C), np.float32)
        r = kdw_emu.emu_wgrad(1, x.ctypes.data, gs.ctypes.data, dw.ctypes.data, N, C, H, W, D, he - hb, hb, he, hb, 3)
        gz = np.zeros_like(g)
        gz[:, hb:he] = g[:, hb:he]
        ref = o.wgrad_exact(x, gz)
        assert np.abs(dw - ref).max() <= 2e-3 * (np.abs(ref).max() + 1.0)
    # shards add up to the full gradient


# ---------------------------------------------------------------------------------------------------------
# The work decomposition shared by host and device code (make_sched, decode_column, decode_remainder,
# StepIter): every (sample, channel slice, tile, plane) unit is owned by exactly one segment, for any shape,
# tile and grid size, and the CTAs' step counts are balanced.
# ---------------------------------------------------------------------------------------------------------
def _schedule(kdw_emu, N, C, W, D, h_begin, h_end, WT, DT, CS, grid_target):
    import ctypes

    nWT, nDT, nCS = -(-W // WT), -(-D // DT), C // CS
    counts = np.zeros(N * nCS * nDT * nWT * (h_end - h_begin), dtype=np.int32)
    lo, hi = ctypes.c_int64(), ctypes.c_int64()
    grid = kdw_emu.emu_schedule(N, C, W, D, h_begin, h_end, WT, DT, CS, grid_target,
                                counts.ctypes.data_as(ctypes.c_void_p), ctypes.byref(lo), ctypes.byref(hi))
    return grid, counts, lo.value, hi.value


def test_schedule_covers_every_unit_once_benchmark_shapes(kdw_emu):
    for C, CS, DT, WT in [(8, 8, 64, 8), (32, 32, 32, 8), (128, 64, 8, 8), (128, 64, 3, 40), (32, 32, 10, 24)]:
        for grid_target in (148, 296):
            grid, counts, lo, hi = _schedule(kdw_emu, 1, C, 350, 128, 0, 350, WT, DT, CS, grid_target)
            assert grid == grid_target
            assert counts.min() == 1 and counts.max() == 1
            # a CTA's steps: its planes plus one extra input plane per segment; balanced to a few per cent
            assert hi - lo <= max(8, 0.03 * hi), (C, CS, DT, WT, grid_target, lo, hi)


def test_schedule_covers_every_unit_once_random_shapes(kdw_emu):
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=150, deadline=None)
    @given(N=st.integers(1, 3), nCS=st.integers(1, 4), W=st.integers(1, 70), D=st.integers(1, 70),
           h0=st.integers(0, 5), Hr=st.integers(1, 40), WT=st.sampled_from([4, 8, 16, 24, 40]),
           DT=st.sampled_from([3, 5, 8, 16, 22, 32, 64]), grid_target=st.integers(1, 300))
    def check(N, nCS, W, D, h0, Hr, WT, DT, grid_target):
        CS = 8
        grid, counts, lo, hi = _schedule(kdw_emu, N, nCS * CS, W, D, h0, h0 + Hr, WT, DT, CS, grid_target)
        assert 1 <= grid <= grid_target
        assert counts.min() == 1 and counts.max() == 1

    check()


# ---------------------------------------------------------------------------------------------------------
# Fused forward + residual add + channel statistics (dwconv_fprop_addstats.cu), every tile of that kernel
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize('which,shape', [(1, (1, 8, 5, 13, 70)), (2, (2, 16, 4, 9, 37)), (3, (1, 32, 6, 11, 21)),
                                         (4, (1, 64, 3, 10, 40)), (5, (2, 64, 4, 7, 9)), (5, (1, 128, 3, 17, 12))])
def test_emulated_fprop_addstats(kdw_emu, which, shape):
    import ctypes

    from oracle import dwconv_oracle as orc

    N, C, H, W, D = shape
    rng = np.random.default_rng(100 + which + C)
    x = rng.standard_normal((N, H, W, D, C)).astype(np.float16)
    r = rng.standard_normal((N, H, W, D, C)).astype(np.float16)
    w = ((rng.random((3, 3, 3, C)) * 2 - 1) / np.sqrt(27)).astype(np.float16)
    y = np.full_like(x, np.float16(777))
    stats = np.zeros(2 * C, dtype=np.float64)
    vp = ctypes.c_void_p
    for grid in (3, 40):
        g = kdw_emu.emu_fprop_addstats(which, x.ctypes.data_as(vp), w.ctypes.data_as(vp), r.ctypes.data_as(vp),
                                       y.ctypes.data_as(vp), stats.ctypes.data_as(vp), N, C, H, W, D, grid)
        assert g > 0
        out, mean, sqmean = orc.addstats_exact(orc.fprop_exact(x, w), r)
        assert np.array_equal(y, out)  # exact products, fp32 sums, one rounding, then an exact fp16 add
        n = N * H * W * D
        np.testing.assert_allclose(stats[:C] / n, mean, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(stats[C:] / n, sqmean, rtol=1e-5, atol=1e-6)


# ---------------------------------------------------------------------------------------------------------
# Fused BN-affine + ReLU prologue (dwconv_fprop_bnrelu.cu), every tile of that kernel
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize('which,shape', [(1, (1, 8, 5, 13, 70)), (2, (2, 16, 4, 9, 37)), (3, (1, 16, 3, 9, 33)),
                                         (4, (1, 64, 3, 10, 40)), (5, (1, 32, 6, 11, 21)), (6, (2, 128, 3, 7, 9))])
def test_emulated_fprop_bnrelu(kdw_emu, which, shape):
    import ctypes

    from oracle import dwconv_oracle as orc

    N, C, H, W, D = shape
    rng = np.random.default_rng(200 + which + C)
    x = rng.standard_normal((N, H, W, D, C)).astype(np.float16)
    w = ((rng.random((3, 3, 3, C)) * 2 - 1) / np.sqrt(27)).astype(np.float16)
    scale = (0.5 + rng.random(C)).astype(np.float32)
    shift = (rng.standard_normal(C) * 0.5 + 0.3).astype(np.float32)  # mostly positive: relu(shift) != 0 on padding
    y = np.full_like(x, np.float16(777))
    vp = ctypes.c_void_p
    ref = orc.fprop_exact(orc.bnrelu_exact(x, scale, shift), w)
    for grid in (3, 40):
        g = kdw_emu.emu_fprop_bnrelu(which, x.ctypes.data_as(vp), scale.ctypes.data_as(vp), shift.ctypes.data_as(vp),
                                     w.ctypes.data_as(vp), y.ctypes.data_as(vp), N, C, H, W, D, grid)
        assert g > 0
        # equal up to the rare double rounding inside the activation (see bnrelu_exact)
        assert (y != ref).mean() < 1e-3
        assert orc.allclose_two_stage(y, ref, rtol_strict=1e-4, atol_strict=1e-3, rtol_narrow=1e-3, atol_narrow=2e-3)
