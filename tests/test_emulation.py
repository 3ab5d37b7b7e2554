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
