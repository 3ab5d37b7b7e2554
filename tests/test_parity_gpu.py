"""Parity of the CUDA path (called through the C-ABI) against the oracle, on a B200.

Tolerances: forward rtol 1e-3 / atol 1e-2 against the fp32 oracle rounded to fp16 (north-star bar) and
the reference test's two-stage bound (tests/ops/test_conv.py:28-36); weight gradient relative L2 <= 1e-3
against fp64 and the reference's cosine/norm bound (tests/ops/test_conv.py:74-82)."""
import glob
import os
import random

import numpy as np
import pytest
import torch

from kerops_b200._lib import KdwError
from oracle import dwconv_oracle as o
from oracle import torch_oracle as to

pytestmark = pytest.mark.gpu

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), 'golden', '*.npz')))
LATTICE = [2, 3, 7, 13, 16, 32, 37, 53, 111, 128]  # tests/conftest.py:19-31 of the reference
CHANNELS = [8, 16, 32, 64, 128]


def make_inputs(seed, N, C, H, W, D, device='cuda'):
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(N, H, W, D, C, generator=g, device=device, dtype=torch.float16).permute(0, 4, 1, 2, 3)
    grad = torch.randn(N, H, W, D, C, generator=g, device=device, dtype=torch.float16).permute(0, 4, 1, 2, 3)
    w = ((torch.rand(3, 3, 3, C, generator=g, device=device) * 2 - 1) / 27 ** 0.5).to(torch.float16)
    return x, grad, w


def check_fprop(y, y_ref, strict=True):
    assert y.shape == y_ref.shape and y.dtype == torch.float16
    assert torch.isfinite(y).all()
    yf, rf = y.float(), y_ref.float()
    assert torch.allclose(yf, rf, rtol=1e-3, atol=1e-2), f'max abs err {(yf - rf).abs().max().item()}'
    if strict:  # the reference test's bound; the cheaper accumulate modes only meet the north-star bound
        assert o.allclose_two_stage(y.cpu().numpy(), y_ref.cpu().numpy(), rtol_strict=1e-4, atol_strict=1e-3,
                                    rtol_narrow=1e-3, atol_narrow=2e-3)


def check_wgrad(dw32, dw16, ref64, bsize=1):
    ref = ref64.cpu().numpy()
    if dw32 is not None:
        assert to.rel_l2(dw32.cpu(), ref64.cpu()) <= 1e-3
    if dw16 is not None:
        assert dw16.dtype == torch.float16 and list(dw16.shape) == list(ref64.shape)
        assert o.weight_grad_similarity(ref, dw16.float().cpu().numpy(), rtol_cos=1e-4, atol_cos=1e-4,
                                        rtol_len=1e-3 * bsize, atol_len=1e-3)


def lattice_sample(seed, count, max_size, max_elems):
    rnd = random.Random(seed)
    sizes = [s for s in LATTICE if s <= max_size]
    out = []
    while len(out) < count:
        shp = (rnd.choice([1, 2, 3]), rnd.choice(sizes), rnd.choice(sizes), rnd.choice(sizes))
        if shp[0] * shp[1] * shp[2] * shp[3] <= max_elems:
            out.append(shp)
    return out


@pytest.fixture(scope='module')
def ops(kdw_lib):
    from kerops_b200.ops.conv import DWConv, DWConvWGRAD, _launch

    return DWConv, DWConvWGRAD, _launch


@pytest.fixture(autouse=True)
def _status_clean(kdw_lib):
    yield
    from kerops_b200 import _lib

    assert _lib.device_status() == 0, 'a kernel reported a timed-out barrier wait'


# --------------------------------------------------------------------------------------------------
# golden vectors produced by the reference kernels
# --------------------------------------------------------------------------------------------------
@pytest.mark.parametrize('path', GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_golden(ops, path):
    DWConv, DWConvWGRAD, _ = ops
    z = np.load(path)
    x = torch.from_numpy(z['x']).cuda().permute(0, 4, 1, 2, 3)
    g = torch.from_numpy(z['grad']).cuda().permute(0, 4, 1, 2, 3)
    w = torch.from_numpy(z['weight']).cuda()
    y = DWConv(x, w)
    assert y.is_contiguous(memory_format=torch.channels_last_3d) and y.stride() == x.stride()
    y_ref = torch.from_numpy(z['y']).permute(0, 4, 1, 2, 3)
    # against the reference kernel's own output, with the reference test's tolerance
    assert o.allclose_two_stage(y.cpu().numpy(), y_ref.numpy(), rtol_strict=1e-4, atol_strict=1e-3, rtol_narrow=1e-3,
                                atol_narrow=2e-3)
    check_fprop(y.cpu(), torch.from_numpy(o.fprop_exact(z['x'], z['weight'])).permute(0, 4, 1, 2, 3))
    dw = DWConvWGRAD(x, g)
    ref64 = torch.from_numpy(o.wgrad_exact(z['x'], z['grad']))
    check_wgrad(None, dw, ref64, bsize=x.shape[0])
    assert to.rel_l2(dw.float().cpu(), torch.from_numpy(z['dw']).float()) <= 2e-3  # vs the reference's fp16 output


# --------------------------------------------------------------------------------------------------
# size lattice of the reference tests, plus C = 64 / 128
# --------------------------------------------------------------------------------------------------
@pytest.mark.parametrize('C', CHANNELS)
def test_fprop_lattice(ops, C):
    DWConv, _, _ = ops
    shapes = lattice_sample(100 + C, 10, 128, 40_000_000 // C) + [(1, 2, 2, 2), (1, 3, 3, 3), (4, 7, 2, 13)]
    if C == 8:
        shapes += [(1, 128, 128, 128), (1, 111, 37, 128)]
    for i, (N, H, W, D) in enumerate(shapes):
        x, _, w = make_inputs(1000 * C + i, N, C, H, W, D)
        y = DWConv(x, w)
        check_fprop(y, to.fprop_shift_fp32(x, w))


@pytest.mark.parametrize('C', CHANNELS)
def test_wgrad_lattice(ops, C):
    _, DWConvWGRAD, _launch = ops
    shapes = lattice_sample(200 + C, 8, 53, 10_000_000 // C) + [(1, 2, 2, 2), (1, 3, 3, 3), (2, 111, 16, 37)]
    for i, (N, H, W, D) in enumerate(shapes):
        x, g, _ = make_inputs(2000 * C + i, N, C, H, W, D)
        ref64 = to.wgrad_fp64(x, g)
        dw16 = DWConvWGRAD(x, g)
        dw32, _ = _launch.wgrad(x, g, want_f32=True, want_f16=False)
        check_wgrad(dw32, dw16, ref64, bsize=N)
        assert torch.equal(dw32.to(torch.float16), dw16)


@pytest.mark.parametrize('C', CHANNELS)
def test_dense_small_lattice(ops, C):
    """Every size triple from the small end of the reference's lattice (tests/conftest.py:19-31), every batch size
    1, 2, 4 on a rotating schedule: all tails, sizes below a tile and below the stencil."""
    DWConv, DWConvWGRAD, _launch = ops
    sizes = [2, 3, 7, 13, 16, 32, 37]
    k = 0
    for H in sizes:
        for W in sizes:
            for D in sizes:
                N = (1, 2, 4)[k % 3]
                k += 1
                x, g, w = make_inputs(7000 * C + k, N, C, H, W, D)
                check_fprop(DWConv(x, w), to.fprop_shift_fp32(x, w))
                if k % 2 == 0:  # the weight-gradient oracle is the slower one: every other shape
                    dw32, dw16 = _launch.wgrad(x, g, want_f32=True, want_f16=True)
                    check_wgrad(dw32, dw16, to.wgrad_fp64(x, g), bsize=N)


def test_small_shapes_numpy_oracle(ops):
    """Small cases straight against the numpy oracle (no torch arithmetic on the checking side)."""
    DWConv, DWConvWGRAD, _ = ops
    for i, (N, C, H, W, D) in enumerate([(1, 8, 5, 7, 13), (2, 16, 4, 9, 5), (1, 64, 3, 10, 9), (1, 128, 2, 3, 11),
                                         (3, 8, 1, 1, 1), (1, 32, 9, 3, 70)]):
        x, g, w = make_inputs(300 + i, N, C, H, W, D)
        xn = x.permute(0, 2, 3, 4, 1).contiguous().cpu().numpy()
        gn = g.permute(0, 2, 3, 4, 1).contiguous().cpu().numpy()
        y = DWConv(x, w).permute(0, 2, 3, 4, 1).cpu()
        check_fprop(y, torch.from_numpy(o.fprop_exact(xn, w.cpu().numpy())))
        check_wgrad(None, DWConvWGRAD(x, g), torch.from_numpy(o.wgrad_exact(xn, gn)), bsize=N)


# --------------------------------------------------------------------------------------------------
# every kernel variant, both accumulate types
# --------------------------------------------------------------------------------------------------
VARIANT_SHAPES = [(2, 5, 19, 37), (1, 21, 9, 130)]


def _shape_rejected(e):
    """A variant built for one channel count (or an even D) refuses other shapes with an argument error."""
    return e.code == -4 and 'needs C' in str(e)


def test_all_fprop_variants(ops, kdw_lib):
    _, _, _launch = ops
    for v in range(1, kdw_lib.kdw_fprop_variants() + 1):
        cs = kdw_lib.kdw_fprop_variant_channels(v)
        ran = 0
        for C in sorted({cs, min(128, 2 * cs)}):
            for (N, H, W, D) in VARIANT_SHAPES:
                x, _, w = make_inputs(31 * v + C, N, C, H, W, D)
                ref = to.fprop_shift_fp32(x, w)
                for acc in ('float32', 'float16'):
                    y = torch.full_like(x, float('nan'))
                    try:
                        _launch.fprop(x, w, y, acc=acc, tune=v)
                    except KdwError as e:
                        # tensor-core variants: float32 accumulate type only, some of them one C (and even D) only
                        assert e.code == -4 and (acc == 'float16' or _shape_rejected(e)), e
                        continue
                    check_fprop(y, ref, strict=(acc == 'float32'))
                    ran += 1
        assert ran, f'forward variant {v} ran on none of the shapes'


def test_all_wgrad_variants(ops, kdw_lib):
    _, _, _launch = ops
    for v in range(1, kdw_lib.kdw_wgrad_variants() + 1):
        cs = kdw_lib.kdw_wgrad_variant_channels(v)
        ran = 0
        for C in sorted({cs, min(128, 2 * cs)}):
            for (N, H, W, D) in VARIANT_SHAPES:
                x, g, _ = make_inputs(57 * v + C, N, C, H, W, D)
                try:
                    dw32, dw16 = _launch.wgrad(x, g, want_f32=True, want_f16=True, tune=v)
                except KdwError as e:
                    assert _shape_rejected(e), e
                    continue
                check_wgrad(dw32, dw16, to.wgrad_fp64(x, g), bsize=N)
                ran += 1
        assert ran, f'weight-gradient variant {v} ran on none of the shapes'


def test_sixteen_channel_slices_on_a_mid_size_volume(ops, kdw_lib):
    """(1, 16, 40, 60, 64): the smallest volume on which a long-deleted weight-gradient kernel with 16-channel slices
    stopped with CUDA error 715; every kernel that slices 16 channels today has to pass on it."""
    _, _, _launch = ops
    x, g, w = make_inputs(715, 1, 16, 40, 60, 64)
    ref_y, ref_dw = to.fprop_shift_fp32(x, w), to.wgrad_fp64(x, g)
    ran = 0
    for v in [0] + [v for v in range(1, kdw_lib.kdw_fprop_variants() + 1) if kdw_lib.kdw_fprop_variant_channels(v) == 16]:
        y = torch.full_like(x, float('nan'))
        _launch.fprop(x, w, y, tune=v)
        check_fprop(y, ref_y)
        ran += 1
    for v in [0] + [v for v in range(1, kdw_lib.kdw_wgrad_variants() + 1) if kdw_lib.kdw_wgrad_variant_channels(v) == 16]:
        dw32, dw16 = _launch.wgrad(x, g, want_f32=True, want_f16=True, tune=v)
        check_wgrad(dw32, dw16, ref_dw, bsize=1)
        ran += 1
    assert ran >= 6


def test_acctype_float16_keyword(ops):
    DWConv, _, _ = ops
    x, _, w = make_inputs(77, 1, 16, 20, 21, 22)
    check_fprop(DWConv(x, w, ACCTYPE='float16'), to.fprop_shift_fp32(x, w), strict=False)


def test_plain_kernels_small_channel_counts(ops):
    DWConv, DWConvWGRAD, _ = ops
    for C in (2, 4):
        x, g, w = make_inputs(88 + C, 2, C, 7, 5, 9)
        y = DWConv(x, w, num_warps=1, D_block=8)
        check_fprop(y, to.fprop_shift_fp32(x, w))
        dw = DWConvWGRAD(x, g, num_warps=1, D_block=8, ILP=1)
        check_wgrad(None, dw, to.wgrad_fp64(x, g), bsize=2)


# --------------------------------------------------------------------------------------------------
# determinism, guard bands, plane ranges
# --------------------------------------------------------------------------------------------------
def test_wgrad_bitwise_reproducible(ops):
    _, DWConvWGRAD, _launch = ops
    x, g, _ = make_inputs(5, 2, 32, 37, 53, 64)
    a32, a16 = _launch.wgrad(x, g, want_f32=True, want_f16=True)
    junk = torch.randn(1 << 22, device='cuda')  # move the allocator around between the runs
    b32, b16 = _launch.wgrad(x, g, want_f32=True, want_f16=True)
    del junk
    assert torch.equal(a32, b32) and torch.equal(a16, b16)
    assert torch.equal(DWConvWGRAD(x, g), a16)


def test_guard_bands_stay_untouched(ops):
    _, _, _launch = ops
    N, C, H, W, D = 2, 16, 9, 11, 13
    x, g, w = make_inputs(6, N, C, H, W, D)
    pad = 4096
    buf = torch.full((N * H * W * D * C + 2 * pad,), 1234.0, dtype=torch.float16, device='cuda')
    y = buf[pad:-pad].view(N, H, W, D, C).permute(0, 4, 1, 2, 3)
    _launch.fprop(x, w, y)
    assert (buf[:pad] == 1234.0).all() and (buf[-pad:] == 1234.0).all()
    check_fprop(y, to.fprop_shift_fp32(x, w))
    # workspace and outputs of the weight gradient
    ws = _launch.wgrad_workspace(x)
    big = torch.full((ws.numel() + 2 * pad,), 77, dtype=torch.uint8, device='cuda')
    dw32, dw16 = _launch.wgrad(x, g, want_f32=True, want_f16=True, workspace=big[pad:-pad])
    assert (big[:pad] == 77).all() and (big[-pad:] == 77).all()
    check_wgrad(dw32, dw16, to.wgrad_fp64(x, g), bsize=N)


def test_inputs_are_not_modified(ops):
    DWConv, DWConvWGRAD, _ = ops
    x, g, w = make_inputs(7, 1, 8, 17, 9, 33)
    x0, g0, w0 = x.clone(), g.clone(), w.clone()
    DWConv(x, w)
    DWConvWGRAD(x, g)
    assert torch.equal(x, x0) and torch.equal(g, g0) and torch.equal(w, w0)


def test_plane_ranges_match_full_volume(ops):
    """The H-sharded entry points reproduce the full-volume result plane for plane."""
    _, _, _launch = ops
    N, C, H, W, D = 1, 32, 23, 17, 40
    x, g, w = make_inputs(8, N, C, H, W, D)
    y_full = torch.empty_like(x)
    _launch.fprop(x, w, y_full)
    dw_full, _ = _launch.wgrad(x, g, want_f32=True, want_f16=False)
    parts = []
    for hb, he in [(0, 6), (6, 7), (7, 23)]:
        y = torch.full((N, he - hb, W, D, C), float('nan'), dtype=torch.float16, device='cuda').permute(0, 4, 1, 2, 3)
        _launch.fprop(x, w, y, h_begin=hb, h_end=he, y_h0=hb)
        assert torch.equal(y, y_full[:, :, hb:he])
        gs = g[:, :, hb:he].contiguous(memory_format=torch.channels_last_3d)
        dw, _ = _launch.wgrad(x, gs, h_begin=hb, h_end=he, g_h0=hb, want_f32=True, want_f16=False)
        parts.append(dw.double())
    assert to.rel_l2(sum(parts), dw_full.double()) <= 1e-5
    assert to.rel_l2(sum(parts), to.wgrad_fp64(x, g)) <= 1e-3


def test_stream_and_device_follow_torch(ops):
    DWConv, _, _ = ops
    x, _, w = make_inputs(9, 1, 8, 30, 31, 32)
    ref = to.fprop_shift_fp32(x, w)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        y = DWConv(x, w)
    s.synchronize()
    check_fprop(y, ref)


# --------------------------------------------------------------------------------------------------
# benchmark-size volumes: slabs against the oracle + size-independent properties
# --------------------------------------------------------------------------------------------------
def checksum_property(x, w, y):
    """sum over voxels of y[.., c] == sum over taps of w[tap, c] * (sum of x over the voxels that tap reads),
    evaluated in fp64; returns the largest deviation relative to sum|x| * max|w|."""
    N, C, H, W, D = x.shape
    xl = x.permute(0, 2, 3, 4, 1)
    want = torch.zeros(C, dtype=torch.float64, device=x.device)
    for a in range(3):
        for b in range(3):
            for t in range(3):
                # tap a=0 reads plane h-1, so the last plane is never read by it; a=2 never reads the first
                hs = slice(0, H - 1) if a == 0 else (slice(1, H) if a == 2 else slice(0, H))
                ws = slice(0, W - 1) if b == 0 else (slice(1, W) if b == 2 else slice(0, W))
                ds = slice(0, D - 1) if t == 0 else (slice(1, D) if t == 2 else slice(0, D))
                want += w[a, b, t].double() * xl[:, hs, ws, ds].sum(dim=(0, 1, 2, 3), dtype=torch.float64)
    got = y.permute(0, 2, 3, 4, 1).sum(dim=(0, 1, 2, 3), dtype=torch.float64)
    scale = (xl.abs().sum(dim=(0, 1, 2, 3), dtype=torch.float64) * w.abs().double().amax(dim=(0, 1, 2))).clamp_min(1.0)
    return ((got - want).abs() / scale).max().item()


@pytest.mark.parametrize('C', CHANNELS)
def test_benchmark_volume(ops, C):
    DWConv, DWConvWGRAD, _launch = ops
    N, H, W, D = 1, 350, 350, 128
    x, g, w = make_inputs(4242 + C, N, C, H, W, D)
    y = DWConv(x, w)
    for hb, he in [(0, 5), (173, 178), (345, 350)]:
        lo, hi = max(0, hb - 1), min(H, he + 1)
        ref = to.fprop_shift_fp32(x[:, :, lo:hi], w)[:, :, hb - lo:hb - lo + (he - hb)]
        check_fprop(y[:, :, hb:he], ref)
    assert checksum_property(x, w, y) <= 1e-5
    dw32, dw16 = _launch.wgrad(x, g, want_f32=True, want_f16=True)
    ref64 = to.wgrad_fp64(x, g, chunk=max(1, 64 // C))
    check_wgrad(dw32, dw16, ref64)
    dw32b, _ = _launch.wgrad(x, g, want_f32=True, want_f16=False)
    assert torch.equal(dw32, dw32b)


def test_volume_beyond_2_pow_31_elements(ops):
    """64-bit addressing: (1, 128, 420, 350, 128) has 2.41e9 elements; the reference's int32 offsets
    (kerops/kernels/dw_conv.py:65,128,132) cannot address it."""
    DWConv, _, _launch = ops
    N, C, H, W, D = 1, 128, 420, 350, 128
    x, g, w = make_inputs(99, N, C, H, W, D)
    assert x.numel() > 2 ** 31
    y = DWConv(x, w)
    for hb, he in [(0, 2), (373, 377), (418, 420)]:
        lo, hi = max(0, hb - 1), min(H, he + 1)
        ref = to.fprop_shift_fp32(x[:, :, lo:hi], w)[:, :, hb - lo:hb - lo + (he - hb)]
        check_fprop(y[:, :, hb:he], ref)
    del y
    dw32, _ = _launch.wgrad(x, g, want_f32=True, want_f16=False)
    # planes around the 2^31-element boundary contribute correctly: compare a shard there against fp64
    hb, he = 370, 380
    gs = g[:, :, hb:he].contiguous(memory_format=torch.channels_last_3d)
    part, _ = _launch.wgrad(x, gs, h_begin=hb, h_end=he, g_h0=hb, want_f32=True, want_f16=False)
    gz = torch.zeros_like(g[:, :, hb - 1:he + 1])  # the owned grad planes between two zero planes
    gz[:, :, 1:-1] = g[:, :, hb:he]
    ref = to.wgrad_fp64(x[:, :, hb - 1:he + 1], gz, chunk=1)
    assert to.rel_l2(part, ref) <= 1e-3
    assert torch.isfinite(dw32).all()
