"""DWConvAddStats on the GPU: the fused kernel against the two-operator composition it replaces - our DWConv
followed by a torch fp16 add and fp32 channel means (bit-exact output), and, when the reference install is
present, the reference's own AddStats(DWConv(x, weight), residual)."""
import math
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, 'baseline', '_ref')


def _inputs(N, C, H, W, D, seed):
    g = torch.Generator(device='cuda').manual_seed(seed)
    x = torch.randn(N, H, W, D, C, generator=g, device='cuda', dtype=torch.float16).permute(0, 4, 1, 2, 3)
    r = torch.randn(N, H, W, D, C, generator=g, device='cuda', dtype=torch.float16).permute(0, 4, 1, 2, 3)
    w = ((torch.rand(3, 3, 3, C, generator=g, device='cuda') * 2 - 1) / math.sqrt(27)).half()
    return x, r, w


def _composition(x, r, w, cuda_core=False):
    """DWConv followed by a torch fp16 add and fp32 channel means.  The fused kernel runs on the CUDA cores; the
    convolution it is compared with bit for bit is a CUDA-core variant of kdw_fprop_f16 too (same order of the fp32
    sums).  The built-in choice of DWConv - a tensor-core kernel, whose fp32 sums are added in another order - must
    agree to the last fp16 bit almost everywhere."""
    from kerops_b200.ops.conv import DWConv

    from kerops_b200.ops.conv import _launch

    from ._util import dwconv_cuda_core

    # The fused kernel is, where a tensor-core forward tile takes the shape, that tile (a kdw_fprop_f16 variant id)
    # with the add and the sums in its epilogue; elsewhere a CUDA-core kernel.  Same arithmetic, same bits.
    C, D = x.shape[1], x.shape[4]
    twin = 0 if cuda_core else {8: 19, 16: 20 if D % 2 == 0 else 0, 32: 17}.get(C, 22)
    if twin:
        y = torch.empty_like(x)
        _launch.fprop(x, w, y, tune=twin)
    else:
        y = dwconv_cuda_core(x, w)
    y_default = DWConv(x, w, num_warps=8, D_block=8)  # keywords given: any power-of-two C is then accepted
    assert float((y != y_default).float().mean()) < 1e-3
    torch.testing.assert_close(y.float(), y_default.float(), rtol=1e-3, atol=2e-3)
    out = y + r
    o = out.float()
    return out, o.mean(dim=(0, 2, 3, 4)), (o * o).mean(dim=(0, 2, 3, 4))


@pytest.mark.parametrize('shape', [(1, 8, 16, 16, 8), (2, 8, 5, 13, 70), (1, 16, 7, 37, 33), (2, 32, 13, 9, 53),
                                   (1, 32, 6, 20, 128), (1, 64, 9, 21, 40), (1, 128, 5, 18, 17), (1, 256, 3, 9, 8)])
def test_fused_equals_composition(shape):
    from kerops_b200 import _lib
    from kerops_b200.ops.conv import DWConvAddStats

    N, C, H, W, D = shape
    x, r, w = _inputs(N, C, H, W, D, seed=C + W)
    x0, r0 = x.clone(), r.clone()
    out, mean, sqmean = DWConvAddStats(x, w, r)
    out_ref, mean_ref, sq_ref = _composition(x, r, w)
    assert out.shape == x.shape and out.stride() == x.stride() and out.dtype == torch.float16
    assert mean.dtype == sqmean.dtype == torch.float32 and list(mean.shape) == [C]
    assert torch.equal(out, out_ref)
    torch.testing.assert_close(mean, mean_ref, rtol=2e-5, atol=2e-6)
    torch.testing.assert_close(sqmean, sq_ref, rtol=2e-5, atol=2e-6)
    assert torch.equal(x, x0) and torch.equal(r, r0)  # inputs untouched
    out2, mean2, sq2 = DWConvAddStats(x, w, r)
    assert torch.equal(mean, mean2) and torch.equal(sqmean, sq2)  # no atomics: same bits every run
    assert _lib.device_status() == 0


def test_benchmark_volume():
    """(1, 32, 350, 350, 128), the benchmark volume at one channel count: output bits against the composition,
    statistics against fp64 sums taken slab by slab."""
    from kerops_b200 import _lib
    from kerops_b200.ops.conv import DWConvAddStats

    from ._util import dwconv_cuda_core

    N, C, H, W, D = 1, 32, 350, 350, 128
    x, r, w = _inputs(N, C, H, W, D, seed=9)
    out, mean, sqmean = DWConvAddStats(x, w, r)
    from kerops_b200.ops.conv import _launch

    ref = torch.empty_like(x)
    _launch.fprop(x, w, ref, tune=17)  # the forward tile whose epilogue the fused kernel extends
    ref += r
    assert torch.equal(out, ref)
    del ref
    s1 = torch.zeros(C, dtype=torch.float64, device='cuda')
    s2 = torch.zeros(C, dtype=torch.float64, device='cuda')
    for h0 in range(0, H, 50):
        o = out[:, :, h0:h0 + 50].double()
        s1 += o.sum(dim=(0, 2, 3, 4))
        s2 += (o * o).sum(dim=(0, 2, 3, 4))
    n = N * H * W * D
    torch.testing.assert_close(mean.double(), s1 / n, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(sqmean.double(), s2 / n, rtol=1e-5, atol=1e-6)
    assert _lib.device_status() == 0


def test_every_tile_and_inplace():
    from kerops_b200 import _lib
    from kerops_b200.ops.conv import DWConvAddStats, _launch

    lib = _lib.load()
    n_var = lib.kdw_fprop_addstats_variants()
    assert n_var >= 5
    x, r, w = _inputs(2, 64, 7, 19, 45, seed=5)
    out_ref, mean_ref, sq_ref = _composition(x, r, w, cuda_core=True)
    for tune in range(1, n_var + 1):
        y = torch.full_like(x, float('nan'))
        mean, sqmean = _launch.fprop_addstats(x, w, r, y, tune=tune)
        assert torch.equal(y, out_ref), tune
        torch.testing.assert_close(mean, mean_ref, rtol=2e-5, atol=2e-6)
        torch.testing.assert_close(sqmean, sq_ref, rtol=2e-5, atol=2e-6)
    r2 = r.clone()
    out, _, _ = DWConvAddStats(x, w, r2, inplace=True)  # the built-in choice, writing over the residual
    assert out.data_ptr() == r2.data_ptr() and torch.equal(r2, _composition(x, r, w)[0])
    assert _lib.device_status() == 0


def test_contract():
    from kerops_b200.ops.conv import DWConvAddStats

    x, r, w = _inputs(1, 8, 4, 4, 8, seed=1)
    with pytest.raises(AssertionError):
        DWConvAddStats(x, w, r[:, :, :2])
    with pytest.raises(AssertionError):
        DWConvAddStats(x.float(), w, r)
    with pytest.raises(AssertionError):
        DWConvAddStats(x[:, :4].contiguous(memory_format=torch.channels_last_3d), w[..., :4].contiguous(),
                       r[:, :4].contiguous(memory_format=torch.channels_last_3d))


def test_against_reference_two_operator_chain():
    if not os.path.isdir(os.path.join(REF, 'kerops')):
        pytest.skip('reference install baseline/_ref/kerops is not present')
    if REF not in sys.path:
        sys.path.append(REF)
    try:
        from kerops.ops.addition import AddStats
        from kerops.ops.conv import DWConv as RefDWConv
        from kerops.utils import allclose_two_stage
    except Exception as e:
        pytest.skip(f'reference not importable: {type(e).__name__}: {e}')
    from kerops_b200.ops.conv import DWConvAddStats

    for shape in [(1, 16, 16, 32, 64), (2, 64, 8, 16, 32)]:
        x, r, w = _inputs(*shape, seed=11)
        out_ref, mean_ref, sq_ref = AddStats(RefDWConv(x, w), r)
        out, mean, sqmean = DWConvAddStats(x, w, r)
        assert allclose_two_stage(out_ref, out, rtol_strict=1e-4, atol_strict=1e-3, rtol_narrow=1e-3, atol_narrow=4e-3,
                                  debug_info='print')
        torch.testing.assert_close(mean, mean_ref.to(torch.float32).flatten(), rtol=1e-3, atol=1e-4)
        torch.testing.assert_close(sqmean, sq_ref.to(torch.float32).flatten(), rtol=1e-3, atol=1e-4)
