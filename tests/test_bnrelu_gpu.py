"""DWConvBNReLU on the GPU: the fused prologue against the two-operator composition it replaces - a torch
fp32 affine + ReLU rounded to fp16, then our DWConv - and, when the reference install is present, the
reference's own DWConv(ApplyBNReLU(x, w, b), weight)."""
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
    w = ((torch.rand(3, 3, 3, C, generator=g, device='cuda') * 2 - 1) / math.sqrt(27)).half()
    scale = 0.5 + torch.rand(C, generator=g, device='cuda')
    shift = torch.randn(C, generator=g, device='cuda') * 0.5 + 0.3  # mostly positive: relu(shift) != 0 on padding
    return x, scale, shift, w


def _composition(x, scale, shift, w):
    from ._util import dwconv_cuda_core

    s = scale.view(1, -1, 1, 1, 1).double()
    b = shift.view(1, -1, 1, 1, 1).double()
    # fp64 then fp32: an fp16 x fp32 product is exact in a double, so this is a fused multiply-add but for the
    # rare double rounding
    act = torch.clamp_min((x.double() * s + b).float(), 0).half().contiguous(memory_format=torch.channels_last_3d)
    return dwconv_cuda_core(act, w)


@pytest.mark.parametrize('shape', [(1, 8, 16, 16, 8), (2, 8, 5, 13, 70), (1, 16, 7, 37, 33), (1, 16, 4, 9, 128),
                                   (2, 32, 13, 9, 53), (1, 32, 6, 20, 128), (1, 64, 9, 21, 40), (1, 128, 5, 18, 17),
                                   (1, 256, 3, 9, 8)])
def test_fused_equals_composition(shape):
    from kerops_b200 import _lib
    from kerops_b200.ops.conv import DWConvBNReLU

    N, C, H, W, D = shape
    x, scale, shift, w = _inputs(N, C, H, W, D, seed=C + W)
    x0 = x.clone()
    y = DWConvBNReLU(x, scale, shift, w)
    ref = _composition(x, scale, shift, w)
    assert y.shape == x.shape and y.stride() == x.stride() and y.dtype == torch.float16
    assert float((y != ref).float().mean()) < 1e-3  # equal but for double rounding inside the activation
    torch.testing.assert_close(y.float(), ref.float(), rtol=1e-3, atol=2e-3)
    assert torch.equal(x, x0)
    assert torch.equal(y, DWConvBNReLU(x, scale, shift, w))
    assert _lib.device_status() == 0


def test_benchmark_volume():
    """(1, 32, 350, 350, 128), the benchmark volume at one channel count, against the composition (the activation
    is formed slab by slab to bound the fp64 temporaries)."""
    from kerops_b200 import _lib
    from kerops_b200.ops.conv import DWConvBNReLU

    from ._util import dwconv_cuda_core

    N, C, H, W, D = 1, 32, 350, 350, 128
    x, scale, shift, w = _inputs(N, C, H, W, D, seed=9)
    y = DWConvBNReLU(x, scale, shift, w)
    act = torch.empty_like(x)
    s = scale.view(1, -1, 1, 1, 1).double()
    b = shift.view(1, -1, 1, 1, 1).double()
    for h0 in range(0, H, 50):
        act[:, :, h0:h0 + 50] = torch.clamp_min((x[:, :, h0:h0 + 50].double() * s + b).float(), 0).half()
    ref = dwconv_cuda_core(act, w)
    del act
    mismatches = 0
    for h0 in range(0, H, 50):
        ys, rs = y[:, :, h0:h0 + 50], ref[:, :, h0:h0 + 50]
        mismatches += int((ys != rs).sum())
        torch.testing.assert_close(ys.float(), rs.float(), rtol=1e-3, atol=2e-3)
    assert mismatches < 1e-3 * y.numel()  # equal but for double rounding inside the activation
    assert _lib.device_status() == 0


def test_every_tile():
    from kerops_b200 import _lib
    from kerops_b200.ops.conv import _launch

    lib = _lib.load()
    n_var = lib.kdw_fprop_bnrelu_variants()
    assert n_var >= 6
    x, scale, shift, w = _inputs(2, 64, 7, 19, 45, seed=5)
    ref = _composition(x, scale, shift, w)
    for tune in range(1, n_var + 1):
        y = torch.full_like(x, float('nan'))
        _launch.fprop_bnrelu(x, scale, shift, w, y, tune=tune)
        assert float((y != ref).float().mean()) < 1e-3, tune
        torch.testing.assert_close(y.float(), ref.float(), rtol=1e-3, atol=2e-3)
    assert _lib.device_status() == 0


def test_identity_prologue_is_plain_dwconv_of_relu():
    from kerops_b200.ops.conv import DWConv, DWConvBNReLU

    from kerops_b200.ops.conv import _launch

    from ._util import dwconv_cuda_core

    x, _, _, w = _inputs(1, 32, 9, 17, 40, seed=3)
    one, zero = torch.ones(32, device='cuda'), torch.zeros(32, device='cuda')
    xr = torch.relu(x)
    # the built-in choice is the tensor-core forward tile 17 with the activation applied to its operands: the same
    # bits as that tile on relu(x), in both prologue arithmetics (scale 1 and shift 0 are exact in fp16)
    ref = torch.empty_like(xr)
    _launch.fprop(xr, w, ref, tune=17)
    assert torch.equal(DWConvBNReLU(x, one, zero, w), ref)
    assert torch.equal(DWConvBNReLU(x, one, zero, w, PROLOGUE='float16'), ref)
    # a CUDA-core tile of the fused kernel against a CUDA-core variant of the plain forward pass: same order of the
    # fp32 sums, same bits
    y = torch.empty_like(x)
    _launch.fprop_bnrelu(x, one, zero, w, y, tune=4)
    assert torch.equal(y, dwconv_cuda_core(xr, w))
    # ... and to the last fp16 bit almost everywhere against the tensor-core tile
    assert float((y != ref).float().mean()) < 1e-3
    torch.testing.assert_close(y.float(), ref.float(), rtol=1e-3, atol=2e-3)


def test_against_reference_two_operator_chain():
    if not os.path.isdir(os.path.join(REF, 'kerops')):
        pytest.skip('reference install baseline/_ref/kerops is not present')
    if REF not in sys.path:
        sys.path.append(REF)
    try:
        from kerops.ops.bnrelu import ApplyBNReLU
        from kerops.ops.conv import DWConv as RefDWConv
        from kerops.utils import allclose_two_stage
    except Exception as e:
        pytest.skip(f'reference not importable: {type(e).__name__}: {e}')
    from kerops_b200.ops.conv import DWConvBNReLU

    for shape in [(1, 16, 16, 32, 64), (2, 64, 8, 16, 32)]:
        x, scale, shift, w = _inputs(*shape, seed=11)
        ref = RefDWConv(ApplyBNReLU(x, scale, shift), w)
        y = DWConvBNReLU(x, scale, shift, w)
        assert allclose_two_stage(ref, y, rtol_strict=1e-4, atol_strict=1e-3, rtol_narrow=1e-3, atol_narrow=4e-3,
                                  debug_info='print')


@pytest.mark.parametrize('shape', [(2, 8, 5, 13, 70), (1, 16, 7, 37, 33), (2, 16, 6, 11, 34), (1, 32, 6, 20, 128),
                                   (1, 64, 9, 21, 40), (1, 128, 5, 18, 17), (1, 256, 4, 9, 20)])
def test_packed_half_prologue(shape):
    """PROLOGUE='float16': scale and shift rounded to fp16, activation = one fused multiply-add with ReLU rounded
    once to fp16; equal to that arithmetic done in fp64 and, loosely, to the fp32 prologue."""
    from kerops_b200 import _lib
    from kerops_b200.ops.conv import DWConv, DWConvBNReLU

    N, C, H, W, D = shape
    x, scale, shift, w = _inputs(N, C, H, W, D, seed=2 * C + D)
    y = DWConvBNReLU(x, scale, shift, w, PROLOGUE='float16')
    s16 = scale.half().view(1, -1, 1, 1, 1).double()
    b16 = shift.half().view(1, -1, 1, 1, 1).double()
    act = torch.clamp_min(x.double() * s16 + b16, 0).half().contiguous(memory_format=torch.channels_last_3d)
    from kerops_b200.ops.conv import _launch

    from ._util import dwconv_cuda_core

    # Where a tensor-core tile takes the shape, the fused kernel is that forward tile with the activation applied to
    # its operands: the same bits as the tile (a kdw_fprop_f16 variant id) run on the activated tensor.
    twin = {8: 19, 16: 20 if D % 2 == 0 else 0, 32: 17}.get(C, 13)
    if twin:
        ref = torch.empty_like(act)
        _launch.fprop(act, w, ref, tune=twin)
        # bit for bit, but for the handful of activations where torch's double -> float -> half conversion above
        # rounds twice and the kernel's fused multiply-add once
        bad = int((y != ref).sum())
        assert bad <= 2 + 1e-4 * y.numel(), f'{bad} of {y.numel()} outputs differ from forward tile {twin}'
        torch.testing.assert_close(y.float(), ref.float(), rtol=2e-3, atol=2e-3)
    core = dwconv_cuda_core(act, w)
    assert float((y != core).float().mean()) < 1e-3  # another order of the fp32 sums: last-bit differences only
    torch.testing.assert_close(y.float(), core.float(), rtol=1e-3, atol=2e-3)
    y32 = DWConvBNReLU(x, scale, shift, w)
    torch.testing.assert_close(y.float(), y32.float(), rtol=1e-2, atol=1e-2)  # only scale / shift rounding differs
    assert _lib.device_status() == 0
