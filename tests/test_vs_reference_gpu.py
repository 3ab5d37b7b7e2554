"""Side by side with the reference itself on the GPU: the unmodified kerops package, installed offline under
baseline/_ref (pip install --no-index --no-deps --target baseline/_ref <kerops checkout>), JIT-compiles its Triton kernels for this GPU; our operators must agree with its
outputs within the tolerances of the reference's own tests (tests/ops/test_conv.py:28-36, 74-82), checked with
the reference's own comparison functions (kerops/utils.py).  Skipped when the install is absent."""
import glob
import math
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, 'baseline', '_ref')
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), 'golden', '*.npz')))


@pytest.fixture(scope='module')
def ref():
    if not os.path.isdir(os.path.join(REF, 'kerops')):
        pytest.skip('reference install baseline/_ref/kerops is not present')
    if REF not in sys.path:
        sys.path.append(REF)  # appended: nothing of this repository is shadowed
    try:
        from kerops.ops.conv import DWConv, DWConvWGRAD
        from kerops.utils import allclose_two_stage, weight_grad_similarity
    except Exception as e:  # e.g. a Triton the reference cannot use
        pytest.skip(f'reference not importable: {type(e).__name__}: {e}')
    return DWConv, DWConvWGRAD, allclose_two_stage, weight_grad_similarity


def _two_stage(fn, a, b):
    return fn(a, b, rtol_strict=1e-4, atol_strict=1e-3, rtol_narrow=1e-3, atol_narrow=2e-3, debug_info='print')


@pytest.mark.parametrize('path', GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_golden_inputs_against_reference_on_gpu(ref, path):
    from kerops_b200.ops.conv import DWConv, DWConvWGRAD

    RefDWConv, RefDWConvWGRAD, two_stage, wsim = ref
    z = np.load(path)
    x = torch.from_numpy(z['x']).cuda().permute(0, 4, 1, 2, 3)
    grad = torch.from_numpy(z['grad']).cuda().permute(0, 4, 1, 2, 3)
    w = torch.from_numpy(z['weight']).cuda()
    y_ref, dw_ref = RefDWConv(x, w), RefDWConvWGRAD(x, grad)
    y, dw = DWConv(x, w), DWConvWGRAD(x, grad)
    assert y.shape == y_ref.shape and y.stride() == y_ref.stride() and y.dtype == y_ref.dtype
    assert dw.shape == dw_ref.shape and dw.dtype == dw_ref.dtype
    assert _two_stage(two_stage, y_ref, y)
    n = x.shape[0]
    assert wsim(dw_ref.float(), dw.float(), rtol_cos=1e-4, atol_cos=1e-4, rtol_len=1e-3 * n, atol_len=1e-3,
                debug_info='print')
    # the committed vectors came from the same kernels under Triton's CPU interpreter
    y_gold = torch.from_numpy(z['y']).cuda().permute(0, 4, 1, 2, 3)
    assert torch.allclose(y_ref.float(), y_gold.float(), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize('C', [8, 16, 32, 64, 128])
@pytest.mark.parametrize('shape', [(1, 37, 16, 53), (2, 13, 32, 7), (1, 111, 3, 128)])
def test_lattice_shapes_against_reference_on_gpu(ref, C, shape):
    from kerops_b200.ops.conv import DWConv, DWConvWGRAD

    RefDWConv, RefDWConvWGRAD, two_stage, wsim = ref
    n, s1, s2, s3 = shape
    torch.manual_seed(322)
    x = torch.randn(n, C, s1, s2, s3, device='cuda', dtype=torch.float16).to(memory_format=torch.channels_last_3d)
    grad = torch.randn(n, C, s1, s2, s3, device='cuda', dtype=torch.float16).to(memory_format=torch.channels_last_3d)
    weight = torch.empty(C, 1, 3, 3, 3, device='cuda', dtype=torch.float16)
    torch.nn.init.kaiming_uniform_(weight, a=math.sqrt(5))
    w = weight[:, 0].permute(1, 2, 3, 0).contiguous()
    assert _two_stage(two_stage, RefDWConv(x, w), DWConv(x, w))
    assert wsim(RefDWConvWGRAD(x, grad).float(), DWConvWGRAD(x, grad).float(), rtol_cos=1e-4, atol_cos=1e-4,
                rtol_len=1e-3 * n, atol_len=1e-3, debug_info='print')
