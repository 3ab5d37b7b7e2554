"""Operators on host-resident volumes (kerops_b200/host.py): the slab pipeline must give what the device
operators give on the whole volume - bit for bit for the forward pass (same kernels, plane ranges), to fp32
rounding of the slab sums for the weight gradient."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(N, C, H, W, D, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, H, W, D, C, generator=g).half().pin_memory().permute(0, 4, 1, 2, 3)
    grad = torch.randn(N, H, W, D, C, generator=g).half().pin_memory().permute(0, 4, 1, 2, 3)
    w = ((torch.rand(3, 3, 3, C, generator=g) * 2 - 1) / math.sqrt(27)).half()
    return x, grad, w


@pytest.mark.parametrize('shape,slab', [((1, 8, 16, 16, 8), 5), ((2, 32, 13, 7, 37), 4), ((1, 64, 9, 20, 16), 1),
                                        ((1, 16, 6, 5, 8), None)])
def test_host_operators_match_device_operators(shape, slab):
    from kerops_b200.host import DWConvHost, DWConvStepHost, DWConvWGRADHost
    from kerops_b200.ops.conv import DWConv, _launch

    N, C, H, W, D = shape
    x, grad, w = _case(N, C, H, W, D, seed=C + H)
    xd, gd, wd = x.cuda(), grad.cuda(), w.cuda()
    y_ref = DWConv(xd, wd)
    dw32_ref, dw16_ref = _launch.wgrad(xd, gd, want_f32=True, want_f16=True)
    torch.cuda.synchronize()

    y = DWConvHost(x, w, slab_planes=slab)
    assert not y.is_cuda and y.shape == x.shape and y.is_contiguous(memory_format=torch.channels_last_3d)
    assert torch.equal(y, y_ref.cpu())
    dw = DWConvWGRADHost(x, grad, slab_planes=slab)
    assert not dw.is_cuda and dw.dtype == torch.float16 and list(dw.shape) == [3, 3, 3, C]
    rel = float((dw.double() - dw32_ref.cpu().double()).norm() / dw32_ref.cpu().double().norm())
    assert rel <= 5e-4, rel  # fp16 rounding of the result

    out = torch.empty(N, H, W, D, C, dtype=torch.float16).pin_memory().permute(0, 4, 1, 2, 3)
    y2, dw2 = DWConvStepHost(x, w, grad, out=out, slab_planes=slab)
    assert y2.data_ptr() == out.data_ptr()
    assert torch.equal(y2, y_ref.cpu())
    assert torch.equal(dw2, dw)  # same slabs, same order of the fp32 slab sums


def test_host_operators_reject_device_tensors():
    from kerops_b200.host import DWConvHost

    x, _, w = _case(1, 8, 4, 4, 8, seed=1)
    with pytest.raises(AssertionError):
        DWConvHost(x.cuda(), w)
