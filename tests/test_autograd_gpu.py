"""Input gradient and autograd wiring against torch's own autograd of conv3d(groups=C) in fp32."""
import pytest
import torch
import torch.nn.functional as F

from oracle import torch_oracle as to

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('shape', [(2, 8, 7, 9, 13), (1, 32, 16, 17, 20), (1, 128, 5, 6, 33)])
def test_gradients_match_torch_autograd(kdw_lib, shape):
    from kerops_b200.autograd import DWConvDGRAD, DepthwiseConv3d, depthwise_conv3d

    N, C, H, W, D = shape
    g = torch.Generator(device='cuda').manual_seed(5)
    x = torch.randn(N, H, W, D, C, generator=g, device='cuda', dtype=torch.float16).permute(0, 4, 1, 2, 3)
    go = torch.randn(N, H, W, D, C, generator=g, device='cuda', dtype=torch.float16).permute(0, 4, 1, 2, 3)
    w = ((torch.rand(3, 3, 3, C, generator=g, device='cuda') * 2 - 1) / 27 ** 0.5).half()

    # fp32 reference through torch autograd (TF32 off so the check is a real fp32 computation)
    old = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        xr = x.float().requires_grad_(True)
        wr = to.to_torch_weight(w).float().requires_grad_(True)
        yr = F.conv3d(xr, wr, None, stride=1, padding=1, groups=C)
        yr.backward(go.float())
    finally:
        torch.backends.cudnn.allow_tf32 = old
    dx_ref = xr.grad
    dw_ref = wr.grad[:, 0].permute(1, 2, 3, 0)

    xa = x.clone().requires_grad_(True)
    wa = w.clone().requires_grad_(True)
    y = depthwise_conv3d(xa, wa)
    y.backward(go)
    assert torch.allclose(y.float(), yr.detach(), rtol=1e-3, atol=1e-2)
    assert xa.grad.dtype == torch.float16 and xa.grad.shape == x.shape
    assert torch.allclose(xa.grad.float(), dx_ref, rtol=1e-3, atol=1e-2)
    assert to.rel_l2(wa.grad.float(), dw_ref) <= 1e-3
    assert torch.equal(DWConvDGRAD(go, w), xa.grad)

    m = DepthwiseConv3d(C, device='cuda')
    out = m(x)
    out.float().square().mean().backward()
    assert m.weight.grad is not None and torch.isfinite(m.weight.grad.float()).all()
