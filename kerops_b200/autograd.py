"""Autograd wiring of the depthwise 3x3x3 convolution: forward, input gradient and weight gradient.

The reference ships the forward and the weight-gradient operators but no input gradient and no
autograd.Function (a TODO at kerops/kernels/dw_conv.py:145 plans a fused backward).  The input gradient of a
stride-1, pad-1 cross-correlation is the same cross-correlation of the upstream gradient with the taps flipped
on all three axes, so it runs on the forward kernel unchanged.
"""
import torch

from .ops.conv import DWConv, DWConvWGRAD


def DWConvDGRAD(grad, weight, *, ACCTYPE='float32'):
    """Input gradient: dx[n,c,h,w,d] = sum_{a,b,t} grad[n,c,h-a+1,w-b+1,d-t+1] * weight[a,b,t,c].

    grad    (N, C, H, W, D) fp16 CUDA tensor, channels_last_3d
    weight  [3, 3, 3, C] fp16 (kerops layout)
    """
    flipped = torch.flip(weight, dims=(0, 1, 2)).contiguous()
    return DWConv(grad, flipped, ACCTYPE=ACCTYPE)


class DepthwiseConv3dFunction(torch.autograd.Function):
    """y = DWConv(x, weight) with gradients for both arguments."""

    @staticmethod
    def forward(ctx, x, weight):
        ctx.save_for_backward(x, weight)
        return DWConv(x, weight)

    @staticmethod
    def backward(ctx, grad_out):
        x, weight = ctx.saved_tensors
        if not grad_out.is_contiguous(memory_format=torch.channels_last_3d):
            grad_out = grad_out.contiguous(memory_format=torch.channels_last_3d)
        grad_x = DWConvDGRAD(grad_out, weight) if ctx.needs_input_grad[0] else None
        grad_w = DWConvWGRAD(x, grad_out) if ctx.needs_input_grad[1] else None
        return grad_x, grad_w


def depthwise_conv3d(x, weight):
    """Differentiable depthwise 3x3x3 convolution (stride 1, zero padding 1, no bias)."""
    return DepthwiseConv3dFunction.apply(x, weight)


class DepthwiseConv3d(torch.nn.Module):
    """Module form; the parameter is kept in the kerops layout [3, 3, 3, C], fp16."""

    def __init__(self, channels, device=None):
        super().__init__()
        bound = 1.0 / 27 ** 0.5  # kaiming_uniform_(a=sqrt(5)) on a (C, 1, 3, 3, 3) weight
        w = (torch.rand(3, 3, 3, channels, device=device) * 2 - 1) * bound
        self.weight = torch.nn.Parameter(w.to(torch.float16))

    def forward(self, x):
        return depthwise_conv3d(x, self.weight)
