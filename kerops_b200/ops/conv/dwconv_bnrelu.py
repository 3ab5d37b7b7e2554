"""DWConv with the per-channel affine map + ReLU that precedes it in a pre-activation block fused into the same
kernel: DWConvBNReLU(x, bn_weight, bn_bias, weight) == kerops.ops.conv.DWConv(kerops.ops.ApplyBNReLU(x, bn_weight,
bn_bias), weight) (kerops/ops/bnrelu.py:11-43 followed by kerops/ops/conv/dwconv.py:25-63), one pass over memory
instead of two."""
import torch

from . import _launch


def _is_pow2(v):
    return v >= 1 and (v & (v - 1)) == 0


def DWConvBNReLU(x, bn_weight, bn_bias, weight, *, PROLOGUE='float32'):
    """y = DWConv(relu(x * bn_weight[c] + bn_bias[c]), weight).

    x                  (N, C, H, W, D) fp16 CUDA tensor, contiguous in channels_last_3d, C a power of two >= 8
    bn_weight, bn_bias C values each (any float dtype; used in fp32 like the reference's kernel does)
    weight             [3, 3, 3, C] fp16 contiguous
    PROLOGUE           'float32': the activation is computed in fp32 and rounded to fp16, as ApplyBNReLU does;
                       'float16': bn_weight / bn_bias are rounded to fp16 and the activation is one packed-half
                       fused multiply-add with ReLU per channel pair (about 25 % faster)
    Returns a new tensor with the shape, strides and dtype of x."""
    channels = x.shape[1]
    assert x.ndim == 5
    assert x.is_contiguous(memory_format=torch.channels_last_3d)
    assert x.dtype == weight.dtype == torch.float16
    assert _is_pow2(channels) and channels >= 8, 'the fused kernel needs C a power of two >= 8'
    assert PROLOGUE in _launch.ACC_TYPES, f'PROLOGUE must be one of {list(_launch.ACC_TYPES)}'
    assert bn_weight.numel() == bn_bias.numel() == channels
    assert list(weight.shape) == [3, 3, 3, channels] and weight.is_contiguous()
    assert x.is_cuda and weight.device == x.device and bn_weight.device == x.device and bn_bias.device == x.device
    out = torch.empty_like(x)
    if x.numel() == 0:
        return out
    scale = bn_weight.reshape(-1).to(torch.float32).contiguous()
    shift = bn_bias.reshape(-1).to(torch.float32).contiguous()
    _launch.fprop_bnrelu(x, scale, shift, weight, out, prologue=PROLOGUE)
    return out
