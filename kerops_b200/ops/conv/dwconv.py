"""Forward depthwise 3x3x3 convolution; drop-in for kerops.ops.conv.DWConv
(kerops/ops/conv/dwconv.py:20-63)."""
import torch

from ...settings import ConfigurableArg, confexc, configure
from . import _launch


def _is_pow2(v):
    return v >= 1 and (v & (v - 1)) == 0


# The reference keeps per-C launch tables for C in {8, 16, 32, 64, 128} (dwconv.py:10-17) and raises
# CongiguratorError for any other C unless the caller passes the keywords.  The CUDA kernels pick
# their own tiles, so the values are only validated, but the same C values stay "configured".
@confexc(KeyError)
def warps(channels):
    return {8: 8, 16: 8, 32: 8, 64: 8, 128: 8}[channels]


@confexc(KeyError)
def dblock(channels):
    return {8: 64, 16: 32, 32: 16, 64: 8, 128: 8}[channels]


@configure(
    ACCTYPE='float32',
    num_warps=lambda x: warps(x.shape[1]),
    D_block=lambda x: dblock(x.shape[1]),
)
def DWConv(x, weight, *, ACCTYPE: ConfigurableArg, num_warps: ConfigurableArg, D_block: ConfigurableArg):
    """y = depthwise conv3d(x, weight), kernel 3, stride 1, zero padding 1, no bias.

    x       (N, C, H, W, D) fp16 CUDA tensor, contiguous in channels_last_3d
    weight  [3, 3, 3, C] fp16 contiguous: weight[a, b, t, c] = torch_weight[c, 0, a, b, t]
    ACCTYPE 'float32' (exact products accumulated in fp32, one rounding to fp16) or 'float16' (the reference's faster,
            less accurate mode; here it runs the same fp32-accumulating kernel, so it is neither)
    num_warps, D_block  accepted for call compatibility; D_block must be a power of two
    Returns a new tensor with the shape, strides and dtype of x.
    """
    channels = x.shape[1]

    assert x.ndim == 5
    assert x.is_contiguous(memory_format=torch.channels_last_3d)
    assert x.dtype == weight.dtype == torch.float16
    assert _is_pow2(channels)
    assert list(weight.shape) == [3, 3, 3, channels]
    assert _is_pow2(D_block)
    assert ACCTYPE in _launch.ACC_TYPES, f'ACCTYPE must be one of {list(_launch.ACC_TYPES)}'
    assert x.is_cuda and weight.device == x.device, 'x and weight must be CUDA tensors on one device'
    assert weight.is_contiguous()

    output = torch.empty_like(x)
    if x.numel() == 0:
        return output
    _launch.fprop(x, weight, output, acc=ACCTYPE)
    return output
