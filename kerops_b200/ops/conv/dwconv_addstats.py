"""DWConv with the residual add and the channel statistics that follow it in a residual block fused into the
same kernel: DWConvAddStats(x, weight, residual) == kerops.ops.AddStats(kerops.ops.conv.DWConv(x, weight), residual)
(kerops/ops/conv/dwconv.py:25-63 followed by kerops/ops/addition.py:11-49), one pass over memory instead of two."""
import torch

from . import _launch


def _is_pow2(v):
    return v >= 1 and (v & (v - 1)) == 0


def DWConvAddStats(x, weight, residual, inplace=False):
    """out = DWConv(x, weight) + residual (fp16), mean and mean of squares of out per channel (fp32 [C]).

    x, residual  (N, C, H, W, D) fp16 CUDA tensors, contiguous in channels_last_3d, C a power of two >= 8
    weight       [3, 3, 3, C] fp16 contiguous
    inplace      write the result over `residual` (the reference's AddStats(x, y, inplace=True) writes over its
                 first argument, the convolution output, which does not exist here)
    Returns (out, mean, sqmean) like AddStats."""
    channels = x.shape[1]
    assert x.ndim == residual.ndim == 5 and x.shape == residual.shape
    assert x.is_contiguous(memory_format=torch.channels_last_3d)
    assert residual.is_contiguous(memory_format=torch.channels_last_3d)
    assert x.dtype == residual.dtype == weight.dtype == torch.float16
    assert _is_pow2(channels) and channels >= 8, 'the fused kernel needs C a power of two >= 8'
    assert list(weight.shape) == [3, 3, 3, channels] and weight.is_contiguous()
    assert x.is_cuda and weight.device == x.device and residual.device == x.device
    out = residual if inplace else torch.empty_like(x)
    if x.numel() == 0:
        z = torch.zeros(channels, dtype=torch.float32, device=x.device)
        return out, z, z.clone()
    mean, sqmean = _launch.fprop_addstats(x, weight, residual, out)
    return out, mean, sqmean
