"""Helpers shared by the GPU tests."""
import torch


def dwconv_cuda_core(x, w):
    """DWConv through a CUDA-core variant of kdw_fprop_f16 (ids 1..12).  The fused operators (DWConvAddStats,
    DWConvBNReLU) run on the CUDA cores and add their fp32 sums in that kernel family's order, so bit-for-bit
    comparisons use it; the built-in choice of DWConv is a tensor-core kernel whose sums are added in another
    order (equal to the last fp16 bit but for about one output in ten thousand)."""
    from kerops_b200 import _lib
    from kerops_b200.ops.conv import _launch

    lib = _lib.load()
    C = x.shape[1]
    tune = next(v for v in range(1, 13) if C % lib.kdw_fprop_variant_channels(v) == 0)
    y = torch.empty_like(x)
    _launch.fprop(x, w, y, tune=tune)
    return y
