"""kerops_b200 - depthwise 3x3x3 channels-last fp16 convolution (forward and weight gradient)
for NVIDIA B200, behind the call signatures of kerops.ops.conv.DWConv / DWConvWGRAD."""
__version__ = '0.1.0'
