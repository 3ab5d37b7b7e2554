from .dwconv import DWConv
from .dwconv_addstats import DWConvAddStats
from .dwconv_bnrelu import DWConvBNReLU
from .dwconv_wgrad import DWConvWGRAD

__all__ = ['DWConv', 'DWConvWGRAD', 'DWConvAddStats', 'DWConvBNReLU']
