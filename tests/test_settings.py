"""Host-side contract of the operators: the @configure keyword injection (kerops/settings/wrapper.py)
and the assertions / exception types of DWConv and DWConvWGRAD (kerops/ops/conv/dwconv.py:28-33,
dwconv_wgrad.py:36-42).  None of this needs a GPU."""
import pytest
import torch

from kerops_b200.ops.conv import DWConv, DWConvWGRAD
from kerops_b200.settings import ConfigurableArg, CongiguratorError, confexc, configure


def test_configure_fills_defaults_and_respects_overrides():
    @confexc(KeyError)
    def table(n):
        return {1: 'one', 2: 'two'}[n]

    @configure(mode='fast', label=lambda n: table(n))
    def op(n, other=5, *, mode: ConfigurableArg, label: ConfigurableArg):
        return n, other, mode, label

    assert op(1) == (1, 5, 'fast', 'one')
    assert op(2, 9, mode='slow') == (2, 9, 'slow', 'two')
    assert op(n=2, label='x') == (2, 5, 'fast', 'x')
    with pytest.raises(CongiguratorError):
        op(3)
    assert op(3, label='given') == (3, 5, 'fast', 'given')
    assert op.can_be_configured(n=1) and not op.can_be_configured(n=3)
    assert 'label: Configurator(n)' in repr(op) and 'mode: fast' in repr(op)
    op.reconfigure(mode='m', label='l')
    assert op(3) == (3, 5, 'm', 'l')
    with pytest.raises(RuntimeError):
        op.reconfigure(mode='m')


def test_configure_signature_rules():
    with pytest.raises(RuntimeError):
        @configure(a=1)
        def bad1(x, a: ConfigurableArg):  # configurable but positional
            pass
    with pytest.raises(RuntimeError):
        @configure()
        def bad2(x, *, a):  # keyword-only but not configurable
            pass
    with pytest.raises(RuntimeError):
        @configure(a=1, b=2)
        def bad3(x, *, a: ConfigurableArg):  # configurator without parameter
            pass


def test_ops_expose_reference_keywords():
    assert DWConv.configurable_args == ['ACCTYPE', 'num_warps', 'D_block']
    assert DWConvWGRAD.configurable_args == ['ACCTYPE', 'num_warps', 'D_block', 'ILP']
    assert DWConv.usual_args == ['x', 'weight'] and DWConvWGRAD.usual_args == ['x', 'grad']
    x = torch.zeros(1, 8, 2, 2, 2)
    assert DWConv.can_be_configured(x=x)
    assert not DWConv.can_be_configured(x=torch.zeros(1, 4, 2, 2, 2))


def _cl(*shape, dtype=torch.float16):
    return torch.zeros(*shape, dtype=dtype).to(memory_format=torch.channels_last_3d)


def test_dwconv_contract_errors_on_host():
    w8 = torch.zeros(3, 3, 3, 8, dtype=torch.float16)
    with pytest.raises(CongiguratorError):  # C outside the configured tables, keywords not given
        DWConv(_cl(1, 4, 4, 4, 4), torch.zeros(3, 3, 3, 4, dtype=torch.float16))
    with pytest.raises(AssertionError):  # not channels_last_3d
        DWConv(torch.zeros(1, 8, 4, 4, 4, dtype=torch.float16), w8)
    with pytest.raises(AssertionError):  # dtype
        DWConv(_cl(1, 8, 4, 4, 4, dtype=torch.float32), w8)
    with pytest.raises(AssertionError):  # weight shape
        DWConv(_cl(1, 8, 4, 4, 4), torch.zeros(8, 3, 3, 3, dtype=torch.float16))
    with pytest.raises(AssertionError):  # D_block must be a power of two
        DWConv(_cl(1, 8, 4, 4, 4), w8, D_block=12)
    with pytest.raises(AssertionError):  # no CPU implementation: CPU tensors are rejected
        DWConv(_cl(1, 8, 4, 4, 4), w8)
    with pytest.raises(AssertionError):  # ndim
        DWConv(torch.zeros(8, 4, 4, 4, dtype=torch.float16), w8, num_warps=1, D_block=8)


def test_dwconv_wgrad_contract_errors_on_host():
    with pytest.raises(CongiguratorError):
        DWConvWGRAD(_cl(1, 4, 4, 4, 4), _cl(1, 4, 4, 4, 4))
    with pytest.raises(AssertionError):  # shape mismatch
        DWConvWGRAD(_cl(1, 8, 4, 4, 4), _cl(1, 8, 4, 4, 5))
    with pytest.raises(AssertionError):  # grad layout
        DWConvWGRAD(_cl(1, 8, 4, 4, 4), torch.zeros(1, 8, 4, 4, 4, dtype=torch.float16))
    with pytest.raises(AssertionError):  # dtype
        DWConvWGRAD(_cl(1, 8, 4, 4, 4), _cl(1, 8, 4, 4, 4, dtype=torch.float32))
    with pytest.raises(AssertionError):  # CPU tensors
        DWConvWGRAD(_cl(1, 8, 4, 4, 4), _cl(1, 8, 4, 4, 4))
