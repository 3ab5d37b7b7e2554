"""The time-out path of the kernels' bounded waits, exercised without any fault: the test hook
(kdw_test_wait_limits) makes the load warp stop after a few plane copies and shortens the wait limit to 20 ms, so the
compute warps' next wait on a TMA barrier runs out.  The kernel must raise device status 1 and return, the context
must stay usable, and the next call - with the hook switched off - must be correct."""
import pytest
import torch

from oracle import torch_oracle as to

pytestmark = pytest.mark.gpu


def _inputs(seed, N, C, H, W, D):
    g = torch.Generator(device='cuda').manual_seed(seed)
    x = torch.randn(N, H, W, D, C, generator=g, device='cuda', dtype=torch.float16).permute(0, 4, 1, 2, 3)
    grad = torch.randn(N, H, W, D, C, generator=g, device='cuda', dtype=torch.float16).permute(0, 4, 1, 2, 3)
    w = ((torch.rand(3, 3, 3, C, generator=g, device='cuda') * 2 - 1) / 27 ** 0.5).to(torch.float16)
    return x, grad, w


@pytest.fixture
def hook(kdw_lib):
    """Arms the hook for the body of a test and always disarms it (2 s limit, no early stop)."""
    yield kdw_lib
    assert kdw_lib.kdw_test_wait_limits(2_000_000_000, -1) == 0


def _variants(lib, C):
    """(fprop variant, wgrad variant) pairs to exercise: the built-in choice and one CUDA-core table variant."""
    f_table = next(v for v in range(1, 13) if C % lib.kdw_fprop_variant_channels(v) == 0)
    w_table = next(v for v in range(1, 25) if C % lib.kdw_wgrad_variant_channels(v) == 0)
    return [(0, 0), (f_table, w_table)]


@pytest.mark.parametrize('C', [8, 64])
def test_wait_runs_out_and_the_next_call_is_correct(hook, C):
    from kerops_b200 import _lib
    from kerops_b200.ops.conv import _launch

    lib = hook
    x, grad, w = _inputs(3, 1, C, 12, 9, 20)
    y_ref = to.fprop_shift_fp32(x, w)
    dw_ref = to.wgrad_fp64(x, grad)
    assert _lib.device_status() == 0
    for ftune, wtune in _variants(lib, C):
        # forward: the load warp stops after two planes
        assert lib.kdw_test_wait_limits(20_000_000, 2) == 0
        y = torch.zeros_like(x)
        _launch.fprop(x, w, y, tune=ftune)
        assert _lib.device_status() == 1, 'the kernel did not report the wait that ran out'
        assert _lib.device_status() == 0, 'reading the status clears it'
        # weight gradient: same hook
        _launch.wgrad(x, grad, want_f32=True, want_f16=False, tune=wtune)
        assert _lib.device_status() == 1
        # hook off: the context is intact and results are right
        assert lib.kdw_test_wait_limits(2_000_000_000, -1) == 0
        y = torch.full_like(x, float('nan'))
        _launch.fprop(x, w, y, tune=ftune)
        assert torch.allclose(y.float(), y_ref.float(), rtol=1e-3, atol=1e-2)
        dw32, _ = _launch.wgrad(x, grad, want_f32=True, want_f16=False, tune=wtune)
        assert to.rel_l2(dw32.cpu(), dw_ref.cpu()) <= 1e-3
        assert _lib.device_status() == 0


def test_hook_rejects_bad_limits(kdw_lib):
    assert kdw_lib.kdw_test_wait_limits(0, -1) == -1
    assert kdw_lib.kdw_test_wait_limits(2_000_000_000, -1) == 0
