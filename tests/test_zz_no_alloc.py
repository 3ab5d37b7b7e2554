"""kdw_wgrad_f16_static: the weight gradient for callers that cannot hand the library a workspace because they
must not allocate device memory around the call (latency-critical loops that cannot afford cudaMalloc's device
synchronisation, fixed memory budgets, plain-C embedders that own no allocator).  Collected last on purpose, so
a failure here cannot hide any other test in a run that stops at the first failure."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _volume(seed, N, C, H, W, D):
    g = torch.Generator(device='cuda').manual_seed(seed)
    x = torch.randn(N, H, W, D, C, generator=g, device='cuda', dtype=torch.float16).permute(0, 4, 1, 2, 3)
    grad = torch.randn(N, H, W, D, C, generator=g, device='cuda', dtype=torch.float16).permute(0, 4, 1, 2, 3)
    return x, grad


def _static(lib, x, grad):
    from kerops_b200 import _lib
    from kerops_b200.ops.conv import _launch

    N, C, H, W, D = x.shape
    xs, gs = _launch.volume_strides(x), _launch.volume_strides(grad)
    dw32 = torch.empty(3, 3, 3, C, dtype=torch.float32, device='cuda')
    dw16 = torch.empty(3, 3, 3, C, dtype=torch.float16, device='cuda')
    rc = lib.kdw_wgrad_f16_static(x.data_ptr(), grad.data_ptr(), dw32.data_ptr(), dw16.data_ptr(), N, C, H, W, D,
                                  xs[0], xs[1], xs[2], gs[0], gs[1], gs[2],
                                  ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(rc)
    return dw32, dw16


def test_static_workspace_entry_point_matches_the_allocating_one(kdw_lib):
    from kerops_b200 import _lib
    from kerops_b200.ops.conv import _launch

    # two calls in a row on different data: the shared built-in rows must not leak from one call into the next
    for seed, shape in [(1, (2, 32, 23, 37, 40)), (2, (1, 128, 9, 21, 33)), (3, (1, 4, 5, 6, 7))]:
        x, grad = _volume(seed, *shape)
        ref32, ref16 = _launch.wgrad(x, grad, want_f32=True, want_f16=True)
        got32, got16 = _static(kdw_lib, x, grad)
        torch.cuda.synchronize()
        err = float((got32.double() - ref32.double()).norm() / ref32.double().norm())
        assert err <= 1e-5, f'shape {shape}: relative L2 difference {err}'
        assert torch.allclose(got16.float(), ref16.float(), rtol=2e-3, atol=1e-3)
        # and against the fp64 oracle, with the bar of the other weight-gradient tests
        from oracle import torch_oracle as to

        assert to.rel_l2(got32.cpu(), to.wgrad_fp64(x, grad).cpu()) <= 1e-3
    assert _lib.device_status() == 0


def test_static_workspace_rejects_sizes_beyond_its_limit(kdw_lib):
    x, grad = _volume(4, 1, 256, 3, 4, 5)
    with pytest.raises(RuntimeError, match='built-in workspace'):
        _static(kdw_lib, x, grad)
