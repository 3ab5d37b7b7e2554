"""Argument marshalling between torch tensors and the C-ABI (include/kdw.h)."""
import ctypes
import os

import torch

from ... import _lib

# ACCTYPE keyword -> KDW_ACC_* (include/kdw.h)
ACC_TYPES = {'float32': 0, 'float16': 1}


class _NoSwitch:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def _on(device):
    """Context in which `device` is the current CUDA device: torch's device guard, or nothing at all when it already
    is (the usual case; the guard costs several microseconds of a call that takes some forty)."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


def _stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _env_tune(name):
    """Kernel-variant override from the environment, for timing one variant through the unchanged Python operators:
    KDW_FPROP_TUNE, KDW_WGRAD_TUNE, KDW_ADDSTATS_TUNE, KDW_BNRELU_TUNE = a variant id of the respective entry point
    (1 .. kdw_*_variants()); unset or 0 = the library chooses.  An explicit `tune=` argument wins."""
    v = os.environ.get(name)
    return int(v) if v else 0


def volume_strides(t):
    """(strideN, strideH, strideW) in elements of a channels_last_3d (N, C, H, W, D) tensor."""
    sN, sC, sH, sW, sD = t.stride()
    C = t.shape[1]
    # channels innermost, D next: the only layout the kernels address
    assert sC == 1 or C == 1, 'channel stride must be 1 (channels_last_3d)'
    assert sD == C or t.shape[4] == 1, 'stride of the innermost spatial axis must equal C (channels_last_3d)'
    return sN, sH, sW


def fprop(x, weight, y, h_begin=None, h_end=None, y_h0=0, acc='float32', tune=0):
    """Enqueues y[:, :, h - y_h0] = conv(x)[h] for h in [h_begin, h_end) on x's device / current stream."""
    lib = _lib.load()
    N, C, Hx, W, D = x.shape
    Hy = y.shape[2]
    if h_begin is None:
        h_begin, h_end = 0, Hx
    xs = volume_strides(x)
    ys = volume_strides(y)
    tune = tune or _env_tune('KDW_FPROP_TUNE')
    with _on(x.device):
        rc = lib.kdw_fprop_f16_range(
            x.data_ptr(), weight.data_ptr(), y.data_ptr(), N, C, Hx, W, D, xs[0], xs[1], xs[2], Hy, ys[0], ys[1],
            ys[2], h_begin, h_end, y_h0, ACC_TYPES[acc], tune, _stream_ptr(x.device),
        )
    _lib.check(rc)
    return y


def wgrad_workspace(x):
    lib = _lib.load()
    N, C, H, W, D = x.shape
    with _on(x.device):
        nbytes = lib.kdw_wgrad_workspace_bytes(N, C, H, W, D)
    if nbytes < 0:
        _lib.check(int(nbytes))
    return torch.empty(nbytes, dtype=torch.uint8, device=x.device)


def wgrad(x, grad, h_begin=None, h_end=None, g_h0=0, want_f32=False, want_f16=True, tune=0, workspace=None,
          out_f32=None):
    """Enqueues the weight gradient over grad planes [h_begin, h_end) (x plane numbering).

    `out_f32`, if given, is a contiguous fp32 buffer of 27*C elements that receives the fp32 result (e.g. a slice
    of a gradient bucket that is all-reduced in one call).
    Returns (dw_f32 or None, dw_f16 or None), each [3, 3, 3, C]."""
    lib = _lib.load()
    N, C, Hx, W, D = x.shape
    Hg = grad.shape[2]
    if h_begin is None:
        h_begin, h_end = 0, Hx
    xs = volume_strides(x)
    gs = volume_strides(grad)
    ws = workspace if workspace is not None else wgrad_workspace(x)
    if out_f32 is not None:
        assert out_f32.dtype == torch.float32 and out_f32.is_contiguous() and out_f32.numel() == 27 * C
        dw32, want_f32 = out_f32.view(3, 3, 3, C), True
    else:
        dw32 = torch.empty([3, 3, 3, C], dtype=torch.float32, device=x.device) if want_f32 else None
    dw16 = torch.empty([3, 3, 3, C], dtype=torch.float16, device=x.device) if want_f16 else None
    tune = tune or _env_tune('KDW_WGRAD_TUNE')
    with _on(x.device):
        rc = lib.kdw_wgrad_f16_range(
            x.data_ptr(), grad.data_ptr(), ws.data_ptr(), ws.numel(),
            dw32.data_ptr() if want_f32 else None, dw16.data_ptr() if want_f16 else None,
            N, C, Hx, W, D, xs[0], xs[1], xs[2], Hg, gs[0], gs[1], gs[2], h_begin, h_end, g_h0, tune,
            _stream_ptr(x.device),
        )
    _lib.check(rc)
    return dw32, dw16


def fprop_addstats(x, weight, residual, y, tune=0):
    """Enqueues y = fp16(conv(x)) + residual and returns (mean, sqmean), fp32 [C], of y per channel."""
    lib = _lib.load()
    N, C, H, W, D = x.shape
    xs, rs, ys = volume_strides(x), volume_strides(residual), volume_strides(y)
    tune = tune or _env_tune('KDW_ADDSTATS_TUNE')
    with _on(x.device):
        nbytes = lib.kdw_fprop_addstats_workspace_bytes(N, C, H, W, D)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
        mean = torch.empty(C, dtype=torch.float32, device=x.device)
        sqmean = torch.empty(C, dtype=torch.float32, device=x.device)
        rc = lib.kdw_fprop_addstats_f16(
            x.data_ptr(), weight.data_ptr(), residual.data_ptr(), y.data_ptr(), ws.data_ptr(), nbytes,
            mean.data_ptr(), sqmean.data_ptr(), N, C, H, W, D, xs[0], xs[1], xs[2], rs[0], rs[1], rs[2], ys[0], ys[1],
            ys[2], tune, _stream_ptr(x.device),
        )
    _lib.check(rc)
    return mean, sqmean


def fprop_bnrelu(x, scale, shift, weight, y, prologue='float32', tune=0):
    """Enqueues y = conv(relu(x * scale + shift)) (scale, shift fp32 [C]; prologue arithmetic 'float32' | 'float16')."""
    lib = _lib.load()
    N, C, H, W, D = x.shape
    xs, ys = volume_strides(x), volume_strides(y)
    tune = tune or _env_tune('KDW_BNRELU_TUNE')
    with _on(x.device):
        rc = lib.kdw_fprop_bnrelu_f16(
            x.data_ptr(), scale.data_ptr(), shift.data_ptr(), weight.data_ptr(), y.data_ptr(), N, C, H, W, D, xs[0],
            xs[1], xs[2], ys[0], ys[1], ys[2], ACC_TYPES[prologue], tune, _stream_ptr(x.device),
        )
    _lib.check(rc)
    return y
