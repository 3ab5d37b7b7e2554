"""Operators on HOST-resident volumes: the same DWConv / DWConvWGRAD arithmetic for callers whose
activations live in (pinned) host memory.  They overlap the PCIe copies with the kernels; they do NOT
bound device memory: full-size device copies of the volumes are allocated, so a volume must still fit
on the device.  No counterpart in the reference, which only takes device tensors.

The volume is cut into slabs of h-planes.  Three CUDA streams form a pipeline: slab i+1 is copied
host->device while slab i is convolved (the plane-range entry points of the C-ABI read the halo
planes from the neighbouring slabs already on the device) and the result of slab i-1 is copied
device->host.  Device staging buffers come from torch's allocator.
"""
import torch

from .ops.conv import _launch


__all__ = ['DWConvHost', 'DWConvWGRADHost', 'DWConvStepHost']


def _slabs(H, planes):
    return [(h0, min(H, h0 + planes)) for h0 in range(0, H, planes)]


def _phys(t):
    """(N, H, W, D, C) contiguous view of a channels_last_3d (N, C, H, W, D) tensor."""
    return t.permute(0, 2, 3, 4, 1)


def _check_host_volume(t, name):
    assert t.ndim == 5 and t.dtype == torch.float16, f'{name}: fp16 (N, C, H, W, D) tensor expected'
    assert not t.is_cuda, f'{name}: host tensor expected'
    assert t.is_contiguous(memory_format=torch.channels_last_3d), f'{name}: channels_last_3d expected'


def DWConvHost(x, weight, out=None, *, device='cuda', slab_planes=None, ACCTYPE='float32'):
    """Forward pass of a host volume.  x (and out, if given) should be pinned for the copies to overlap.
    Returns `out` (a pinned host tensor shaped like x)."""
    _check_host_volume(x, 'x')
    N, C, H, W, D = x.shape
    assert list(weight.shape) == [3, 3, 3, C] and weight.dtype == torch.float16
    dev = torch.device(device)
    if out is None:
        out = torch.empty_like(x, pin_memory=True)
    else:
        _check_host_volume(out, 'out')
        assert out.shape == x.shape
    if x.numel() == 0:
        return out
    if slab_planes is None:
        # ~64 MB slabs: large enough for full PCIe rate, small enough to fill the pipeline quickly
        slab_planes = max(1, min(H, (64 << 20) // max(1, W * D * C * 2)))
    w_dev = weight.to(dev, non_blocking=True).contiguous()
    x_dev = torch.empty_like(x, device=dev)
    y_dev = torch.empty_like(x, device=dev)
    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_in.wait_stream(main)
    s_out.wait_stream(main)
    work = [(n, h0, h1) for n in range(N) for (h0, h1) in _slabs(H, slab_planes)]
    copied = []
    for (n, h0, h1) in work:
        with torch.cuda.stream(s_in):
            _phys(x_dev)[n, h0:h1].copy_(_phys(x)[n, h0:h1], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(s_in)
            copied.append(ev)
    for i, (n, h0, h1) in enumerate(work):
        # planes h0-1 .. h1 must be on the device: this slab and, inside one sample, the next one
        need = i + 1 if (i + 1 < len(work) and work[i + 1][0] == n) else i
        main.wait_event(copied[need])
        _launch.fprop(x_dev[n:n + 1], w_dev, y_dev[n:n + 1], h_begin=h0, h_end=h1, y_h0=0, acc=ACCTYPE)
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            _phys(out)[n, h0:h1].copy_(_phys(y_dev)[n, h0:h1], non_blocking=True)
    main.wait_stream(s_out)
    x_dev.record_stream(s_in)
    y_dev.record_stream(s_out)
    main.synchronize()
    return out


def DWConvWGRADHost(x, grad, *, device='cuda', slab_planes=None):
    """Weight gradient of host volumes; returns fp16 [3, 3, 3, C] on the host (fp32 partial sums per slab,
    added in slab order, so the result is reproducible)."""
    _check_host_volume(x, 'x')
    _check_host_volume(grad, 'grad')
    assert x.shape == grad.shape
    N, C, H, W, D = x.shape
    dev = torch.device(device)
    if x.numel() == 0:
        return torch.zeros([3, 3, 3, C], dtype=torch.float16)
    if slab_planes is None:
        slab_planes = max(1, min(H, (64 << 20) // max(1, W * D * C * 2)))
    x_dev = torch.empty_like(x, device=dev)
    g_dev = torch.empty_like(grad, device=dev)
    main = torch.cuda.current_stream(dev)
    s_in = torch.cuda.Stream(dev)
    s_in.wait_stream(main)
    work = [(n, h0, h1) for n in range(N) for (h0, h1) in _slabs(H, slab_planes)]
    copied = []
    for (n, h0, h1) in work:
        with torch.cuda.stream(s_in):
            _phys(x_dev)[n, h0:h1].copy_(_phys(x)[n, h0:h1], non_blocking=True)
            _phys(g_dev)[n, h0:h1].copy_(_phys(grad)[n, h0:h1], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(s_in)
            copied.append(ev)
    ws = _launch.wgrad_workspace(x_dev)
    total = torch.zeros([3, 3, 3, C], dtype=torch.float32, device=dev)
    for i, (n, h0, h1) in enumerate(work):
        need = i + 1 if (i + 1 < len(work) and work[i + 1][0] == n) else i
        main.wait_event(copied[need])
        dw32, _ = _launch.wgrad(x_dev[n:n + 1], g_dev[n:n + 1], h_begin=h0, h_end=h1, g_h0=0, want_f32=True,
                                want_f16=False, workspace=ws)
        total += dw32
    x_dev.record_stream(s_in)
    g_dev.record_stream(s_in)
    result = total.to(torch.float16).cpu()
    return result


def DWConvStepHost(x, weight, grad, out=None, *, device='cuda', slab_planes=None, ACCTYPE='float32'):
    """Forward pass AND weight gradient of a host volume in one sweep: every slab of x crosses the bus once and
    feeds both kernels (a training step needs y = DWConv(x, weight) and dw = DWConvWGRAD(x, grad) of the same x).
    Returns (y, dw): y a pinned host tensor shaped like x (or `out`), dw fp16 [3, 3, 3, C] on the host."""
    _check_host_volume(x, 'x')
    _check_host_volume(grad, 'grad')
    assert x.shape == grad.shape
    N, C, H, W, D = x.shape
    assert list(weight.shape) == [3, 3, 3, C] and weight.dtype == torch.float16
    dev = torch.device(device)
    if out is None:
        out = torch.empty_like(x, pin_memory=True)
    else:
        _check_host_volume(out, 'out')
        assert out.shape == x.shape
    if x.numel() == 0:
        return out, torch.zeros([3, 3, 3, C], dtype=torch.float16)
    if slab_planes is None:
        slab_planes = max(1, min(H, (64 << 20) // max(1, W * D * C * 2)))
    w_dev = weight.to(dev, non_blocking=True).contiguous()
    x_dev = torch.empty_like(x, device=dev)
    g_dev = torch.empty_like(x, device=dev)
    y_dev = torch.empty_like(x, device=dev)
    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_in.wait_stream(main)
    s_out.wait_stream(main)
    work = [(n, h0, h1) for n in range(N) for (h0, h1) in _slabs(H, slab_planes)]
    copied = []
    for (n, h0, h1) in work:
        with torch.cuda.stream(s_in):
            _phys(x_dev)[n, h0:h1].copy_(_phys(x)[n, h0:h1], non_blocking=True)
            _phys(g_dev)[n, h0:h1].copy_(_phys(grad)[n, h0:h1], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(s_in)
            copied.append(ev)
    ws = _launch.wgrad_workspace(x_dev)
    total = torch.zeros([3, 3, 3, C], dtype=torch.float32, device=dev)
    for i, (n, h0, h1) in enumerate(work):
        need = i + 1 if (i + 1 < len(work) and work[i + 1][0] == n) else i
        main.wait_event(copied[need])
        _launch.fprop(x_dev[n:n + 1], w_dev, y_dev[n:n + 1], h_begin=h0, h_end=h1, y_h0=0, acc=ACCTYPE)
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            _phys(out)[n, h0:h1].copy_(_phys(y_dev)[n, h0:h1], non_blocking=True)
        dw32, _ = _launch.wgrad(x_dev[n:n + 1], g_dev[n:n + 1], h_begin=h0, h_end=h1, g_h0=0, want_f32=True,
                                want_f16=False, workspace=ws)
        total += dw32
    main.wait_stream(s_out)
    x_dev.record_stream(s_in)
    g_dev.record_stream(s_in)
    y_dev.record_stream(s_out)
    dw = total.to(torch.float16).cpu()  # synchronises the current stream
    main.synchronize()
    return out, dw
