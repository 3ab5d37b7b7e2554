"""Multi-GPU use of the depthwise-conv path: one process per GPU, torch.distributed for the plumbing.

The reference is single-GPU (no distributed code anywhere in kerops); this module adds the two ways the path
shards, neither of which needs a collective on the activation data:

* by SAMPLE - every rank convolves its own samples; the only exchange is one all-reduce of the fp32
  [3,3,3,C] weight gradient (864 B at C=8 ... 13.8 KB at C=128);
* along H (torch dim 2, the outermost spatial axis, whose planes are contiguous slabs) for one large volume -
  rank r owns planes [r*H/G, (r+1)*H/G); a 3-tap stencil needs ONE halo plane from each neighbour.  The local
  buffer holds Hs+2 planes (halo, owned..., halo); neighbours' boundary planes are received into the halo planes
  (point-to-point over NVLink), zero at the two ends of the volume.  The interior planes do not depend on the halo
  and are computed while the exchange is in flight; the two boundary planes follow.  The weight gradient needs
  only the x halo (grad is read at the owned voxel).

The device work goes through `LocalOps`, by default the CUDA kernels behind the C-ABI plane-range entry points
(kdw_fprop_f16_range / kdw_wgrad_f16_range).  Tests of the host logic on CPU (gloo) pass their own LocalOps.

The gradient all-reduce is NCCL's by default; `GradPushAllReduce` is the library's own one-kernel version over
peer memory (kdw_allreduce_push_f32) and can be passed as `reducer=` to the helpers below.
"""
import ctypes

import torch
import torch.distributed as dist


class LocalOps:
    """Device work on one rank: plane-range forward and weight gradient of a halo'd local volume."""

    def fprop_range(self, x_halo, weight, y, h_begin, h_end, y_h0):
        """y[:, :, h - y_h0] = conv(x_halo)[h] for h in [h_begin, h_end)."""
        raise NotImplementedError

    def wgrad_range(self, x_halo, grad, h_begin, h_end, g_h0):
        """fp32 [3,3,3,C]: sum over grad planes h in [h_begin, h_end) (x plane numbering), grad plane h - g_h0."""
        raise NotImplementedError


class CudaOps(LocalOps):
    def fprop_range(self, x_halo, weight, y, h_begin, h_end, y_h0):
        from .ops.conv import _launch

        _launch.fprop(x_halo, weight, y, h_begin=h_begin, h_end=h_end, y_h0=y_h0)

    def wgrad_range(self, x_halo, grad, h_begin, h_end, g_h0):
        from .ops.conv import _launch

        dw32, _ = _launch.wgrad(x_halo, grad, h_begin=h_begin, h_end=h_end, g_h0=g_h0, want_f32=True, want_f16=False)
        return dw32


class GradPushAllReduce:
    """All-reduce (sum) of small fp32 tensors - the [3,3,3,C] weight gradients - through peer stores: one kernel
    per rank pushes its values into every rank's exchange buffer, waits (with a time limit) for the others and
    adds the slots in rank order, so every rank gets the same bits.  A collective: construct it and call it on
    every rank of `group`, always from the same stream.

    The exchange buffers are torch symmetric memory (torch.distributed._symmetric_memory): every rank allocates
    one, the rendezvous maps all of them into every process with access for the local GPU, and the kernel gets
    their addresses.  NVLink multicast is not used and is switched off for the mapping."""

    def __init__(self, max_numel, group=None, device=None, timeout_s=10.0):
        from . import _lib

        self._lib = _lib
        self.lib = _lib.load()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device) if device is not None else torch.device('cuda', torch.cuda.current_device())
        self.max_numel = int(max_numel)
        self.timeout_ns = int(timeout_s * 1e9)
        nbytes = self.lib.kdw_allreduce_buffer_bytes(self.max_numel, self.world)
        if nbytes <= 0:
            raise ValueError(f'GradPushAllReduce: max_numel={max_numel}, world={self.world} not supported')
        if self.world == 1:
            self.buffer = torch.zeros(nbytes // 4, dtype=torch.float32, device=self.device)
            ptrs = [self.buffer.data_ptr()]
        else:
            import os

            os.environ.setdefault('TORCH_SYMM_MEM_DISABLE_MULTICAST', '1')
            import torch.distributed._symmetric_memory as symm_mem

            pg = group if group is not None else dist.group.WORLD
            with torch.cuda.device(self.device):
                self.buffer = symm_mem.empty(nbytes // 4, dtype=torch.float32, device=self.device)
                self.buffer.zero_()  # zero = "no flag raised yet"
                torch.cuda.synchronize(self.device)
                try:
                    self.handle = symm_mem.rendezvous(self.buffer, pg)
                except TypeError:
                    self.handle = symm_mem.rendezvous(self.buffer, pg.group_name)
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
            if len(ptrs) != self.world or ptrs[self.rank] != self.buffer.data_ptr() or not all(ptrs):
                raise RuntimeError(f'GradPushAllReduce: unexpected peer mapping {ptrs} (own {self.buffer.data_ptr()})')
            dist.barrier(group)  # every buffer is zeroed and mapped before anybody pushes
        self._ptrs = (ctypes.c_void_p * self.world)(*ptrs)
        self.seq = 0

    def __call__(self, local, out=None):
        """Returns the sum over ranks of `local` (fp32, contiguous, on this rank's device, numel <= max_numel)."""
        assert local.dtype == torch.float32 and local.is_contiguous() and local.device == self.device
        n = local.numel()
        assert 0 < n <= self.max_numel, f'numel {n} exceeds the {self.max_numel} this reducer was built for'
        if out is None:
            out = torch.empty_like(local)
        assert out.dtype == torch.float32 and out.is_contiguous() and out.numel() == n
        self.seq = self.seq % 0xFFFFFFFE + 1  # 1, 2, ..., 2^32-2, 1, ...: never 0, parity always alternates
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device).cuda_stream
            self._lib.check(self.lib.kdw_allreduce_push_f32(local.data_ptr(), out.data_ptr(), None, self._ptrs, n,
                                                             self.max_numel, self.rank, self.world, self.seq,
                                                             self.timeout_ns, ctypes.c_void_p(stream)))
        return out


def _reduce(dw, group, reducer):
    if reducer is not None:
        return reducer(dw)
    dist.all_reduce(dw, group=group)
    return dw


def shard_planes(H, world, rank):
    """Plane range [begin, end) of the H axis owned by `rank` (contiguous, sizes differ by at most one)."""
    base, extra = divmod(H, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def alloc_halo_volume(N, C, Hs, W, D, device, dtype=torch.float16):
    """channels_last_3d (N, C, Hs+2, W, D) buffer; planes 0 and Hs+1 are the halo planes (zero-initialised)."""
    buf = torch.zeros((N, Hs + 2, W, D, C), dtype=dtype, device=device)
    return buf.permute(0, 4, 1, 2, 3)


def exchange_halo(x_halo, group=None):
    """Fills the two halo planes of a local H-shard from the neighbouring ranks (zero at the volume's ends).

    Starts the transfers and returns a `finish()` callable; call it before anything reads planes 0 and Hs+1.
    On NCCL the transfers run on the process group's own stream and `finish()` only makes the current stream wait
    for them, so kernels launched in between overlap with the exchange."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    Hs = x_halo.shape[2] - 2
    # a rank without planes would send its halo plane as if it were data: every rank must own at least one plane
    assert Hs >= 1, f'H-sharding needs at least one owned plane per rank (this rank has {Hs}; H < world?)'
    phys = x_halo.permute(0, 2, 3, 4, 1)  # (N, Hs+2, W, D, C) contiguous view
    ops = []
    # planes are contiguous only within one sample, so a plane of every sample is sent as one strided tensor
    if rank > 0:
        ops.append(dist.P2POp(dist.isend, phys[:, 1].contiguous(), rank - 1, group))
    if rank < world - 1:
        ops.append(dist.P2POp(dist.isend, phys[:, Hs].contiguous(), rank + 1, group))
    recv_lo = recv_hi = None
    if rank > 0:
        recv_lo = phys[:, 0] if phys[:, 0].is_contiguous() else torch.empty_like(phys[:, 0])
        ops.append(dist.P2POp(dist.irecv, recv_lo, rank - 1, group))
    else:
        phys[:, 0].zero_()
    if rank < world - 1:
        recv_hi = phys[:, Hs + 1] if phys[:, Hs + 1].is_contiguous() else torch.empty_like(phys[:, Hs + 1])
        ops.append(dist.P2POp(dist.irecv, recv_hi, rank + 1, group))
    else:
        phys[:, Hs + 1].zero_()
    reqs = dist.batch_isend_irecv(ops) if ops else []

    def finish():
        for r in reqs:
            r.wait()
        if recv_lo is not None and recv_lo.data_ptr() != phys[:, 0].data_ptr():
            phys[:, 0].copy_(recv_lo)
        if recv_hi is not None and recv_hi.data_ptr() != phys[:, Hs + 1].data_ptr():
            phys[:, Hs + 1].copy_(recv_hi)

    return finish


def hsharded_fprop(x_halo, weight, group=None, ops=None, halo_ready=None):
    """Forward pass of the local H-shard.  x_halo: (N, C, Hs+2, W, D) with the owned planes at 1..Hs.
    If `halo_ready` is None the halo exchange is started here and overlapped with the interior planes.
    Returns y (N, C, Hs, W, D)."""
    ops = ops or CudaOps()
    N, C, Hp, W, D = x_halo.shape
    Hs = Hp - 2
    assert Hs >= 1, 'H-sharding needs at least one owned plane per rank'
    y = torch.empty((N, Hs, W, D, C), dtype=x_halo.dtype, device=x_halo.device).permute(0, 4, 1, 2, 3)
    finish = halo_ready if halo_ready is not None else exchange_halo(x_halo, group)
    if Hs > 2:
        ops.fprop_range(x_halo, weight, y, 2, Hs, 1)  # planes that do not touch the halo
    finish()
    if Hs > 2:
        ops.fprop_range(x_halo, weight, y, 1, 2, 1)
        ops.fprop_range(x_halo, weight, y, Hs, Hs + 1, 1)
    else:
        ops.fprop_range(x_halo, weight, y, 1, Hs + 1, 1)
    return y


def hsharded_wgrad(x_halo, grad, group=None, ops=None, halo_ready=None, reduce=True, reducer=None):
    """Weight gradient of the whole (sharded) volume, fp32 [3,3,3,C], identical on every rank when reduce=True.
    grad: (N, C, Hs, W, D), the owned planes only.  `reducer`: a GradPushAllReduce to use instead of NCCL."""
    ops = ops or CudaOps()
    Hs = x_halo.shape[2] - 2
    assert Hs >= 1, 'H-sharding needs at least one owned plane per rank'
    finish = halo_ready if halo_ready is not None else exchange_halo(x_halo, group)
    dw = None
    if Hs > 2:
        dw = ops.wgrad_range(x_halo, grad, 2, Hs, 1)
    finish()
    if Hs > 2:
        dw = dw + ops.wgrad_range(x_halo, grad, 1, 2, 1) + ops.wgrad_range(x_halo, grad, Hs, Hs + 1, 1)
    else:
        dw = ops.wgrad_range(x_halo, grad, 1, Hs + 1, 1)
    if reduce:
        dw = _reduce(dw, group, reducer)
    return dw


def _mark(events, i):
    if events is not None:
        events[i].record()


def hsharded_step(x_halo, weight, grad, y=None, group=None, ops=None, reducer=None, events=None):
    """Forward pass and weight gradient of the local H-shard as ONE step: the halo exchange is started first and
    overlaps with the forward pass over the planes that do not touch the halo; the two boundary planes follow; the
    weight gradient then needs a single launch over all owned planes, because the halo is in place by then; its
    fp32 result is all-reduced.  x_halo: (N, C, Hs+2, W, D), grad: (N, C, Hs, W, D).  Returns (y, dw_fp32).
    `events`: six CUDA events recorded on the current stream at the phase boundaries (start, interior forward
    done, halo arrived, boundary forward done, weight gradient done, all-reduce done)."""
    ops = ops or CudaOps()
    N, C, Hp, W, D = x_halo.shape
    Hs = Hp - 2
    assert Hs >= 1, 'H-sharding needs at least one owned plane per rank'
    if y is None:
        y = torch.empty((N, Hs, W, D, C), dtype=x_halo.dtype, device=x_halo.device).permute(0, 4, 1, 2, 3)
    sharded = dist.is_initialized() and dist.get_world_size(group) > 1
    _mark(events, 0)
    if sharded and Hs > 2:
        finish = exchange_halo(x_halo, group)
        ops.fprop_range(x_halo, weight, y, 2, Hs, 1)  # planes that do not touch the halo
        _mark(events, 1)
        finish()
        _mark(events, 2)
        ops.fprop_range(x_halo, weight, y, 1, 2, 1)
        ops.fprop_range(x_halo, weight, y, Hs, Hs + 1, 1)
    else:
        _mark(events, 1)
        if sharded:
            exchange_halo(x_halo, group)()
        _mark(events, 2)
        ops.fprop_range(x_halo, weight, y, 1, Hs + 1, 1)
    _mark(events, 3)
    dw = ops.wgrad_range(x_halo, grad, 1, Hs + 1, 1)
    _mark(events, 4)
    if sharded:
        dw = _reduce(dw, group, reducer)
    _mark(events, 5)
    return y, dw


def sample_sharded_step(x, weight, grad, group=None, ops=None, reducer=None, y=None, events=None):
    """Data-parallel slice of a training step: y = DWConv(x) for the local samples and the weight gradient of
    the global batch.  Returns (y, dw_fp32): the local output and the all-reduced fp32 [3,3,3,C] gradient.
    `events`: four CUDA events recorded at the phase boundaries (start, forward, weight gradient, all-reduce)."""
    ops = ops or CudaOps()
    N, C, H, W, D = x.shape
    if y is None:
        y = torch.empty((N, H, W, D, C), dtype=x.dtype, device=x.device).permute(0, 4, 1, 2, 3)
    _mark(events, 0)
    if N > 0:
        ops.fprop_range(x, weight, y, 0, H, 0)
    _mark(events, 1)
    if N > 0:
        dw = ops.wgrad_range(x, grad, 0, H, 0)
    else:  # a rank without samples (batch smaller than the group) still takes part in the sum
        dw = torch.zeros(3, 3, 3, C, dtype=torch.float32, device=x.device)
    _mark(events, 2)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dw = _reduce(dw, group, reducer)
    _mark(events, 3)
    return y, dw
