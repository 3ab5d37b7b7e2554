"""Host logic of the multi-GPU layer (kerops_b200/dist.py) on CPU: two gloo ranks, the device work replaced by
the oracle (tests may use it; the product path uses the CUDA kernels)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kerops_b200 import dist as kd
from oracle import torch_oracle as to


class OracleOps(kd.LocalOps):
    """Plane-range forward / weight gradient computed by the torch oracle on CPU tensors."""

    def fprop_range(self, x_halo, weight, y, h_begin, h_end, y_h0):
        lo, hi = max(0, h_begin - 1), min(x_halo.shape[2], h_end + 1)
        full = to.fprop_shift_fp32(x_halo[:, :, lo:hi], weight)
        # planes outside [0, Hx) read as zero: fprop_shift_fp32 pads the slab with zeros, which is the same
        y[:, :, h_begin - y_h0:h_end - y_h0] = full[:, :, h_begin - lo:h_end - lo]

    def wgrad_range(self, x_halo, grad, h_begin, h_end, g_h0):
        lo, hi = max(0, h_begin - 1), min(x_halo.shape[2], h_end + 1)
        xs = x_halo[:, :, lo:hi]
        gs = torch.zeros_like(xs)
        gs[:, :, h_begin - lo:h_end - lo] = grad[:, :, h_begin - g_h0:h_end - g_h0]
        return to.wgrad_fp64(xs, gs, chunk=4).float()


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _full_volume(seed, N, C, H, W, D):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, H, W, D, C, generator=g).half().permute(0, 4, 1, 2, 3)
    grad = torch.randn(N, H, W, D, C, generator=g).half().permute(0, 4, 1, 2, 3)
    w = ((torch.rand(3, 3, 3, C, generator=g) * 2 - 1) / 27 ** 0.5).half()
    return x, grad, w


def _worker(rank, world, port, shape, out_dir):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        N, C, H, W, D = shape
        x, grad, w = _full_volume(123, N, C, H, W, D)  # every rank builds the same volume and takes its shard
        ops = OracleOps()
        # ---- H-sharded volume with halo exchange
        hb, he = kd.shard_planes(H, world, rank)
        xh = kd.alloc_halo_volume(N, C, he - hb, W, D, 'cpu')
        xh[:, :, 1:-1] = x[:, :, hb:he]
        y = kd.hsharded_fprop(xh, w, ops=ops)
        gl = grad[:, :, hb:he].contiguous(memory_format=torch.channels_last_3d)
        xh2 = kd.alloc_halo_volume(N, C, he - hb, W, D, 'cpu')
        xh2[:, :, 1:-1] = x[:, :, hb:he]
        dw = kd.hsharded_wgrad(xh2, gl, ops=ops)
        # ---- sample-sharded step: rank r takes samples r::world
        ys, dws = kd.sample_sharded_step(x[rank::world].contiguous(memory_format=torch.channels_last_3d), w,
                                         grad[rank::world].contiguous(memory_format=torch.channels_last_3d), ops=ops)
        # ---- the same two reductions through a caller-supplied reducer (the place GradPushAllReduce plugs in)
        calls = []

        def reducer(t):
            calls.append(t.numel())
            dist.all_reduce(t)
            return t

        xh3 = kd.alloc_halo_volume(N, C, he - hb, W, D, 'cpu')
        xh3[:, :, 1:-1] = x[:, :, hb:he]
        dw_r = kd.hsharded_wgrad(xh3, gl, ops=ops, reducer=reducer)
        _, dws_r = kd.sample_sharded_step(x[rank::world].contiguous(memory_format=torch.channels_last_3d), w,
                                          grad[rank::world].contiguous(memory_format=torch.channels_last_3d), ops=ops,
                                          reducer=reducer)
        assert calls == [27 * C, 27 * C] and torch.equal(dw_r, dw) and torch.equal(dws_r, dws)
        # ---- forward + weight gradient as one step (halo exchange overlapped, one weight-gradient range)
        xh4 = kd.alloc_halo_volume(N, C, he - hb, W, D, 'cpu')
        xh4[:, :, 1:-1] = x[:, :, hb:he]
        y_s, dw_s = kd.hsharded_step(xh4, w, gl, ops=ops)
        assert torch.equal(y_s, y) and to.rel_l2(dw_s, dw) <= 1e-6
        torch.save({'hb': hb, 'he': he, 'y': y.contiguous(), 'dw': dw, 'ys': ys.contiguous(), 'dws': dws,
                    'halo_lo': xh[:, :, 0].clone(), 'halo_hi': xh[:, :, -1].clone()},
                   os.path.join(out_dir, f'rank{rank}.pt'))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('shape,world', [((2, 8, 7, 5, 6), 2), ((1, 16, 5, 4, 9), 2), ((2, 8, 9, 3, 4), 3)])
def test_sharded_paths_match_single_device(tmp_path, shape, world):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, shape, str(tmp_path)), nprocs=world, join=True)
    N, C, H, W, D = shape
    x, grad, w = _full_volume(123, N, C, H, W, D)
    y_full = to.fprop_shift_fp32(x, w)
    dw_full = to.wgrad_fp64(x, grad).float()
    covered = 0
    for r in range(world):
        res = torch.load(os.path.join(str(tmp_path), f'rank{r}.pt'))
        hb, he = res['hb'], res['he']
        assert (hb, he) == kd.shard_planes(H, world, r)
        covered += he - hb
        # halo planes: the neighbours' boundary planes, zero at the ends of the volume
        lo_ref = x[:, :, hb - 1] if hb > 0 else torch.zeros_like(x[:, :, 0])
        hi_ref = x[:, :, he] if he < H else torch.zeros_like(x[:, :, 0])
        assert torch.equal(res['halo_lo'], lo_ref) and torch.equal(res['halo_hi'], hi_ref)
        assert torch.equal(res['y'], y_full[:, :, hb:he])
        assert to.rel_l2(res['dw'], dw_full) <= 1e-5
        # sample sharding
        assert torch.equal(res['ys'], y_full[r::world])
        assert to.rel_l2(res['dws'], dw_full) <= 1e-5
    assert covered == H


def _worker_empty_shard(rank, world, port):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        hb, he = kd.shard_planes(1, world, rank)  # H = 1 < world: rank 1 owns no plane
        xh = kd.alloc_halo_volume(1, 8, he - hb, 3, 4, 'cpu')
        if he - hb == 0:
            with pytest.raises(AssertionError, match='at least one owned plane'):
                kd.exchange_halo(xh)
            with pytest.raises(AssertionError, match='at least one owned plane'):
                kd.hsharded_step(xh, torch.zeros(3, 3, 3, 8).half(), xh[:, :, 1:-1], ops=OracleOps())
    finally:
        dist.destroy_process_group()


def test_empty_shard_is_rejected():
    """H < world would hand a rank zero planes; the helpers refuse instead of sending a halo plane as data."""
    mp.spawn(_worker_empty_shard, args=(2, _free_port()), nprocs=2, join=True)


def test_shard_planes_partitions_the_axis():
    for H in (1, 2, 7, 350, 1400):
        for world in (1, 2, 3, 4, 8):
            spans = [kd.shard_planes(H, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == H
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0 and a1 >= a0
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
