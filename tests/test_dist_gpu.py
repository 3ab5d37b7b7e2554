"""The multi-GPU layer on real GPUs (needs >= 2): NCCL ranks as child processes, results compared with the
single-device kernels.  NVLS is switched off for these short-lived ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank, world, port, shape, out_dir):
    try:
        _worker_body(rank, world, port, shape, out_dir)
    except BaseException:
        # leave at once, without the process-group teardown: the other ranks may be inside a collective this rank
        # will never join, and the parent ends them as soon as it sees this exit code
        import traceback

        traceback.print_exc()
        os._exit(1)


def _worker_body(rank, world, port, shape, out_dir):
    import datetime

    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=60))
    try:
        from kerops_b200 import _lib
        from kerops_b200 import dist as kd
        from kerops_b200.ops.conv import _launch

        N, C, H, W, D = shape
        g = torch.Generator(device=dev).manual_seed(77)  # the same volume on every rank
        x = torch.randn(N, H, W, D, C, generator=g, device=dev, dtype=torch.float16).permute(0, 4, 1, 2, 3)
        grad = torch.randn(N, H, W, D, C, generator=g, device=dev, dtype=torch.float16).permute(0, 4, 1, 2, 3)
        w = ((torch.rand(3, 3, 3, C, generator=g, device=dev) * 2 - 1) / 27 ** 0.5).half()
        y_full = torch.empty_like(x)
        _launch.fprop(x, w, y_full)
        dw_full, _ = _launch.wgrad(x, grad, want_f32=True, want_f16=False)

        hb, he = kd.shard_planes(H, world, rank)
        xh = kd.alloc_halo_volume(N, C, he - hb, W, D, dev)
        xh[:, :, 1:-1] = x[:, :, hb:he]
        y = kd.hsharded_fprop(xh, w)
        gl = grad[:, :, hb:he].contiguous(memory_format=torch.channels_last_3d)
        dw = kd.hsharded_wgrad(xh, gl)
        ys, dws = kd.sample_sharded_step(x[rank::world].contiguous(memory_format=torch.channels_last_3d), w,
                                         grad[rank::world].contiguous(memory_format=torch.channels_last_3d))
        # the library's own all-reduce over peer memory against NCCL's
        red = kd.GradPushAllReduce(27 * C, timeout_s=5.0)
        gl_ = torch.Generator(device=dev).manual_seed(1234 + rank)
        push_equal, push_err = True, 0.0
        for it in range(6):
            local = torch.randn(27 * C, generator=gl_, device=dev)
            ref = local.clone()
            dist.all_reduce(ref)
            got = red(local)
            push_err = max(push_err, float((got - ref).abs().max() / ref.abs().max()))
            push_equal = push_equal and bool(torch.equal(got, ref))
        _, dws_push = kd.sample_sharded_step(x[rank::world].contiguous(memory_format=torch.channels_last_3d), w,
                                             grad[rank::world].contiguous(memory_format=torch.channels_last_3d),
                                             reducer=red)
        torch.cuda.synchronize()
        ok = {
            'push_err': push_err,
            'push_equal': push_equal,
            'dp_wgrad_push': float((dws_push.double() - dw_full.double()).norm() / dw_full.double().norm()),
            'fprop': bool(torch.equal(y, y_full[:, :, hb:he])),
            'wgrad': float((dw.double() - dw_full.double()).norm() / dw_full.double().norm()),
            'dp_fprop': bool(torch.equal(ys, y_full[rank::world])),
            'dp_wgrad': float((dws.double() - dw_full.double()).norm() / dw_full.double().norm()),
            'status': _lib.device_status(),
        }
        torch.save(ok, os.path.join(out_dir, f'rank{rank}.pt'))
        dist.barrier()
    finally:
        pass
    dist.destroy_process_group()


@pytest.mark.parametrize('shape', [(2, 32, 37, 21, 40), (2, 128, 11, 9, 33)])
def test_sharded_paths_on_gpus(tmp_path, shape):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip('needs at least two GPUs')
    mp.spawn(_worker, args=(world, _free_port(), shape, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(os.path.join(str(tmp_path), f'rank{r}.pt'))
        assert res['fprop'] and res['dp_fprop'], res
        assert res['wgrad'] <= 1e-5 and res['dp_wgrad'] <= 1e-5, res
        assert res['push_err'] <= 1e-6 and res['dp_wgrad_push'] <= 1e-5, res
        if world == 2:
            assert res['push_equal'], res  # two addends: any order gives the same bits
        assert res['status'] == 0
