"""kdw_allreduce_push_f32 on ONE GPU: argument checks, the single-rank case, the wait that runs out, and the
two-rank data path driven one rank after the other (the kernels of two ranks never wait on one another on the
same GPU: the first one's wait is allowed to run out, the second finds the flag already raised)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _push(lib, local, out, bufs, rank, world, seq, timeout_ms, capacity=None):
    ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return lib.kdw_allreduce_push_f32(local.data_ptr(), out.data_ptr(), None, ptrs, local.numel(),
                                      local.numel() if capacity is None else capacity, rank, world, seq,
                                      int(timeout_ms * 1e6), stream)


def _buffers(lib, n, world):
    nbytes = lib.kdw_allreduce_buffer_bytes(n, world)
    assert nbytes >= 2 * world * (n + 32) * 4
    return [torch.zeros(nbytes // 4, dtype=torch.float32, device='cuda') for _ in range(world)]


def test_single_rank_is_a_copy(kdw_lib):
    from kerops_b200 import _lib

    lib = kdw_lib
    n = 27 * 32
    bufs = _buffers(lib, n, 1)
    for seq in (1, 2, 3):
        local = torch.randn(n, device='cuda')
        out = torch.full_like(local, float('nan'))
        assert _push(lib, local, out, bufs, 0, 1, seq, 1000) == 0
        assert torch.equal(out, local)
    assert _lib.device_status() == 0


def test_wait_runs_out_and_sets_status(kdw_lib):
    from kerops_b200 import _lib

    lib = kdw_lib
    n = 27 * 8
    bufs = _buffers(lib, n, 2)
    local = torch.randn(n, device='cuda')
    out = torch.full_like(local, 7.0)
    # rank 0 of 2, and nobody plays rank 1: the flag never comes, the kernel gives up after 20 ms
    assert _push(lib, local, out, bufs, 0, 2, 1, 20) == 0
    assert _lib.device_status() == 3
    assert torch.equal(out, torch.full_like(out, 7.0))  # outputs untouched
    assert _lib.device_status() == 0  # reading cleared it; the context is still usable
    assert torch.equal(local + 0, local)


@pytest.mark.parametrize('n', [27 * 8, 27 * 128, 1000])
def test_two_ranks_one_after_the_other(kdw_lib, n):
    from kerops_b200 import _lib

    lib = kdw_lib
    bufs = _buffers(lib, n, 2)
    for seq in (1, 2, 3, 4):
        a = torch.randn(n, device='cuda')
        b = torch.randn(n, device='cuda')
        out1 = torch.full_like(a, float('nan'))
        out0 = torch.full_like(a, float('nan'))
        # rank 1 pushes and raises its flags; rank 0 has not run yet, so rank 1's own wait runs out (10 ms)
        assert _push(lib, b, out1, bufs, 1, 2, seq, 10) == 0
        assert _lib.device_status() == 3
        # rank 0 finds both flags and sums in rank order
        assert _push(lib, a, out0, bufs, 0, 2, seq, 1000) == 0
        assert _lib.device_status() == 0
        assert torch.equal(out0, a + b)


def test_alternating_sizes_on_one_buffer_set(kdw_lib):
    """One reducer serving layers of different width: calls alternate between n = 27*128 and n = 27*8 on buffers made
    for the larger one.  Slots and flags lie where the CAPACITY puts them, so the small call of step s+1 cannot land
    in the region the large call of step s is still read from."""
    from kerops_b200 import _lib

    lib = kdw_lib
    cap = 27 * 128
    bufs = _buffers(lib, cap, 2)
    for seq in range(1, 9):
        n = cap if seq % 2 else 27 * 8
        a = torch.randn(n, device='cuda')
        b = torch.randn(n, device='cuda')
        out0 = torch.full_like(a, float('nan'))
        out1 = torch.full_like(a, float('nan'))
        assert _push(lib, b, out1, bufs, 1, 2, seq, 10, capacity=cap) == 0  # rank 1 first: its own wait runs out
        assert _lib.device_status() == 3
        assert _push(lib, a, out0, bufs, 0, 2, seq, 1000, capacity=cap) == 0
        assert _lib.device_status() == 0
        assert torch.equal(out0, a + b)
        # rank 1 again with the same sequence number: both flags are up now, its sum has the same bits
        assert _push(lib, b, out1, bufs, 1, 2, seq, 1000, capacity=cap) == 0
        assert _lib.device_status() == 0
        assert torch.equal(out1, out0)
    # n beyond the capacity is refused
    big = torch.randn(cap + 32, device='cuda')
    assert _push(lib, big, torch.empty_like(big), bufs, 0, 2, 9, 10, capacity=cap) == -1


def test_argument_errors(kdw_lib):
    lib = kdw_lib
    n = 64
    bufs = _buffers(lib, n, 2)
    local = torch.randn(n, device='cuda')
    out = torch.empty_like(local)
    assert lib.kdw_allreduce_buffer_bytes(n, 17) == 0
    assert _push(lib, local, out, bufs, 2, 2, 1, 10) == -1  # rank outside the world
    assert _push(lib, local, out, bufs, 0, 2, 0, 10) == -1  # sequence numbers start at 1
    assert b'sequence' in lib.kdw_last_error()
    mis = [bufs[0], bufs[1][1:]]
    assert _push(lib, local, out, mis, 0, 2, 1, 10) == -2
