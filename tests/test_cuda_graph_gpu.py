"""The operators only enqueue work on the current stream (no synchronisation, no allocation on the C side), so a
forward + weight-gradient step can be captured into a CUDA graph and replayed on new data in the same buffers."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_forward_and_weight_gradient_replay_from_a_cuda_graph():
    from kerops_b200 import _lib
    from kerops_b200.ops.conv import DWConv, DWConvWGRAD, _launch

    C, H, W, D = 32, 24, 40, 64
    g = torch.Generator(device='cuda').manual_seed(3)
    x = torch.randn(2, H, W, D, C, generator=g, device='cuda', dtype=torch.float16).permute(0, 4, 1, 2, 3)
    grad = torch.randn(2, H, W, D, C, generator=g, device='cuda', dtype=torch.float16).permute(0, 4, 1, 2, 3)
    w = ((torch.rand(3, 3, 3, C, generator=g, device='cuda') * 2 - 1) / math.sqrt(27)).half()
    y = torch.empty_like(x)
    ws = _launch.wgrad_workspace(x)
    dw32 = torch.empty(27 * C, dtype=torch.float32, device='cuda')

    def step():
        _launch.fprop(x, w, y)
        _launch.wgrad(x, grad, want_f16=False, workspace=ws, out_f32=dw32)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up outside the capture: module load, function attributes
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for seed in (10, 11):  # new contents, same buffers
        g2 = torch.Generator(device='cuda').manual_seed(seed)
        x.copy_(torch.randn(2, H, W, D, C, generator=g2, device='cuda', dtype=torch.float16).permute(0, 4, 1, 2, 3))
        grad.copy_(torch.randn(2, H, W, D, C, generator=g2, device='cuda', dtype=torch.float16).permute(0, 4, 1, 2, 3))
        y.fill_(float('nan'))
        dw32.fill_(float('nan'))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, DWConv(x, w))
        ref32, _ = _launch.wgrad(x, grad, want_f32=True, want_f16=False)
        assert torch.equal(dw32.view(3, 3, 3, C), ref32)
    assert _lib.device_status() == 0
