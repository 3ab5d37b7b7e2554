"""torch restatement of the oracle formulas, device-agnostic (CPU or CUDA).

TEST INFRASTRUCTURE ONLY (see dwconv_oracle.py).  Used where the numpy oracle would take too long:
full-size parity checks on the GPU box and the timed CPU baseline of the benchmark.

fprop_conv3d  is the check the reference's own test applies (tests/ops/test_conv.py:25:
              F.conv3d(x, weight, None, padding=1, stride=1, groups=C)), evaluated in fp32 and
              rounded once to fp16.
wgrad_fp64    is the 27-shift definition of the weight gradient in fp64, chunked along dim 2 so it
              fits next to a multi-GB input.
"""
import torch
import torch.nn.functional as F


def to_torch_weight(weight_ker):
    """[3,3,3,C] kerops layout -> [C,1,3,3,3] torch layout (inverse of tests/ops/test_conv.py:23)."""
    return weight_ker.permute(3, 0, 1, 2)[:, None].contiguous()


def fprop_conv3d(x, weight_ker, dtype=torch.float32):
    C = x.shape[1]
    y = F.conv3d(x.to(dtype), to_torch_weight(weight_ker).to(dtype), None, stride=1, padding=1, groups=C)
    return y.to(torch.float16)


def wgrad_fp64(x, grad, chunk=8):
    """dw[a,b,t,c] in fp64; x, grad are (N, C, H, W, D) tensors of any memory format."""
    N, C, H, W, D = x.shape
    dw = torch.zeros(3, 3, 3, C, dtype=torch.float64, device=x.device)
    for h0 in range(0, H, chunk):
        h1 = min(H, h0 + chunk)
        lo, hi = max(0, h0 - 1), min(H, h1 + 1)
        # padded x slab covering planes h0-1 .. h1 (zeros outside the volume)
        xs = x[:, :, lo:hi].to(torch.float64)
        xs = F.pad(xs, (1, 1, 1, 1, 1 if h0 == 0 else 0, 1 if h1 == H else 0))
        g = grad[:, :, h0:h1].to(torch.float64)
        n = h1 - h0
        for a in range(3):
            for b in range(3):
                for t in range(3):
                    dw[a, b, t] += (g * xs[:, :, a:a + n, b:b + W, t:t + D]).sum(dim=(0, 2, 3, 4))
    return dw


def rel_l2(a, b):
    a = a.to(torch.float64)
    b = b.to(torch.float64)
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def fprop_shift_fp32(x, weight_ker, chunk=16):
    """27 shifted fp32 multiply-adds (no library convolution, so no TF32 or algorithm choice can
    interfere); rounds once to fp16.  x is (N, C, H, W, D) in any memory format; the result is
    channels_last_3d."""
    N, C, H, W, D = x.shape
    xl = x.permute(0, 2, 3, 4, 1)  # N H W D C view
    w = weight_ker.to(torch.float32)
    y = torch.empty((N, H, W, D, C), dtype=torch.float16, device=x.device)
    for h0 in range(0, H, chunk):
        h1 = min(H, h0 + chunk)
        lo, hi = max(0, h0 - 1), min(H, h1 + 1)
        xs = F.pad(xl[:, lo:hi].to(torch.float32), (0, 0, 1, 1, 1, 1, 1 if h0 == 0 else 0, 1 if h1 == H else 0))
        n = h1 - h0
        acc = torch.zeros((N, n, W, D, C), dtype=torch.float32, device=x.device)
        for a in range(3):
            for b in range(3):
                for t in range(3):
                    acc.addcmul_(xs[:, a:a + n, b:b + W, t:t + D], w[a, b, t])
        y[:, h0:h1] = acc.to(torch.float16)
    return y.permute(0, 4, 1, 2, 3)
