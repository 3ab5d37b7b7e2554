"""CPU oracle for the depthwise 3x3x3 channels-last convolution path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module;
it is used by tests/, by the smoke check and by the CPU-baseline leg of the
benchmark as the checker, never as the thing that is measured or shipped.

Arrays are numpy, in the PHYSICAL order of a channels_last_3d tensor:
``x[n, h, w, d, c]`` (kerops names the three spatial axes H, W, D =
torch dims 2, 3, 4; d is the innermost spatial axis) and ``weight[a, b, t, c]``
with a, b, t the taps along h, w, d (kerops layout, tests/ops/test_conv.py:23).

Functions
---------
fprop_exact              y = sum_{a,b,t} x[h+a-1, w+b-1, d+t-1, c] * w[a,b,t,c] in fp32/fp64,
                         rounded once to fp16.  Same arithmetic as the check the reference's
                         test uses (conv3d with groups=C, tests/ops/test_conv.py:25), evaluated
                         in higher precision.
fprop_reference_numerics restates the arithmetic order of kerops/kernels/dw_conv.py:49-121:
                         fp16 products, the three d-taps summed in fp16, the nine (a, b)
                         partials accumulated in fp32 in the order b outer / a inner, one final
                         cast to fp16.
wgrad_exact              dw[a,b,t,c] = sum_{n,h,w,d} g[n,h,w,d,c] * x[n,h+a-1,w+b-1,d+t-1,c]
                         in fp64 (kerops/kernels/dw_conv.py:224-275 computes the same sum from
                         fp16 products with fp32/fp16 partials).
addstats_exact           out = conv_out + residual (fp16 add) with the fp64 channel mean and mean of squares
                         of out, the arithmetic of kerops/kernels/addition.py:28-37.
bnrelu_exact             fp16(max(fma(x, scale[c], shift[c]), 0)), the arithmetic of kerops/kernels/bnrelu.py:25-31.

Pinning: tests/test_oracle_golden.py checks these functions against vectors
produced by the reference kernels themselves (tests/golden/*.npz, made by
tests/golden/make_golden.py from the reference sources under Triton's CPU
interpreter): fprop_reference_numerics reproduces the reference output bit for
bit, fprop_exact within the reference test's two-stage tolerance, wgrad_exact
within the reference's cosine/norm tolerance and 1e-3 relative L2.
"""
import numpy as np


def _pad_spatial(x):
    # zero padding of 1 on h, w, d (padding=1 in kerops/ops/conv/dwconv.py via masks,
    # kerops/kernels/dw_conv.py:32-34,60-67)
    return np.pad(x, ((0, 0), (1, 1), (1, 1), (1, 1), (0, 0)))


def fprop_exact(x, weight, acc_dtype=np.float32):
    """fp16 in, high-precision accumulate, one rounding to fp16 (kerops/ops/conv/dwconv.py:25-63)."""
    assert x.ndim == 5 and weight.shape == (3, 3, 3, x.shape[-1])
    N, H, W, D, C = x.shape
    xp = _pad_spatial(x.astype(acc_dtype))
    w = weight.astype(acc_dtype)
    y = np.zeros((N, H, W, D, C), dtype=acc_dtype)
    for a in range(3):
        for b in range(3):
            for t in range(3):
                y += xp[:, a:a + H, b:b + W, t:t + D, :] * w[a, b, t]
    return y.astype(np.float16)


def fprop_reference_numerics(x, weight):
    """Restates the rounding sequence of kerops/kernels/dw_conv.py:49-121.

    x * weight is an fp16 product (:71 ff.), tl.sum over the 4-lane tap axis is an fp16 sum of
    (p0, p1, p2, 0) -> (p0 + p1) + p2, the result is added to an fp32 accumulator (:49-52), and
    the 16-step loop visits columns with the w-offset outer and the h-offset inner (:124-125),
    so every output accumulates its nine partials in the order b = 0..2 (outer), a = 0..2 (inner).
    """
    assert x.dtype == np.float16 and weight.dtype == np.float16
    N, H, W, D, C = x.shape
    xp = _pad_spatial(x)
    acc = np.zeros((N, H, W, D, C), dtype=np.float32)
    for b in range(3):
        for a in range(3):
            p0 = xp[:, a:a + H, b:b + W, 0:D, :] * weight[a, b, 0]
            p1 = xp[:, a:a + H, b:b + W, 1:1 + D, :] * weight[a, b, 1]
            p2 = xp[:, a:a + H, b:b + W, 2:2 + D, :] * weight[a, b, 2]
            part = ((p0 + p1).astype(np.float16) + p2).astype(np.float16)
            acc += part.astype(np.float32)
    return acc.astype(np.float16)


def wgrad_exact(x, grad, acc_dtype=np.float64):
    """fp64 weight gradient, shape [3,3,3,C] (kerops/ops/conv/dwconv_wgrad.py:31-79)."""
    assert x.shape == grad.shape and x.ndim == 5
    N, H, W, D, C = x.shape
    xp = _pad_spatial(x.astype(acc_dtype))
    g = grad.astype(acc_dtype)
    dw = np.zeros((3, 3, 3, C), dtype=acc_dtype)
    for a in range(3):
        for b in range(3):
            for t in range(3):
                dw[a, b, t] = np.einsum('nhwdc,nhwdc->c', g, xp[:, a:a + H, b:b + W, t:t + D, :])
    return dw


def dgrad_exact(grad, weight, acc_dtype=np.float32):
    """Input gradient = fprop of grad with the taps flipped on all three axes."""
    return fprop_exact(grad, weight[::-1, ::-1, ::-1].copy(), acc_dtype)


def addstats_exact(conv_out, residual):
    """out = conv_out + residual as an fp16 add, and the per-channel mean and mean of squares of out in fp64
    (kerops/kernels/addition.py:28-37: output = x + y, mean = sum(output) / numel_no_channels, sqmean likewise)."""
    assert conv_out.dtype == np.float16 and residual.dtype == np.float16 and conv_out.shape == residual.shape
    out = (conv_out.astype(np.float32) + residual.astype(np.float32)).astype(np.float16)  # exact sum, one rounding
    o = out.astype(np.float64).reshape(-1, out.shape[-1])
    return out, o.mean(axis=0), (o * o).mean(axis=0)


def bnrelu_exact(x, scale, shift):
    """fp16(max(x * scale[c] + shift[c], 0)) with the multiply-add in fp32 as one fused operation
    (kerops/kernels/bnrelu.py:25-31; evaluated in fp64 and rounded to fp32: an fp16 x fp32 product fits a double
    exactly, so only the rare double rounding of the sum can differ from a hardware FMA)."""
    assert x.dtype == np.float16
    f = (x.astype(np.float64) * scale.astype(np.float32).astype(np.float64)
         + shift.astype(np.float32).astype(np.float64)).astype(np.float32)
    return np.maximum(f, np.float32(0)).astype(np.float16)


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


# ---------------------------------------------------------------------------------------------
# Tolerances of the reference test-suite, restated for numpy (kerops/utils.py:5-102).
# ---------------------------------------------------------------------------------------------
def allclose_two_stage(inp, other, rtol_strict=1e-4, atol_strict=1e-4, percentile_strict=0.99,
                       rtol_narrow=1e-3, atol_narrow=1e-3):
    """>= percentile_strict of the elements within the strict bound, all the others within the
    narrow bound (kerops/utils.py:35-69; note the strict '>' at :55)."""
    a = np.asarray(inp, dtype=np.float64).reshape(-1)
    b = np.asarray(other, dtype=np.float64).reshape(-1)
    strict = np.abs(a - b) < atol_strict + rtol_strict * np.abs(b)
    n_true = int(strict.sum())
    if n_true == a.size:
        return True
    if n_true / a.size > percentile_strict:
        a2, b2 = a[~strict], b[~strict]
        return bool((np.abs(a2 - b2) < atol_narrow + rtol_narrow * np.abs(b2)).all())
    return False


def weight_grad_similarity(inp, other, rtol_cos=1e-4, atol_cos=1e-4, rtol_len=1e-3, atol_len=1e-3):
    """cosine(inp, other) ~ 1 and |inp| ~ |other| (kerops/utils.py:72-102)."""
    a = np.asarray(inp, dtype=np.float64).reshape(-1)
    b = np.asarray(other, dtype=np.float64).reshape(-1)
    na, nb = np.linalg.norm(a), np.linalg.norm(b)
    cos = float(a @ b / max(na * nb, 1e-8))
    if not abs(1.0 - cos) <= atol_cos + rtol_cos * abs(cos):
        return False
    return bool(abs(na - nb) <= atol_len + rtol_len * abs(nb))
