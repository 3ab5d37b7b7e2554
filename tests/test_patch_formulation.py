"""The patch products the tensor-core kernels are built on, restated in numpy and checked against the oracle.

`kerops_b200/csrc/dwconv_fprop_mma.cu` and `dwconv_wgrad_mma.cu` compute the depthwise 3x3x3 convolution
(kerops/kernels/dw_conv.py:5-142) and its weight gradient (dw_conv.py:146-287) as small dense products over
BLOCKS of 2 x 2 output voxels (w, d) and their 4 x 4 input PATCHES.  These tests pin the algebra of the three forms
the kernels use - which tap sits where in the B matrices, which output plane an accumulator lane belongs to - on
the CPU; the kernels themselves are compared with the same oracle on the GPU (tests/test_parity_gpu.py).
"""
import numpy as np
import pytest

from oracle import dwconv_oracle as o

SHAPES = [(1, 2, 3, 4, 6), (2, 4, 5, 7, 5), (1, 8, 1, 2, 2), (1, 2, 4, 9, 8)]


def _data(shape, seed):
    N, C, H, W, D = shape
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((N, H, W, D, C)).astype(np.float16)  # physical order of channels_last_3d, as the oracle
    g = rng.standard_normal((N, H, W, D, C)).astype(np.float16)
    w = ((rng.random((3, 3, 3, C)) * 2 - 1) / np.sqrt(27)).astype(np.float16)
    return x, g, w


def _patches(plane, nbw, nbd):
    """plane: (W, D, C) -> A[block, slot, c]; slot = 4 * i + j of the 4 x 4 patch whose origin is the block's
    origin minus one voxel; voxels outside the plane read as zero (what the TMA fill delivers)."""
    W, D, C = plane.shape
    pad = np.zeros((2 * nbw + 2, 2 * nbd + 2, C), dtype=np.float64)
    pad[1:W + 1, 1:D + 1] = plane
    A = np.empty((nbw * nbd, 16, C))
    for bw in range(nbw):
        for bd in range(nbd):
            A[bw * nbd + bd] = pad[2 * bw:2 * bw + 4, 2 * bd:2 * bd + 4].reshape(16, C)
    return A


def _blocks(plane, nbw, nbd):
    """plane: (W, D, C) -> G[block, out, c]; out = 2 * oi + oj inside the 2 x 2 block (zero outside the plane)."""
    W, D, C = plane.shape
    pad = np.zeros((2 * nbw, 2 * nbd, C), dtype=np.float64)
    pad[:W, :D] = plane
    G = np.empty((nbw * nbd, 4, C))
    for bw in range(nbw):
        for bd in range(nbd):
            G[bw * nbd + bd] = pad[2 * bw:2 * bw + 2, 2 * bd:2 * bd + 2].reshape(4, C)
    return G


def _unblocks(Dm, W, D, nbw, nbd):
    """inverse of _blocks, clipped to the plane"""
    C = Dm.shape[2]
    pad = np.empty((2 * nbw, 2 * nbd, C))
    for bw in range(nbw):
        for bd in range(nbd):
            pad[2 * bw:2 * bw + 2, 2 * bd:2 * bd + 2] = Dm[bw * nbd + bd].reshape(2, 2, C)
    return pad[:W, :D]


def _tap_matrix(w_a):
    """w_a: (3, 3) taps of one channel and one plane offset a -> B[slot, out]: tap (i - oi, j - oj) where that is
    inside the 3 x 3 window of output (oi, oj), zero elsewhere (27 of the 3 x 64 entries are taps)."""
    B = np.zeros((16, 4))
    for i in range(4):
        for j in range(4):
            for oi in range(2):
                for oj in range(2):
                    b, t = i - oi, j - oj
                    if 0 <= b <= 2 and 0 <= t <= 2:
                        B[4 * i + j, 2 * oi + oj] = w_a[b, t]
    return B


@pytest.mark.parametrize('shape', SHAPES, ids=str)
def test_channel_pair_form(shape):
    """K = 16 slots x 2 channels, N = 4 outputs x 2 channels; B is zero where the two channels differ.
    Input plane p feeds output plane p + 1 - a with the taps of plane offset a."""
    x, _, w = _data(shape, 1)
    N, C, H, W, D = shape
    nbw, nbd = (W + 1) // 2, (D + 1) // 2
    y = np.zeros((N, H, W, D, C))
    for n in range(N):
        for c0 in range(0, C, 2):
            Bs = []
            for a in range(3):
                B = np.zeros((16, 2, 4, 2))  # (slot, cc, out, cc')
                for cc in range(2):
                    B[:, cc, :, cc] = _tap_matrix(w[a, :, :, c0 + cc].astype(np.float64))
                Bs.append(B.reshape(32, 8))
            for p in range(H):
                A = _patches(x[n, p, :, :, c0:c0 + 2], nbw, nbd).reshape(-1, 32)
                for a in range(3):
                    q = p + 1 - a
                    if 0 <= q < H:
                        Dm = (A @ Bs[a]).reshape(-1, 4, 2)
                        y[n, q, :, :, c0:c0 + 2] += _unblocks(Dm, W, D, nbw, nbd)
    ref = o.fprop_exact(x, w, acc_dtype=np.float64).astype(np.float64)
    got = y.astype(np.float16).astype(np.float64)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize('shape', SHAPES, ids=str)
def test_per_channel_two_lane_form(shape):
    """K = the 16 slots of ONE channel, N = 4 outputs x 2 lanes; the lanes of an accumulator are two output
    planes.  At input plane p the lane p % 2 receives the a = 2 taps and is complete (output plane p - 1), the other
    lane receives the a = 1 taps; the finished lane is emitted, cleared and started again with the a = 0 taps
    (output plane p + 1)."""
    x, _, w = _data(shape, 2)
    N, C, H, W, D = shape
    nbw, nbd = (W + 1) // 2, (D + 1) // 2
    y = np.full((N, H, W, D, C), np.nan)
    for n in range(N):
        for c in range(C):
            taps = [_tap_matrix(w[a, :, :, c].astype(np.float64)) for a in range(3)]
            acc = np.zeros((nbw * nbd, 4, 2))  # (block, out, lane)
            for p in range(H + 1):  # one step past the last plane drains the pipeline
                fl = p % 2
                A = (_patches(x[n, p, :, :, c:c + 1], nbw, nbd)[:, :, 0] if p < H
                     else np.zeros((nbw * nbd, 16)))
                B21 = np.zeros((16, 4, 2))
                B21[:, :, fl] = taps[2]
                B21[:, :, 1 - fl] = taps[1]
                acc += (A @ B21.reshape(16, 8)).reshape(-1, 4, 2)
                if p >= 1:
                    y[n, p - 1, :, :, c] = _unblocks(acc[:, :, fl:fl + 1], W, D, nbw, nbd)[:, :, 0]
                acc[:, :, fl] = 0.0
                B0 = np.zeros((16, 4, 2))
                B0[:, :, fl] = taps[0]
                acc += (A @ B0.reshape(16, 8)).reshape(-1, 4, 2)
    assert not np.isnan(y).any()
    ref = o.fprop_exact(x, w, acc_dtype=np.float64).astype(np.float64)
    got = y.astype(np.float16).astype(np.float64)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize('shape', SHAPES, ids=str)
def test_weight_gradient_transposed_form(shape):
    """dW[(slot), (out)] += sum over blocks of X[block, slot] * G[block, out], x plane p against grad plane
    p + 1 - a; the tap (b, t) of plane offset a is the sum of the four entries (slot, out) with slot - out = (b, t)."""
    x, g, _ = _data(shape, 3)
    N, C, H, W, D = shape
    nbw, nbd = (W + 1) // 2, (D + 1) // 2
    dw = np.zeros((3, 3, 3, C))
    for n in range(N):
        for c in range(C):
            for p in range(H):
                X = _patches(x[n, p, :, :, c:c + 1], nbw, nbd)[:, :, 0]
                for a in range(3):
                    q = p + 1 - a
                    if not 0 <= q < H:
                        continue
                    G = _blocks(g[n, q, :, :, c:c + 1], nbw, nbd)[:, :, 0]
                    M = X.T @ G  # (slot, out)
                    for b in range(3):
                        for t in range(3):
                            dw[a, b, t, c] += sum(M[4 * (oi + b) + (oj + t), 2 * oi + oj]
                                                  for oi in range(2) for oj in range(2))
    ref = o.wgrad_exact(x, g)
    assert np.allclose(dw, ref, rtol=1e-12, atol=1e-12)


def test_useful_fraction_of_the_products():
    """The share of useful products quoted for the tensor-pipe work: 27 of 96 per channel and output in the
    channel-pair form (three 32 x 8 products per channel pair), 27 of 64 in the per-channel form (two 16 x 8
    products per channel)."""
    taps = [np.arange(1, 10, dtype=np.float64).reshape(3, 3) + 9 * a for a in range(3)]
    mats = [_tap_matrix(t) for t in taps]
    # every tap appears once per output of the block, nowhere else
    for a, m in enumerate(mats):
        vals, counts = np.unique(m[m != 0], return_counts=True)
        assert np.array_equal(vals, taps[a].ravel()) and (counts == 4).all()
    nonzero = sum(int((m != 0).sum()) for m in mats)
    assert nonzero == 27 * 4
    # channel-pair form: 3 products of (32 x 8) per channel pair and block row
    assert nonzero * 2 / (3 * 32 * 8) == pytest.approx(27 / 96)
    # per-channel form: one (16 x 8) product with two tap sets and one with a single set per channel and block row
    assert nonzero / (2 * 16 * 8) == pytest.approx(27 / 64)
