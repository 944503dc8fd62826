"""Pins the oracle's Conv2d / MaxPool2d restatement against what tests/test_cnn.mojo and the pooling tests of
the reference check: the one forward literal, output shapes under stride / dilation / padding, gradients
against central differences (the reference's own method, tests/test_cnn.mojo:222-322) and the bias-gradient
count (tests/test_cnn.mojo:325-350).  CPU only."""
import numpy as np
import pytest


def test_basic_forward_literal(oracle):
    # tests/test_cnn.mojo:24-48
    img = np.zeros((1, 1, 3, 3), np.float32)
    img[0, 0, 0, 0], img[0, 0, 0, 1], img[0, 0, 1, 0], img[0, 0, 1, 1] = 1, 2, 3, 4
    ker = np.array([[[[1, 0], [0, 1]]]], np.float32)
    out = oracle.conv2d_fwd(img, ker, None)
    assert out.shape == (1, 1, 2, 2) and out[0, 0, 0, 0] == 5.0 and out[0, 0, 0, 1] == 2.0


def test_shapes_stride_dilation_padding(oracle):
    # tests/test_cnn.mojo:51-146
    img = np.arange(16, dtype=np.float32).reshape(1, 1, 4, 4)
    ones = np.ones((1, 1, 2, 2), np.float32)
    assert oracle.conv2d_fwd(img, ones, None, stride=1).shape[2:] == (3, 3)
    r2 = oracle.conv2d_fwd(img, ones, None, stride=2)
    assert r2.shape[2:] == (2, 2) and r2[0, 0, 0, 0] == 0 + 1 + 4 + 5 and r2[0, 0, 1, 1] == 10 + 11 + 14 + 15
    img5 = np.arange(25, dtype=np.float32).reshape(1, 1, 5, 5)
    rd = oracle.conv2d_fwd(img5, ones, None, dilation=2)
    assert rd.shape[2:] == (3, 3) and rd[0, 0, 0, 0] == 0 + 2 + 10 + 12
    k3 = np.ones((1, 1, 3, 3), np.float32)
    same = oracle.conv2d_fwd(img5, k3, None, pad=1)
    assert same.shape[2:] == (5, 5) and same[0, 0, 0, 0] == 0 + 1 + 5 + 6


def test_matches_direct_definition_and_gradients(oracle):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, 3, 7, 6)).astype(np.float32)
    k = rng.standard_normal((4, 3, 3, 2)).astype(np.float32)
    b = rng.standard_normal(4).astype(np.float32)
    for stride, dil, pad in ((1, 1, 0), (2, 1, 1), (1, 2, 2)):
        out = oracle.conv2d_fwd(x, k, b, stride=stride, dilation=dil, pad=pad)
        xp = np.pad(x, ((0, 0), (0, 0), (pad, pad), (pad, pad))).astype(np.float64)
        ref = np.zeros(out.shape)
        for co in range(4):
            for oy in range(out.shape[2]):
                for ox in range(out.shape[3]):
                    win = xp[:, :, oy * stride:oy * stride + (3 - 1) * dil + 1:dil, ox * stride:ox * stride + (2 - 1) * dil + 1:dil]
                    ref[:, co, oy, ox] = (win * k[co].astype(np.float64)).sum(axis=(1, 2, 3)) + b[co]
        assert np.allclose(out, ref, rtol=1e-5, atol=1e-5)
        g = rng.standard_normal(out.shape).astype(np.float32)
        dx, dk, db = oracle.conv2d_bwd(g, x, k, stride=stride, dilation=dil, pad=pad)
        assert np.allclose(db, g.sum(axis=(0, 2, 3)), rtol=1e-5, atol=1e-5)
        # central differences on a few coordinates of x and k, loss = sum(out * g)
        f = lambda xx, kk: float((oracle.conv2d_fwd(xx, kk, b, stride=stride, dilation=dil, pad=pad).astype(np.float64) * g).sum())
        eps = 1e-2
        for idx in [(0, 0, 0, 0), (1, 2, 3, 4), (0, 1, 6, 5)]:
            xp_, xm_ = x.copy(), x.copy()
            xp_[idx] += eps
            xm_[idx] -= eps
            assert abs((f(xp_, k) - f(xm_, k)) / (2 * eps) - dx[idx]) < 2e-2
        for idx in [(0, 0, 0, 0), (3, 2, 2, 1)]:
            kp_, km_ = k.copy(), k.copy()
            kp_[idx] += eps
            km_[idx] -= eps
            assert abs((f(x, kp_) - f(x, km_)) / (2 * eps) - dk[idx]) < 5e-2


def test_bias_gradient_counts_positions(oracle):
    # tests/test_cnn.mojo:325-350: ones everywhere, grad of sum = N * Ho * Wo per channel
    x, k = np.ones((2, 1, 3, 3), np.float32), np.ones((2, 1, 2, 2), np.float32)
    out = oracle.conv2d_fwd(x, k, np.zeros(2, np.float32))
    _, _, db = oracle.conv2d_bwd(np.ones_like(out), x, k)
    assert np.array_equal(db, np.full(2, 2 * 2 * 2, np.float32))


def test_maxpool_first_max_wins_and_backward(oracle):
    x = np.array([[[[1, 1, 2, 0], [1, 1, 0, 2], [5, 3, 7, 7], [3, 5, 7, 7]]]], np.float32)
    out, arg = oracle.maxpool2d_fwd(x)
    assert np.array_equal(out[0, 0], [[1, 2], [5, 7]])
    assert np.array_equal(arg[0, 0], [[0, 2], [8, 10]])  # ties: the first position in row-major window order
    dx = oracle.maxpool2d_bwd(np.array([[[[10, 20], [30, 40]]]], np.float32), arg, x.shape)
    want = np.zeros((4, 4), np.float32)
    want[0, 0], want[0, 2], want[2, 0], want[2, 2] = 10, 20, 30, 40
    assert np.array_equal(dx[0, 0], want)
    # padded window: positions outside the image are skipped
    o2, a2 = oracle.maxpool2d_fwd(-np.ones((1, 1, 3, 3), np.float32), k=2, stride=2, pad=1)
    assert o2.shape == (1, 1, 2, 2) and np.all(o2 == -1) and a2[0, 0, 0, 0] == 0
