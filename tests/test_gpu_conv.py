"""Conv2d as an implicit GEMM, MaxPool2d and the CIFAR-shaped CNN step ((256,3,32,32) images, two 3x3 convolutions with
ReLU and 2x2 max pooling, Linear 4096 -> 10) against the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def g():
    from tests import gpu_util

    gpu_util.handle()
    return gpu_util


GEOMS = [  # N, Cin, H, W, Cout, k, stride, dilation, pad
    (2, 3, 8, 8, 5, 3, 1, 1, 1),
    (3, 4, 9, 7, 6, 2, 2, 1, 0),      # gather kernels: 2x2 kernel, stride 2
    (2, 2, 11, 10, 3, 3, 1, 2, 2),    # gather kernels: dilation 2
    (2, 5, 13, 19, 7, 3, 2, 1, 1),    # gather kernels: 3x3 with stride 2
    (4, 3, 32, 32, 32, 3, 1, 1, 1),   # conv1 of the CNN
    (2, 32, 16, 16, 64, 3, 1, 1, 1),  # conv2 of the CNN
    (3, 40, 19, 21, 70, 3, 1, 1, 0),  # staged kernels with ragged tiles, two input-channel chunks, three channel blocks, no padding
    (5, 9, 35, 33, 33, 3, 1, 1, 2),   # staged kernels, padding 2, image larger than one tile in both directions
]


@pytest.mark.parametrize("geom", GEOMS, ids=str)
def test_conv2d_forward_backward_vs_oracle(g, oracle, geom):
    from tenmo_b200.cnn import Conv2d

    N, Cin, H, W, Cout, k, stride, dil, pad = geom
    rng = np.random.default_rng(sum(geom))
    x = rng.standard_normal((N, Cin, H, W)).astype(np.float32)
    w = (rng.standard_normal((Cout, Cin, k, k)) * 0.2).astype(np.float32)
    b = rng.standard_normal(Cout).astype(np.float32)
    h = g.handle()
    conv = Conv2d(h, N, Cin, H, W, Cout, k, stride, dil, pad, relu=False)
    xd, wd, bd = g.dev(x), g.dev(w), g.dev(b)
    out = g.host(conv.forward(xd, wd, bd))
    ref = oracle.conv2d_fwd(x, w, b, stride=stride, dilation=dil, pad=pad, contract=1)
    # the strict-fp32 GEMM starts its accumulators at the bias and runs the same (c, ky, kx) fma chain
    assert np.array_equal(out, ref)
    gr = rng.standard_normal(ref.shape).astype(np.float32)
    dW, db = g.empty(Cout, Cin, k, k), g.empty(Cout)
    dx = conv.backward(g.dev(gr), wd, dW, db)
    rdx, rdw, rdb = oracle.conv2d_bwd(gr, x, w, stride=stride, dilation=dil, pad=pad)
    tol = dict(rtol=1e-4, atol=1e-4)  # same sums in a different order
    assert np.allclose(g.host(db), rdb, **tol)
    assert np.allclose(g.host(dW), rdw, **tol)
    assert np.allclose(g.host(dx), rdx, **tol)
    # the same layer with ReLU: output and 0/1 mask from the epilogue, the mask multiplied into g by the backward kernels
    convr = Conv2d(h, N, Cin, H, W, Cout, k, stride, dil, pad, relu=True)
    outr = g.host(convr.forward(xd, wd, bd))
    r_out, r_mask = oracle.relu_fwd(ref)
    assert np.array_equal(outr, r_out) and np.array_equal(g.host(convr.mask), r_mask)
    dxr = convr.backward(g.dev(gr), wd, dW, db)
    rdx, rdw, rdb = oracle.conv2d_bwd(oracle.relu_bwd(gr, r_mask), x, w, stride=stride, dilation=dil, pad=pad)
    assert np.allclose(g.host(db), rdb, **tol) and np.allclose(g.host(dW), rdw, **tol) and np.allclose(g.host(dxr), rdx, **tol)
    # run to run the gradients are the same bits (slab order, not arrival order)
    dW2, db2 = g.empty(Cout, Cin, k, k), g.empty(Cout)
    convr.backward(g.dev(gr), wd, dW2, db2)
    assert torch.equal(dW, dW2) and torch.equal(db, db2)
    h.check_device_status()


def test_im2col_matches_the_padded_image(g):
    N, Cin, H, W, k, stride, dil, pad = 2, 3, 9, 8, 3, 2, 1, 1
    rng = np.random.default_rng(12)
    x = rng.standard_normal((N, Cin, H, W)).astype(np.float32)
    Ho, Wo = (H + 2 * pad - 3) // stride + 1, (W + 2 * pad - 3) // stride + 1
    pat = g.empty(N * Ho * Wo, Cin * k * k)
    g.handle().im2col(g.dev(x).data_ptr(), N, Cin, H, W, k, k, stride, dil, pad, pat.data_ptr())
    patches = g.host(pat).reshape(N, Ho, Wo, Cin, k, k)
    xp = np.pad(x, ((0, 0), (0, 0), (pad, pad), (pad, pad)))
    for oy, ox in ((0, 0), (Ho - 1, Wo // 2), (Ho - 1, Wo - 1)):
        assert np.array_equal(patches[:, oy, ox], xp[:, :, oy * stride:oy * stride + (k - 1) * dil + 1:dil,
                                                     ox * stride:ox * stride + (k - 1) * dil + 1:dil])


@pytest.mark.parametrize("shape_k", [((2, 3, 8, 8), 2, 2, 0), ((3, 5, 9, 7), 3, 2, 1), ((256, 32, 32, 32), 2, 2, 0)], ids=str)
def test_maxpool_vs_oracle(g, oracle, shape_k):
    from tenmo_b200.cnn import MaxPool2d

    shape, k, stride, pad = shape_k
    rng = np.random.default_rng(k + shape[0])
    x = np.round(rng.standard_normal(shape), 1).astype(np.float32)  # rounded: ties inside windows
    pool = MaxPool2d(g.handle(), *shape, k=k, stride=stride, pad=pad)
    out = g.host(pool.forward(g.dev(x)))
    rout, rarg = oracle.maxpool2d_fwd(x, k, stride, pad)
    assert np.array_equal(out, rout) and np.array_equal(g.host(pool.argmax), rarg)
    gr = rng.standard_normal(rout.shape).astype(np.float32)
    dx = g.host(pool.backward(g.dev(gr)))
    rdx = oracle.maxpool2d_bwd(gr, rarg, shape)
    if stride >= k:
        assert np.array_equal(dx, rdx)      # disjoint windows: one writer per element
    else:
        assert np.allclose(dx, rdx, rtol=1e-6, atol=1e-6)


def test_channel_sum_and_col2im_adjoint(g, oracle):
    h = g.handle()
    rng = np.random.default_rng(4)
    gr = rng.standard_normal((7, 5, 33)).astype(np.float32)
    out = g.empty(5)
    h.channel_sum(g.dev(gr).data_ptr(), 7, 5, 33, out.data_ptr())
    assert np.allclose(g.host(out), gr.sum(axis=(0, 2)), rtol=1e-5, atol=1e-5)
    # <im2col(x), P> == <x, col2im(P)>  for any x, P
    N, C, H, W, k, stride, dil, pad = 2, 3, 9, 8, 3, 2, 1, 1
    Ho, Wo = (H + 2 * pad - 3) // stride + 1, (W + 2 * pad - 3) // stride + 1
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    P = rng.standard_normal((N * Ho * Wo, C * k * k)).astype(np.float32)
    pat, back = g.empty(N * Ho * Wo, C * k * k), g.empty(N, C, H, W)
    h.im2col(g.dev(x).data_ptr(), N, C, H, W, k, k, stride, dil, pad, pat.data_ptr())
    h.col2im(g.dev(P).data_ptr(), N, C, H, W, k, k, stride, dil, pad, back.data_ptr())
    lhs = float((g.host(pat).astype(np.float64) * P).sum())
    rhs = float((x.astype(np.float64) * g.host(back)).sum())
    assert abs(lhs - rhs) <= 1e-4 * max(1.0, abs(lhs))


def _cnn_params(rng, hw=32):
    he = lambda shape, fan_in: (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)
    feat = 64 * (hw // 4) ** 2
    return {"conv1.weight": he((32, 3, 3, 3), 27), "conv1.bias": np.zeros(32, np.float32),
            "conv2.weight": he((64, 32, 3, 3), 288), "conv2.bias": np.zeros(64, np.float32),
            "fc.weight": he((feat, 10), feat), "fc.bias": np.zeros(10, np.float32)}


def _oracle_cnn_step(oracle, p, X, y):
    """The same network composed from oracle ops; returns (loss, logits, grads)."""
    z1 = oracle.conv2d_fwd(X, p["conv1.weight"], p["conv1.bias"], pad=1)
    a1, m1 = oracle.relu_fwd(z1)
    q1, arg1 = oracle.maxpool2d_fwd(a1)
    z2 = oracle.conv2d_fwd(q1, p["conv2.weight"], p["conv2.bias"], pad=1)
    a2, m2 = oracle.relu_fwd(z2)
    q2, arg2 = oracle.maxpool2d_fwd(a2)
    B = X.shape[0]
    flat = q2.reshape(B, -1)
    logits = oracle.add_bias(oracle.matmul(flat, p["fc.weight"], threads=4), p["fc.bias"])
    loss, sm, valid = oracle.ce_fwd(logits, y)
    dl = oracle.ce_bwd(sm, y, valid)
    grads = {"fc.weight": oracle.matmul(oracle.View.of(flat).t(), oracle.View.of(dl)), "fc.bias": oracle.colsum(dl)}
    dflat = oracle.matmul(oracle.View.of(dl), oracle.View.of(p["fc.weight"]).t())
    d_a2 = oracle.maxpool2d_bwd(dflat.reshape(q2.shape), arg2, a2.shape)
    d_z2 = oracle.relu_bwd(d_a2, m2)
    d_q1, grads["conv2.weight"], grads["conv2.bias"] = oracle.conv2d_bwd(d_z2, q1, p["conv2.weight"], pad=1)
    d_a1 = oracle.maxpool2d_bwd(d_q1, arg1, a1.shape)
    d_z1 = oracle.relu_bwd(d_a1, m1)
    _, grads["conv1.weight"], grads["conv1.bias"] = oracle.conv2d_bwd(d_z1, X, p["conv1.weight"], pad=1)
    return float(loss), logits, grads


def test_cifar_shaped_cnn_step_matches_oracle(g, oracle):
    from tenmo_b200.cnn import CNNTrainer

    rng = np.random.default_rng(55)
    p = _cnn_params(rng)
    B = 8
    X = rng.uniform(0, 1, (B, 3, 32, 32)).astype(np.float32)
    y = rng.integers(0, 10, B)
    tr = CNNTrainer(p, batch=B, handle=g.handle())
    tr.step(X, y, update=False)
    torch.cuda.synchronize()
    loss, logits, grads = _oracle_cnn_step(oracle, p, X, y)
    got = tr.logits.cpu().numpy()
    assert np.array_equal(got, logits)           # forward is the same fma chains end to end
    assert np.array_equal(np.argmax(got, 1), np.argmax(logits, 1)) and tr.accuracy() == oracle.accuracy(logits, y)
    assert abs(tr.loss_value() - loss) <= 1e-5
    for name, rg in grads.items():
        gg = tr.grads()[name]
        assert np.max(np.abs(gg - rg)) <= 1e-4 * max(np.max(np.abs(rg)), 1e-6), name
    # a few SGD steps lower the loss on a fixed batch
    first = tr.loss_value()
    for _ in range(15):
        tr.step(X, y)
    tr.step(X, y, update=False)
    assert tr.loss_value() < first
    g.handle().check_device_status()


def test_cnn_checkpoint_round_trip_with_the_reference_key_names(g, tmp_path):
    """state_dict uses "<module index>.weight" / ".bias" as the reference's save_checkpoint does for
    Sequential(Conv2D, ReLU, MaxPool2d, Conv2D, ReLU, MaxPool2d, Flatten, Linear) (tests/test_checkpoint.mojo:41-54,
    102-117); a trainer restored from the file continues with the same bits, momentum included."""
    from tenmo_b200.cnn import CNNTrainer

    rng = np.random.default_rng(56)
    B = 8
    X = rng.uniform(0, 1, (B, 3, 32, 32)).astype(np.float32)
    y = rng.integers(0, 10, B)
    a = CNNTrainer(_cnn_params(rng), batch=B, handle=g.handle())
    for _ in range(3):
        a.step(X, y)
    sd = a.state_dict()
    assert sorted(k for k in sd if not k.startswith("__")) == ["0.bias", "0.weight", "3.bias", "3.weight", "7.bias", "7.weight"]
    assert sd["0.weight"].shape == (32, 3, 3, 3) and sd["3.weight"].shape == (64, 32, 3, 3) and sd["7.weight"].shape == (4096, 10)
    np.save(tmp_path / "cnn.npy", sd, allow_pickle=True)
    b = CNNTrainer(_cnn_params(np.random.default_rng(57)), batch=B, handle=g.handle())
    b.load_state_dict(np.load(tmp_path / "cnn.npy", allow_pickle=True).item())
    for tr in (a, b):
        tr.step(X, y)
    torch.cuda.synchronize()
    pa, pb = a.params(), b.params()
    assert all(np.array_equal(pa[n], pb[n]) for n in pa)
    g.handle().check_device_status()
