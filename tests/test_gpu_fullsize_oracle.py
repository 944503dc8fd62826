"""The attention-shaped / broadcast-batched products and the wide MLP at their full benchmark sizes, on both GEMM
kernels, against the CPU oracle.

Every output element of these products is an independent chain over k, and every row of an MLP activation depends on
one input row only, so a sample of batches / rows of the full-size GPU result must equal the oracle's result for just
that sample: bit for bit on the strict-fp32 kernel, within 1e-4 of sum_k |a||b| on the 3xTF32 kernel.  Each stage is
checked with the GPU's own inputs to that stage (teacher forcing), so one stage's rounding is never blamed on the next.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

TC_TOL = 1e-4   # relative to sum_k |a||b| (the bar of the 3xTF32 kernel)


@pytest.fixture(scope="module")
def T():
    import tenmo_b200.tensor as tensor

    tensor.handle()
    yield tensor
    tensor.set_gemm_algo("simt")


def product_matches(got, a_view, b_view, oracle, strict, threads=8):
    """got == oracle(a . b): bitwise for the strict kernel, else within TC_TOL of sum |a||b|."""
    ref = oracle.matmul(a_view, b_view, threads=threads)
    if strict:
        return np.array_equal(got, ref)
    scale = np.abs(a_view.numpy()).astype(np.float64) @ np.abs(b_view.numpy()).astype(np.float64)
    return float(np.max(np.abs(got.astype(np.float64) - ref) / np.maximum(scale, 1e-30))) <= TC_TOL


@pytest.mark.parametrize("algo", ["simt", "3xtf32"])
def test_attention_fullsize_forward_backward_vs_oracle(T, oracle, algo):
    """(384, 512, 64) @ (384, 64, 512)-view, softmax, @ (384, 512, 64); backward from a random upstream gradient."""
    T.set_gemm_algo(algo)
    strict = algo == "simt"
    V_ = oracle.View
    rng = np.random.default_rng(21)
    BH, S, D = 384, 512, 64
    q, k, v = (rng.standard_normal((BH, S, D)).astype(np.float32) * 0.125 for _ in range(3))
    up = rng.standard_normal((BH, S, D)).astype(np.float32)
    Q, K, V = (T.Tensor.from_numpy(a, requires_grad=True) for a in (q, k, v))
    scores = Q.matmul(K.transpose())          # K^T is a stride view: nothing is materialised
    assert T.handle().gemm_last_algo() == (0 if strict else 1)
    P = scores.softmax()
    ctx = P.matmul(V)
    ctx.backward(T.Tensor.from_numpy(up))
    T.handle().check_device_status()
    sc, p, cx = scores.numpy(), P.numpy(), ctx.numpy()
    dq, dk, dv = Q.grad().numpy(), K.grad().numpy(), V.grad().numpy()
    for b in (0, 101, 383):
        assert product_matches(sc[b], V_.of(q[b]), V_.of(k[b]).t(), oracle, strict), f"Q.K^T batch {b}"
        p_ref = oracle.softmax_fwd(sc[b])
        assert np.max(np.abs(p[b] - p_ref)) <= 2e-6 * np.max(p_ref) + 1e-9
        assert product_matches(cx[b], V_.of(p[b]), V_.of(v[b]), oracle, strict), f"P.V batch {b}"
        # backward (matmul.mojo:101-137): dV = P^T . g, dP = g . V^T, dS = softmax backward, dQ = dS . K, dK = dS^T . Q
        assert product_matches(dv[b], V_.of(p[b]).t(), V_.of(up[b]), oracle, strict), f"dV batch {b}"
        dP = oracle.matmul(V_.of(up[b]), V_.of(v[b]).t())
        dS = oracle.softmax_bwd(dP, p[b])
        # dS feeds two more products; on the 3xTF32 path dP itself carries the kernel's rounding, so the bar for
        # dQ / dK is taken against sum |dS||k| with the oracle's dS
        for name, got, a_view, b_view in (("dQ", dq[b], V_.of(dS), V_.of(k[b])), ("dK", dk[b], V_.of(dS).t(), V_.of(q[b]))):
            ref = oracle.matmul(a_view, b_view)
            scale = np.abs(a_view.numpy()).astype(np.float64) @ np.abs(b_view.numpy()).astype(np.float64)
            err = float(np.max(np.abs(got.astype(np.float64) - ref) / np.maximum(scale, 1e-30)))
            assert err <= (2e-5 if strict else 2 * TC_TOL), f"{name} batch {b}: {err}"


@pytest.mark.parametrize("algo", ["simt", "3xtf32"])
def test_broadcast_batched_fullsize_vs_oracle(T, oracle, algo):
    """(32, 512, 768) @ (1, 768, 768): forward, dA, and dB summed back over the broadcast batch, random upstream."""
    T.set_gemm_algo(algo)
    strict = algo == "simt"
    V_ = oracle.View
    rng = np.random.default_rng(22)
    a = rng.standard_normal((32, 512, 768)).astype(np.float32) * 0.05
    b = rng.standard_normal((1, 768, 768)).astype(np.float32) * 0.05
    up = rng.standard_normal((32, 512, 768)).astype(np.float32)
    A, B = T.Tensor.from_numpy(a, requires_grad=True), T.Tensor.from_numpy(b, requires_grad=True)
    C = A.matmul(B)
    assert T.handle().gemm_last_algo() == (0 if strict else 1)
    C.backward(T.Tensor.from_numpy(up))
    T.handle().check_device_status()
    c, da, db = C.numpy(), A.grad().numpy(), B.grad().numpy()
    assert db.shape == (1, 768, 768)
    for i in (0, 13, 31):
        assert product_matches(c[i], V_.of(a[i]), V_.of(b[0]), oracle, strict), f"C batch {i}"
        assert product_matches(da[i], V_.of(up[i]), V_.of(b[0]).t(), oracle, strict), f"dA batch {i}"
    # dB = sum over the batch of A_i^T . dC_i (sum_over_broadcasted_axes, sum_mean_reduction.mojo:184-211: the leading
    # axis is added sequentially, batch ascending): sampled rows of the (768, 768) result
    rows = np.sort(rng.choice(768, 6, replace=False))
    want = np.zeros((len(rows), 768), np.float32)
    scale = np.zeros((len(rows), 768), np.float64)
    for i in range(32):
        left = V_.of(np.ascontiguousarray(a[i][:, rows])).t()
        want = want + oracle.matmul(left, V_.of(up[i]))
        scale += np.abs(left.numpy()).astype(np.float64) @ np.abs(up[i]).astype(np.float64)
    if strict:
        assert np.array_equal(db[0][rows], want)
    else:
        assert float(np.max(np.abs(db[0][rows].astype(np.float64) - want) / scale)) <= TC_TOL


def wide_mlp_params(rng):
    dims = [4096, 4096, 4096, 4096, 1000]
    Ws = [rng.uniform(-1, 1, (dims[i], dims[i + 1])).astype(np.float32) * np.float32(np.sqrt(6.0 / dims[i])) for i in range(4)]
    bs = [(rng.standard_normal(d) * 0.01).astype(np.float32) for d in dims[1:]]
    return dims, Ws, bs


@pytest.mark.parametrize("algo", ["simt", "3xtf32"])
def test_wide_mlp_fullsize_step_vs_oracle(oracle, algo):
    """4096-4096-4096-4096-1000, batch 8192: one step; sampled rows of every activation, of dlogits, of every dX and
    dW, every db, and the updated weights against the oracle (Linear net.mojo:179-216, ReLU relu.mojo:97-141,
    cross-entropy crossentropy.mojo:285-432,664-823, backward matmul.mojo:24-54, SGD optim.mojo:123-158)."""
    from tenmo_b200.trainer import MLPTrainer

    strict = algo == "simt"
    V_ = oracle.View
    rng = np.random.default_rng(23)
    dims, Ws, bs = wide_mlp_params(rng)
    B = 8192
    X = rng.standard_normal((B, dims[0])).astype(np.float32)
    y = rng.integers(0, dims[-1], B)
    tr = MLPTrainer(Ws, bs, batch=B, lr=0.01, momentum=0.9, algo=algo)
    tr.step(X, y, update=False)
    torch.cuda.synchronize()
    tr.h.check_device_status()
    rows = np.sort(rng.choice(B, 8, replace=False))
    ridx = torch.as_tensor(rows, device="cuda")
    acts = [t[ridx].cpu().numpy() for t in tr.act]
    # forward, layer by layer on the GPU's own input rows
    for l in range(4):
        pre = oracle.add_bias(oracle.matmul(acts[l], Ws[l], threads=8), bs[l])
        want = pre if l == 3 else oracle.relu_fwd(pre)[0]
        if strict:
            assert np.array_equal(acts[l + 1], want), f"activation {l + 1}"
            if l < 3:
                assert np.array_equal(tr.mask[l][ridx].cpu().numpy(), oracle.relu_fwd(pre)[1])
        else:
            scale = np.abs(acts[l]).astype(np.float64) @ np.abs(Ws[l]).astype(np.float64) + np.abs(bs[l])
            assert float(np.max(np.abs(acts[l + 1].astype(np.float64) - want) / scale)) <= TC_TOL, f"activation {l + 1}"
    # loss and dlogits from the GPU's logits
    logits = tr.logits()
    r_loss, r_sm, valid = oracle.ce_fwd(logits, y)
    assert abs(tr.loss_value() - float(r_loss)) <= 1e-5 * abs(float(r_loss))
    dlog = tr.gout[3].cpu().numpy()
    assert np.allclose(dlog[rows], oracle.ce_bwd(r_sm, y, valid)[rows], rtol=1e-5, atol=1e-9)
    # backward: dX rows (row-independent), dW rows (a row of dW = one column of the layer input against all of dY), db
    gouts = [t.cpu().numpy() for t in tr.gout]
    for l in range(3, -1, -1):
        g = gouts[l]
        if l > 0:
            dx = oracle.matmul(V_.of(np.ascontiguousarray(g[rows])), V_.of(Ws[l]).t(), threads=8)
            want = oracle.relu_bwd(dx, tr.mask[l - 1][ridx].cpu().numpy())
            if strict:
                assert np.array_equal(gouts[l - 1][rows], want), f"dX of layer {l}"
            else:
                scale = np.abs(g[rows]).astype(np.float64) @ np.abs(Ws[l]).astype(np.float64).T
                assert float(np.max(np.abs(gouts[l - 1][rows].astype(np.float64) - want) / scale)) <= TC_TOL, f"dX of layer {l}"
        wrows = np.sort(rng.choice(dims[l], 4, replace=False))
        a_full = tr.act[l].cpu().numpy()
        left = V_.of(np.ascontiguousarray(a_full[:, wrows])).t()
        got_dw = tr.dW[l][torch.as_tensor(wrows, device="cuda")].cpu().numpy()
        assert product_matches(got_dw, left, V_.of(g), oracle, strict), f"dW of layer {l}"
        # db: 8192 rows are summed as slabs on the GPU, a different order from the oracle's row-ascending fp32 chain; both
        # must sit within fp32 summation error of the exact column sums (bar: 1e-5 of sum |g|)
        exact = g.astype(np.float64).sum(axis=0)
        bound = np.abs(g).astype(np.float64).sum(axis=0)
        assert float(np.max(np.abs(oracle.colsum(g) - exact) / bound)) <= 1e-5
        assert float(np.max(np.abs(tr.db[l].cpu().numpy().astype(np.float64) - exact) / bound)) <= 1e-5, f"db of layer {l}"
    # SGD-momentum on the GPU's own gradients: sampled rows of every updated weight, bit for bit
    dWs = [t.cpu().numpy() for t in tr.dW]
    tr._update()
    torch.cuda.synchronize()
    for l in range(4):
        wrows = np.sort(rng.choice(dims[l], 4, replace=False))
        p = np.ascontiguousarray(Ws[l][wrows])
        vel = np.zeros_like(p)
        oracle.sgd_step(p, np.ascontiguousarray(dWs[l][wrows]), vel, 0.01, 0.9, 0.0)
        assert np.array_equal(tr.W[l][torch.as_tensor(wrows, device="cuda")].cpu().numpy(), p), f"W[{l}] after SGD"
    tr.h.check_device_status()


def test_wide_mlp_fullsize_argmax_identical_to_oracle(oracle):
    """The whole batch of 8192 through the strict-fp32 path: logits, argmax and the correct-count are the oracle's bit
    for bit; on the 3xTF32 path the same inputs give the same predictions except at near-ties."""
    from tenmo_b200.trainer import MLPTrainer

    rng = np.random.default_rng(24)
    dims, Ws, bs = wide_mlp_params(rng)
    B = 8192
    X = rng.standard_normal((B, dims[0])).astype(np.float32)
    y = rng.integers(0, dims[-1], B)
    ref = oracle.MLP(Ws, bs)
    import os

    threads = len(os.sched_getaffinity(0))
    _, r_logits = ref.step(X, y, update=False, threads=threads)
    tr = MLPTrainer(Ws, bs, batch=B, algo="simt")
    tr.step(X, y, update=False)
    got = tr.logits()
    assert np.array_equal(got, r_logits)
    assert np.array_equal(np.argmax(got, 1), np.argmax(r_logits, 1))
    assert tr.accuracy() == oracle.accuracy(r_logits, y)
    del tr
    torch.cuda.empty_cache()
    tc = MLPTrainer(Ws, bs, batch=B, algo="3xtf32")
    tc.step(X, y, update=False)
    agree = float(np.mean(np.argmax(tc.logits(), 1) == np.argmax(r_logits, 1)))
    assert agree >= 0.999, agree
    assert abs(tc.accuracy() - oracle.accuracy(r_logits, y)) <= 8
    tc.h.check_device_status()
