"""Broadcast-batched and attention-shaped matmul with full autograd backward (384 x (512, 64) heads and (32, 512, 768) @ (1, 768, 768)).

Small shapes go through the strict-fp32 kernel and are compared with the oracle chain element by element;
the full-size shapes (B*H = 384, S = 512, D = 64 and (32,512,768)@(1,768,768)) go through the tensor-core
kernel and are checked on sampled batches against fp64 plus size-independent properties (softmax rows sum
to one, gradients of a sum are column sums).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def T():
    import tenmo_b200.tensor as tensor

    tensor.handle()
    return tensor


def test_attention_chain_small_matches_oracle(T, oracle):
    """scores = Q.K^T (K^T a stride view), P = softmax(scores), ctx = P.V, loss = sum(ctx); every gradient."""
    T.set_gemm_algo("simt")
    rng = np.random.default_rng(3)
    BH, S, D = 6, 40, 16
    q, k, v = (rng.standard_normal((BH, S, D)).astype(np.float32) * 0.25 for _ in range(3))
    Q, K, V = (T.Tensor.from_numpy(a, requires_grad=True) for a in (q, k, v))
    scores = Q.matmul(K.transpose())
    P = scores.softmax()
    ctx = P.matmul(V)
    ctx.sum().backward()
    # oracle chain (tests/test_attn_matmul.mojo:194-259 does the same with ones)
    s_ref = oracle.matmul(oracle.View.of(q), oracle.View.of(k).t())
    assert np.array_equal(scores.numpy(), s_ref)
    p_ref = oracle.softmax_fwd(s_ref)
    assert np.allclose(P.numpy(), p_ref, rtol=2e-6, atol=1e-8)
    c_ref = oracle.matmul(p_ref, v)
    assert np.allclose(ctx.numpy(), c_ref, rtol=1e-5, atol=1e-6)
    g = np.ones_like(c_ref)
    dV = oracle.matmul(oracle.View.of(p_ref).t(), oracle.View.of(g))
    dP = oracle.matmul(oracle.View.of(g), oracle.View.of(v).t())
    dS = oracle.softmax_bwd(dP, p_ref)
    dQ = oracle.matmul(dS, k)
    dK = np.swapaxes(oracle.matmul(oracle.View.of(q).t(), oracle.View.of(dS)), 1, 2)
    assert np.allclose(V.grad().numpy(), dV, rtol=1e-5, atol=1e-6)
    assert np.allclose(Q.grad().numpy(), dQ, rtol=1e-4, atol=1e-6)
    assert np.allclose(K.grad().numpy(), dK, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("mc", [(7, 5), (300, 512), (64, 1000), (10, 2500)], ids=str)
def test_softmax_kernels_vs_oracle(T, oracle, mc):
    from tests import gpu_util as g

    M, C = mc
    h = g.handle()
    rng = np.random.default_rng(M + C)
    x = (rng.standard_normal((M, C)) * 3).astype(np.float32)
    up = rng.standard_normal((M, C)).astype(np.float32)
    xd, yd, gd, dd = g.dev(x), g.empty(M, C), g.dev(up), g.empty(M, C)
    h.softmax_fwd(xd.data_ptr(), C, yd.data_ptr(), M, C)
    y = g.host(yd)
    ref = oracle.softmax_fwd(x)
    assert np.allclose(y, ref, rtol=1e-5, atol=1e-8) and np.allclose(y.sum(axis=1), 1.0, atol=1e-5)
    h.softmax_bwd(yd.data_ptr(), gd.data_ptr(), dd.data_ptr(), M, C)
    assert np.allclose(g.host(dd), oracle.softmax_bwd(up, y), rtol=1e-4, atol=1e-6)
    h.softmax_bwd(yd.data_ptr(), gd.data_ptr(), dd.data_ptr(), M, C, beta=1.0)
    assert np.allclose(g.host(dd), 2 * oracle.softmax_bwd(up, y), rtol=1e-4, atol=1e-6)


def test_attention_full_size_tensor_core(T):
    """Config 3 (ii) at full size on the 3xTF32 kernel: forward + backward of both batched GEMMs."""
    T.set_gemm_algo("3xtf32")
    try:
        rng = np.random.default_rng(11)
        BH, S, D = 384, 512, 64
        q, k, v = (rng.standard_normal((BH, S, D)).astype(np.float32) * 0.125 for _ in range(3))
        Q, K, V = (T.Tensor.from_numpy(a, requires_grad=True) for a in (q, k, v))
        scores = Q.matmul(K.transpose())
        assert T.handle().gemm_last_algo() == 1
        P = scores.softmax()
        ctx = P.matmul(V)
        ctx.sum().backward()
        T.handle().check_device_status()
        p = P.numpy()
        assert np.allclose(p.sum(axis=-1), 1.0, atol=1e-5)           # softmax rows sum to one
        dv = V.grad().numpy()
        assert np.allclose(dv, np.repeat(p.sum(axis=1)[:, :, None], D, axis=2), rtol=1e-4, atol=1e-5)  # dV = P^T.1
        sc, cx, dq, dk = scores.numpy(), ctx.numpy(), Q.grad().numpy(), K.grad().numpy()
        for b in (0, 191, 383):  # sampled batches against fp64
            q64, k64, v64 = q[b].astype(np.float64), k[b].astype(np.float64), v[b].astype(np.float64)
            s64 = q64 @ k64.T
            assert np.max(np.abs(sc[b] - s64)) <= 1e-5
            e = np.exp(s64 - s64.max(axis=1, keepdims=True))
            p64 = e / e.sum(axis=1, keepdims=True)
            assert np.max(np.abs(cx[b] - p64 @ v64)) <= 1e-5
            dP = np.ones((S, D)) @ v64.T
            dS = p64 * (dP - (dP * p64).sum(axis=1, keepdims=True))
            assert np.max(np.abs(dq[b] - dS @ k64)) <= 1e-5 * max(1.0, np.max(np.abs(dS @ k64)))
            assert np.max(np.abs(dk[b] - dS.T @ q64)) <= 1e-5 * max(1.0, np.max(np.abs(dS.T @ q64)))
    finally:
        T.set_gemm_algo("simt")


def test_broadcast_batched_full_size(T):
    """Config 3 (i): (32, 512, 768) @ (1, 768, 768); dB is summed back over the broadcast batch."""
    T.set_gemm_algo("3xtf32")
    try:
        rng = np.random.default_rng(12)
        a = rng.standard_normal((32, 512, 768)).astype(np.float32) * 0.05
        b = rng.standard_normal((1, 768, 768)).astype(np.float32) * 0.05
        A, B = T.Tensor.from_numpy(a, requires_grad=True), T.Tensor.from_numpy(b, requires_grad=True)
        C = A.matmul(B)
        C.sum().backward()
        T.handle().check_device_status()
        a64, b64 = a.astype(np.float64), b.astype(np.float64)
        c = C.numpy()
        for i in (0, 17, 31):
            assert np.max(np.abs(c[i] - a64[i] @ b64[0])) <= 1e-5
        # d sum(C) / dA = 1 . B^T (every row the row sums of B); dB = sum_b A_b^T . 1 (column sums of A over batch and rows)
        assert np.allclose(A.grad().numpy(), np.broadcast_to(b64[0].sum(axis=1), a.shape), rtol=1e-4, atol=1e-5)
        want_db = np.repeat(a64.sum(axis=(0, 1))[:, None], 768, axis=1)[None]
        assert B.grad().shape() == (1, 768, 768)
        assert np.allclose(B.grad().numpy(), want_db, rtol=1e-4, atol=1e-3)
    finally:
        T.set_gemm_algo("simt")
