"""Pins the CPU oracle against the known-answer vectors of the reference's own tests (CPU only)."""
import math

import numpy as np
import pytest

from tests.golden import reference_kat as kat


def f32(x):
    return np.asarray(x, dtype=np.float32)


def all_close(a, b, rtol=1e-5, atol=1e-8):
    # buffers.mojo:1909-1946: |a-b| <= atol + rtol*|b|
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return a.shape == b.shape and bool(np.all(np.abs(a - b) <= atol + rtol * np.abs(b)))


@pytest.mark.parametrize("case", kat.MM2D, ids=lambda c: c["name"])
@pytest.mark.parametrize("contract", [0, 1])
def test_mm2d_literals(oracle, case, contract):
    A, B = f32(case["A"]), f32(case["B"])
    C = oracle.matmul(A, B, contract_scalar=contract)
    assert all_close(C, f32(case["C"]))
    # validate_matmul_2d_grads (tests/test_mm2d.mojo:39-100): dA = dC.B^T, dB = A^T.dC with dC = ones
    dC = np.ones_like(C)
    dA = oracle.matmul(dC, oracle.View.of(B).t(), contract_scalar=contract)
    dB = oracle.matmul(oracle.View.of(A).t(), dC, contract_scalar=contract)
    assert all_close(dA, dC @ B.T) and all_close(dB, A.T @ dC)


@pytest.mark.parametrize("case", kat.MM2D_VIEWS, ids=lambda c: c["name"])
def test_mm2d_views(oracle, case):
    A = oracle.View(f32(case["A_base"]), case["A_shape"], case["A_strides"], case["A_offset"])
    C = oracle.matmul(A, f32(case["B"]))
    assert all_close(C, f32(case["C"]))


@pytest.mark.parametrize("case", kat.MMND_GRADS, ids=lambda c: c["name"])
def test_mmnd_grads(oracle, case):
    A, B = f32(case["A"]), f32(case["B"])
    C = oracle.matmul(A, B)
    if "C" in case:
        assert all_close(C, f32(case["C"]), atol=1e-5)
    dC = np.ones_like(C)
    # MatmulNdBackward (matmul.mojo:101-137): batched GEMMs on transposed views, then
    # sum_over_broadcasted_axes back to each parent's shape.
    dA_full = oracle.matmul(dC, oracle.View.of(B).t())
    dB_full = oracle.matmul(oracle.View.of(A).t(), dC)

    def sum_to(x, shape):
        while x.ndim > len(shape):
            x = x.sum(axis=0)
        for i, s in enumerate(shape):
            if x.shape[i] != s and x.shape[i] > 1:
                x = x.sum(axis=i, keepdims=True)
        return x

    assert all_close(sum_to(dA_full, A.shape), f32(case["dA"]))
    assert all_close(sum_to(dB_full, B.shape), f32(case["dB"]))


@pytest.mark.parametrize("shapes", kat.ONES_SHAPES, ids=str)
def test_ones_fill_k(oracle, shapes):
    sa, sb = shapes
    C = oracle.matmul(np.ones(sa, np.float32), np.ones(sb, np.float32))
    assert C.shape == tuple(np.broadcast_shapes(sa[:-2], sb[:-2])) + (sa[-2], sb[-1])
    assert np.all(C == sa[-1])


@pytest.mark.parametrize("mkn", kat.SHAPE_SWEEP, ids=str)
@pytest.mark.parametrize("layout", ["nn", "a_t", "b_t", "b_padded"])
def test_shape_sweep_vs_naive(oracle, mkn, layout):
    M, K, N = mkn
    if layout != "nn" and M * K * N > 2_000_000:
        pytest.skip("large case only in the contiguous layout")
    rng = np.random.default_rng(M * 1000003 + K * 1009 + N)
    A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32)
    Av, Bv = oracle.View.of(A), oracle.View.of(B)
    if layout == "a_t":
        Av = oracle.View.of(np.ascontiguousarray(A.T)).t()
    elif layout == "b_t":
        Bv = oracle.View.of(np.ascontiguousarray(B.T)).t()
    elif layout == "b_padded":  # tests/test_matmul_2d_verify.mojo:85-110
        wide = np.zeros((K, N + 2), np.float32)
        wide[:, :N] = B
        Bv = oracle.View(wide.reshape(-1), (K, N), (N + 2, 1), 0)
    C = oracle.matmul(Av, Bv, threads=2)
    ref = oracle.matmul_naive(Av, Bv)
    assert all_close(C, ref, atol=1e-4 * max(1, K // 32))
    # the fp64 product bounds both
    assert np.max(np.abs(C - A.astype(np.float64) @ B.astype(np.float64))) < 1e-5 * K * 16


def test_fma_chain_is_bit_exact(oracle):
    """Every output is one k-ascending fused-multiply-add chain, whatever the tiling or thread count."""
    rng = np.random.default_rng(7)
    for (M, K, N) in [(3, 70, 5), (70, 129, 300), (130, 33, 40)]:
        A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32)
        C = oracle.matmul(A, B, threads=3)
        ref = np.zeros((M, N), np.float32)
        for k in range(K):  # float64 a*b is exact for fp32 inputs, one rounding per step = fmaf
            ref = (A[:, k:k + 1].astype(np.float64) * B[k:k + 1, :].astype(np.float64) + ref.astype(np.float64)
                   ).astype(np.float32)
        # double rounding (exact product + fp32 acc rounded once from fp64) can differ from a true FMA
        # only when the fp64 sum itself rounds, which needs > 53 significant bits: rare, so compare with
        # a 1-ulp allowance and require bit equality for almost all entries.
        assert np.mean(C == ref) > 0.999
        assert np.max(np.abs(C - ref)) <= np.max(np.abs(ref)) * 2.0 ** -22
        # transposed-view operand goes down the scalar path; with contraction on it is the same chain
        Ct = oracle.matmul(oracle.View.of(np.ascontiguousarray(A.T)).t(), B, contract_scalar=1)
        Cb = oracle.matmul(A, oracle.View.of(np.ascontiguousarray(B.T)).t(), contract_scalar=1)
        assert np.array_equal(C, Ct) and np.array_equal(C, Cb)


@pytest.mark.parametrize("case", kat.SGD, ids=lambda c: c["name"])
def test_sgd_literals(oracle, case):
    p = np.ones((2, 2), np.float32)
    v = np.zeros_like(p)
    for g, want in zip(case["grads"], case["expect"]):
        oracle.sgd_step(p, np.full((2, 2), g, np.float32), v, case["lr"], case["momentum"], case["wd"])
        assert all_close(p, np.full((2, 2), want, np.float32))


@pytest.mark.parametrize("case", kat.ACCURACY, ids=lambda c: str(c["correct"]))
def test_accuracy_literals(oracle, case):
    assert oracle.accuracy(f32(case["pred"]), case["target"]) == case["correct"]


def test_accuracy_large_batch(oracle):
    # tests/test_accuracy.mojo:57-72
    M, Cc = 1000, 10
    pred = np.full((M, Cc), 0.1, np.float32)
    tgt = np.arange(M) % Cc
    pred[np.arange(M), tgt] = 0.9
    assert oracle.accuracy(pred, tgt) == M


def test_ce_ignore_index_label_smoothing(oracle):
    c = kat.CE_IGNORE_LS
    logits, tg = f32(c["logits"]), c["targets"]
    kw = dict(ignore_index=c["ignore_index"], label_smoothing=c["label_smoothing"])
    loss, sm, valid = oracle.ce_fwd(logits, tg, "mean", **kw)
    assert valid == 2 and all_close(loss, c["mean_loss"])
    assert all_close(oracle.ce_bwd(sm, tg, valid, "mean", **kw), f32(c["mean_grad"]), atol=1e-7)
    loss, sm, valid = oracle.ce_fwd(logits, tg, "sum", **kw)
    assert all_close(loss, c["sum_loss"])
    assert all_close(oracle.ce_bwd(sm, tg, valid, "sum", **kw), f32(c["sum_grad"]), atol=1e-7)
    loss, sm, valid = oracle.ce_fwd(logits, tg, "none", **kw)
    assert all_close(loss, f32(c["none_loss"]))
    assert all_close(oracle.ce_bwd(sm, tg, valid, "none", **kw), f32(c["sum_grad"]), atol=1e-7)


def test_ce_closed_forms(oracle):
    c = kat.CE_UNIFORM
    loss, sm, _ = oracle.ce_fwd(f32(c["logits"]), c["targets"])
    assert abs(loss - (-math.log(1.0 / 3.0))) < 1e-6
    assert all_close(sm, np.full((2, 3), 1 / 3, np.float32))
    c = kat.CE_BASIC
    loss, sm, valid = oracle.ce_fwd(f32(c["logits"]), c["targets"])
    s1 = math.exp(2.0) / (math.exp(2.0) + math.exp(1.0) + math.exp(0.5))
    s2 = math.exp(2.0) / (math.exp(1.0) + math.exp(2.0) + math.exp(0.1))
    assert abs(loss - (-math.log(s1) - math.log(s2)) / 2.0) < 1e-6
    # tests/test_cross_entropy.mojo:1465-1476: grad = (softmax - onehot) / batch
    g = oracle.ce_bwd(sm, c["targets"], valid)
    oh = np.eye(3, dtype=np.float32)[c["targets"]]
    assert all_close(g, (sm - oh) / 2, atol=1e-7)


def test_elementwise_and_colsum(oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((37, 19), np.float32)
    b = rng.standard_normal(19, np.float32)
    assert np.array_equal(oracle.add_bias(x, b), x + b)
    out, mask = oracle.relu_fwd(x)
    assert np.array_equal(out, np.maximum(x, 0)) and np.array_equal(mask, (x > 0).astype(np.float32))
    assert np.array_equal(oracle.relu_bwd(x, mask), x * mask)
    y = oracle.sigmoid_fwd(x)
    assert all_close(y, 1 / (1 + np.exp(-x.astype(np.float64))), rtol=1e-6)
    assert np.array_equal(oracle.sigmoid_bwd(x, y), (x * y) * (np.float32(1) - y))
    cs = oracle.colsum(x)
    seq = np.zeros(19, np.float32)
    for i in range(37):
        seq = seq + x[i]
    assert np.array_equal(cs, seq)


def test_mlp_step_matches_composed_ops(oracle):
    """The fused step driver of the oracle equals the op-by-op sequence and lowers the loss."""
    rng = np.random.default_rng(11)
    dims = [20, 16, 8, 5]
    Ws = [rng.uniform(-0.4, 0.4, (dims[i], dims[i + 1])).astype(np.float32) for i in range(3)]
    bs = [np.zeros(dims[i + 1], np.float32) for i in range(3)]
    X = rng.uniform(0, 1, (12, 20)).astype(np.float32)
    y = rng.integers(0, 5, 12)
    mlp = oracle.MLP(Ws, bs)
    loss0, logits = mlp.step(X, y, update=False)
    # op-by-op forward
    h = X
    for l in range(3):
        z = oracle.add_bias(oracle.matmul(h, Ws[l]), bs[l])
        h = oracle.relu_fwd(z)[0] if l < 2 else z
    assert np.array_equal(h, logits)
    l_ref, sm, valid = oracle.ce_fwd(h, y)
    assert loss0 == pytest.approx(float(l_ref), abs=0)
    g = oracle.ce_bwd(sm, y, valid)
    assert np.array_equal(mlp.db[2], oracle.colsum(g))
    losses = [mlp.step(X, y, lr=0.05)[0] for _ in range(60)]
    assert losses[-1] < 0.9 * losses[0]
