"""Parity of the CUDA path (through the C ABI) with the CPU oracle, on a B200.

Bars: the strict-FP32 SIMT GEMM must be BIT-IDENTICAL to the oracle's fused-multiply-add chain
(stricter than the 1e-5 relative error the path asks for); reductions whose summation order differs
from the reference's sequential loops are held to 1e-5 relative to the sum of magnitudes; integer
results (accuracy counts, valid counts) are exact.
"""
import numpy as np
import pytest

from tests.golden import reference_kat as kat

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def g():
    from tests import gpu_util

    gpu_util.handle()
    return gpu_util


def f32(x):
    return np.asarray(x, dtype=np.float32)


SIMT = 0


# ---------------------------------------------------------------------------------------------------
# GEMM: reference literals
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", kat.MM2D, ids=lambda c: c["name"])
def test_gemm_mm2d_literals(g, oracle, case):
    A, B = oracle.View.of(f32(case["A"])), oracle.View.of(f32(case["B"]))
    C, _, _ = g.gpu_matmul(A, B, algo=SIMT)
    assert np.array_equal(C, f32(case["C"]))
    dC = oracle.View.of(np.ones_like(C))
    dA, _, _ = g.gpu_matmul(dC, B.t(), algo=SIMT)
    dB, _, _ = g.gpu_matmul(A.t(), dC, algo=SIMT)
    assert np.array_equal(dA, np.ones_like(C) @ f32(case["B"]).T)
    assert np.array_equal(dB, f32(case["A"]).T @ np.ones_like(C))


@pytest.mark.parametrize("case", kat.MM2D_VIEWS, ids=lambda c: c["name"])
def test_gemm_views(g, oracle, case):
    A = oracle.View(f32(case["A_base"]), case["A_shape"], case["A_strides"], case["A_offset"])
    C, _, _ = g.gpu_matmul(A, oracle.View.of(f32(case["B"])), algo=SIMT)
    assert np.array_equal(C, f32(case["C"]))


@pytest.mark.parametrize("case", kat.MMND_GRADS, ids=lambda c: c["name"])
def test_gemm_nd_grads(g, oracle, case):
    A, B = f32(case["A"]), f32(case["B"])
    Av, Bv = oracle.View.of(A), oracle.View.of(B)
    C, _, _ = g.gpu_matmul(Av, Bv, algo=SIMT)
    assert np.array_equal(C, oracle.matmul(Av, Bv))
    if "C" in case:
        assert np.array_equal(C, f32(case["C"]))
    dC = oracle.View.of(np.ones_like(C))
    dA_full, _, _ = g.gpu_matmul(dC, Bv.t(), algo=SIMT)
    dB_full, _, _ = g.gpu_matmul(Av.t(), dC, algo=SIMT)
    h = g.handle()

    def sum_leading(x, shape):
        # sum_over_broadcasted_axes through tenmo_colsum_f32: leading batch -> rows, the rest -> columns
        if x.shape == shape:
            return x
        lead = int(np.prod(x.shape)) // int(np.prod(shape))
        xd, out = g.dev(x), g.empty(int(np.prod(shape)))
        h.colsum(xd.data_ptr(), lead, int(np.prod(shape)), int(np.prod(shape)), out.data_ptr())
        return g.host(out).reshape(shape)

    assert np.array_equal(sum_leading(dA_full, A.shape), f32(case["dA"]))
    assert np.array_equal(sum_leading(dB_full, B.shape), f32(case["dB"]))


@pytest.mark.parametrize("shapes", kat.ONES_SHAPES, ids=str)
def test_gemm_ones_fill_k(g, oracle, shapes):
    sa, sb = shapes
    C, _, _ = g.gpu_matmul(oracle.View.of(np.ones(sa, np.float32)), oracle.View.of(np.ones(sb, np.float32)), algo=SIMT)
    assert C.shape == tuple(np.broadcast_shapes(sa[:-2], sb[:-2])) + (sa[-2], sb[-1])
    assert np.all(C == sa[-1])


# ---------------------------------------------------------------------------------------------------
# GEMM: shape sweep, all layouts, bit-exact against the oracle
# ---------------------------------------------------------------------------------------------------
EXTRA_SHAPES = [(64, 784, 128), (64, 128, 32), (64, 32, 10), (130, 257, 131), (256, 64, 384), (1, 1, 300), (300, 1, 1),
                (129, 16, 127), (33, 17, 65), (257, 300, 129)]


def _layout_views(oracle, A, B, layout, rng):
    Av, Bv = oracle.View.of(A), oracle.View.of(B)
    M, K = A.shape
    N = B.shape[1]
    if layout == "a_t":
        Av = oracle.View.of(np.ascontiguousarray(A.T)).t()
    elif layout == "b_t":
        Bv = oracle.View.of(np.ascontiguousarray(B.T)).t()
    elif layout == "both_t":
        Av = oracle.View.of(np.ascontiguousarray(A.T)).t()
        Bv = oracle.View.of(np.ascontiguousarray(B.T)).t()
    elif layout == "padded":  # padded rows + odd offsets: unaligned scalar path (test_matmul_2d_verify.mojo:85-229)
        wa = rng.standard_normal((M, K + 3), np.float32)
        wa[:, :K] = A
        wb = rng.standard_normal((K, N + 2), np.float32)
        wb[:, :N] = B
        Av = oracle.View(np.concatenate([np.zeros(1, np.float32), wa.reshape(-1)]), (M, K), (K + 3, 1), 1)
        Bv = oracle.View(np.concatenate([np.zeros(3, np.float32), wb.reshape(-1)]), (K, N), (N + 2, 1), 3)
    elif layout == "strided":  # inner stride 2 on both operands (tests/test_mmnd.mojo:170-190)
        wa = rng.standard_normal((M, 2 * K), np.float32)
        wa[:, ::2] = A
        wb = rng.standard_normal((K, 2 * N), np.float32)
        wb[:, ::2] = B
        Av = oracle.View(wa.reshape(-1), (M, K), (2 * K, 2), 0)
        Bv = oracle.View(wb.reshape(-1), (K, N), (2 * N, 2), 0)
    return Av, Bv


@pytest.mark.parametrize("mkn", kat.SHAPE_SWEEP + EXTRA_SHAPES, ids=str)
@pytest.mark.parametrize("layout", ["nn", "a_t", "b_t", "both_t", "padded", "strided"])
def test_gemm_simt_bit_exact(g, oracle, mkn, layout):
    M, K, N = mkn
    if layout != "nn" and M * K * N > 20_000_000:
        pytest.skip("largest case only in the contiguous layout")
    rng = np.random.default_rng(M * 1000003 + K * 1009 + N)
    A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32)
    Av, Bv = _layout_views(oracle, A, B, layout, rng)
    C, _, _ = g.gpu_matmul(Av, Bv, algo=SIMT)
    ref = oracle.matmul(Av, Bv, contract_scalar=1, threads=4)
    assert np.array_equal(C, ref), f"max abs diff {np.max(np.abs(C - ref))}"
    # the reference's own check: naive loop at atol 1e-4 (scaled for long K)
    assert np.allclose(C, oracle.matmul_naive(Av, Bv), rtol=1e-5, atol=1e-4 * max(1, K // 32))


@pytest.mark.parametrize("mkn", [(256, 4096, 10), (5, 700, 1), (33, 513, 32), (4, 512, 7), (1000, 1555, 3)], ids=str)
@pytest.mark.parametrize("layout", ["nn", "a_t", "b_t", "strided"])
def test_gemm_narrow_result_kernel_bit_exact(g, oracle, mkn, layout):
    """A result of at most 32 columns over a long contraction runs on its own strict-fp32 kernel: same chain, same bits,
    with the Linear epilogue (bias, ReLU + mask) and the accumulate."""
    M, K, N = mkn
    rng = np.random.default_rng(M + 3 * K + 7 * N)
    A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32) * 0.05
    bias = rng.standard_normal(N).astype(np.float32)
    Av, Bv = _layout_views(oracle, A, B, layout, rng)
    C, _, _ = g.gpu_matmul(Av, Bv, algo=SIMT)
    assert g.handle().gemm_last_kernel() == "gemm_skinny_kernel"
    ref = oracle.matmul(Av, Bv, contract_scalar=1, threads=4)
    assert np.array_equal(C, ref)
    C, aux, _ = g.gpu_matmul(Av, Bv, algo=SIMT, bias=bias, act=1, want_aux=True)
    out, mask = oracle.relu_fwd(oracle.add_bias(ref, bias))
    assert np.array_equal(C, out) and np.array_equal(aux, mask)
    init = rng.standard_normal((M, N), np.float32)
    C, _, _ = g.gpu_matmul(Av, Bv, algo=SIMT, beta=1.0, c_init=init)
    assert np.array_equal(C, init + ref)


def test_gemm_small_exhaustive(g, oracle):
    """Every M, N, K in a small box on the scalar-tail-heavy sizes: one launch each, all bit-exact."""
    rng = np.random.default_rng(5)
    for M in (1, 2, 3, 5, 8, 31, 33):
        for N in (1, 2, 4, 7, 9, 32, 35):
            for K in (0, 1, 3, 4, 17, 32, 40):
                A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32)
                C, _, _ = g.gpu_matmul(oracle.View.of(A), oracle.View.of(B), algo=SIMT)
                ref = oracle.matmul(A, B) if K > 0 else np.zeros((M, N), np.float32)
                assert np.array_equal(C, ref), (M, N, K)


def test_gemm_batched_broadcast_and_transposed_view(g, oracle):
    rng = np.random.default_rng(21)
    # (B,M,K) @ (1,K,N)
    A = rng.standard_normal((5, 70, 48), np.float32)
    B = rng.standard_normal((1, 48, 36), np.float32)
    C, _, _ = g.gpu_matmul(oracle.View.of(A), oracle.View.of(B), algo=SIMT)
    assert np.array_equal(C, oracle.matmul(A, B))
    # attention-shaped: Q @ K^T with K^T a stride-permuted view, then P @ V
    BH, S, D = 6, 40, 16
    Q, Kt, V = (rng.standard_normal((BH, S, D), np.float32) * 0.125 for _ in range(3))
    Kv = oracle.View.of(Kt).t()
    scores, _, _ = g.gpu_matmul(oracle.View.of(Q), Kv, algo=SIMT)
    assert np.array_equal(scores, oracle.matmul(oracle.View.of(Q), Kv))
    ctx, _, _ = g.gpu_matmul(oracle.View.of(scores), oracle.View.of(V), algo=SIMT)
    assert np.array_equal(ctx, oracle.matmul(scores, V))
    # 4-D broadcast batch (1,2,M,K) @ (3,2,K,N)  (tests/test_attn_matmul.mojo broadcast case)
    A4 = rng.standard_normal((1, 2, 9, 8), np.float32)
    B4 = rng.standard_normal((3, 2, 8, 5), np.float32)
    C4, _, _ = g.gpu_matmul(oracle.View.of(A4), oracle.View.of(B4), algo=SIMT)
    assert np.array_equal(C4, oracle.matmul(A4, B4))
    # overlapping batch view with offset (tests/test_mmnd.mojo:94-128): shape (2,2,2), strides (2,2,1), offset 4
    base = np.arange(12, dtype=np.float32)
    Av = oracle.View(base, (2, 2, 2), (2, 2, 1), 4)
    Bv = oracle.View.of(np.eye(2, dtype=np.float32))
    Co, _, _ = g.gpu_matmul(Av, Bv, algo=SIMT)
    assert np.array_equal(Co, oracle.matmul(Av, Bv))


@pytest.mark.parametrize("mkn", [(64, 784, 128), (130, 70, 33), (256, 256, 256)], ids=str)
def test_gemm_epilogue(g, oracle, mkn):
    """Linear = matmul + bias (+ ReLU with mask | Sigmoid) and the beta = 1 accumulate."""
    M, K, N = mkn
    rng = np.random.default_rng(M + N)
    A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32) * 0.1
    bias = rng.standard_normal(N).astype(np.float32)
    Av, Bv = oracle.View.of(A), oracle.View.of(B)
    z = oracle.add_bias(oracle.matmul(A, B), bias)
    C, _, _ = g.gpu_matmul(Av, Bv, algo=SIMT, bias=bias)
    assert np.array_equal(C, z)
    C, aux, _ = g.gpu_matmul(Av, Bv, algo=SIMT, bias=bias, act=1, want_aux=True)
    out, mask = oracle.relu_fwd(z)
    assert np.array_equal(C, out) and np.array_equal(aux, mask)
    C, _, _ = g.gpu_matmul(Av, Bv, algo=SIMT, bias=bias, act=2)
    assert np.allclose(C, oracle.sigmoid_fwd(z), rtol=2e-6, atol=1e-7)  # expf vs libm exp
    init = rng.standard_normal((M, N), np.float32)
    C, _, _ = g.gpu_matmul(Av, Bv, algo=SIMT, beta=1.0, c_init=init)
    assert np.array_equal(C, init + oracle.matmul(A, B))
    # dW = X^T . dY with db riding along as the column sum of dY
    C, _, cs = g.gpu_matmul(Av.t(), oracle.View.of(init), algo=SIMT, colsum=True)
    assert np.array_equal(C, oracle.matmul(Av.t(), oracle.View.of(init)))
    assert np.array_equal(cs, oracle.colsum(init))


def test_gemm_argument_errors(g):
    from tenmo_b200 import TenmoError, make_mat

    h = g.handle()
    a = g.empty(4, 4)
    ma = make_mat(a.data_ptr(), (4, 4), (4, 1))
    with pytest.raises(TenmoError) as e:
        h.gemm(4, 4, 4, ma, ma, a.data_ptr(), beta=0.5)
    assert e.value.status == -1
    with pytest.raises(TenmoError):
        h.gemm(-1, 4, 4, ma, ma, a.data_ptr())
    with pytest.raises(TenmoError):
        h.gemm(4, 4, 4, ma, ma, a.data_ptr(), act=7)
    b3 = make_mat(a.data_ptr(), (3, 2, 2), (4, 2, 1))
    b2 = make_mat(a.data_ptr(), (2, 2, 2), (4, 2, 1))
    with pytest.raises(TenmoError) as e:  # batch shapes not broadcastable (matmul_cpu.mojo:658-662)
        h.gemm(2, 2, 2, b3, b2, a.data_ptr())
    assert "broadcast" in str(e.value)
    h.gemm(0, 4, 4, ma, ma, a.data_ptr())  # empty output is a no-op, not an error


# ---------------------------------------------------------------------------------------------------
# elementwise, reductions
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 3, 4, 1023, 4096, 100003])
def test_elementwise(g, oracle, n):
    h = g.handle()
    rng = np.random.default_rng(n)
    x, y = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    xd, yd, od, md = g.dev(x), g.dev(y), g.empty(n), g.empty(n)
    h.relu_fwd(xd.data_ptr(), od.data_ptr(), md.data_ptr(), n)
    out, mask = oracle.relu_fwd(x)
    assert np.array_equal(g.host(od), out) and np.array_equal(g.host(md), mask)
    h.relu_bwd(yd.data_ptr(), md.data_ptr(), od.data_ptr(), n)
    assert np.array_equal(g.host(od), oracle.relu_bwd(y, mask))
    h.relu_bwd(yd.data_ptr(), md.data_ptr(), od.data_ptr(), n, beta=1.0)
    assert np.array_equal(g.host(od), oracle.relu_bwd(y, mask) * 2)
    h.sigmoid_fwd(xd.data_ptr(), od.data_ptr(), n)
    sg = oracle.sigmoid_fwd(x)
    assert np.allclose(g.host(od), sg, rtol=2e-6, atol=1e-7)
    sd = g.dev(sg)
    h.sigmoid_bwd(yd.data_ptr(), sd.data_ptr(), od.data_ptr(), n)
    assert np.array_equal(g.host(od), oracle.sigmoid_bwd(y, sg))
    # in place: the gradient buffer is also the output (what the convolution layers do with the ReLU mask), and the
    # activation is overwritten by its own sigmoid / its own backward
    gd = g.dev(y)
    h.relu_bwd(gd.data_ptr(), md.data_ptr(), gd.data_ptr(), n)
    assert np.array_equal(g.host(gd), oracle.relu_bwd(y, mask))
    gd = g.dev(y)
    h.sigmoid_bwd(gd.data_ptr(), sd.data_ptr(), gd.data_ptr(), n)
    assert np.array_equal(g.host(gd), oracle.sigmoid_bwd(y, sg))
    xi = g.dev(x)
    h.relu_fwd(xi.data_ptr(), xi.data_ptr(), 0, n)
    assert np.array_equal(g.host(xi), out)
    h.add_inplace(xd.data_ptr(), yd.data_ptr(), n)
    assert np.array_equal(g.host(xd), x + y)
    h.fill(xd.data_ptr(), 0.0, n)
    assert not g.host(xd).any()
    # unaligned views of a larger buffer take the scalar path
    if n > 8:
        big = g.dev(np.concatenate([[0.0], x]).astype(np.float32))
        o2 = g.empty(n + 1)
        h.relu_fwd(big.data_ptr() + 4, o2.data_ptr() + 4, 0, n)
        assert np.array_equal(g.host(o2)[1:], out)


@pytest.mark.parametrize("mn", [(64, 128), (64, 10), (7, 33), (1000, 4096), (4099, 130), (8192, 1000), (513, 1), (20000, 12)],
                         ids=str)
def test_add_bias_and_colsum(g, oracle, mn):
    M, N = mn
    h = g.handle()
    rng = np.random.default_rng(M * 7 + N)
    x, b = rng.standard_normal((M, N), np.float32), rng.standard_normal(N).astype(np.float32)
    xd, bd, od = g.dev(x), g.dev(b), g.empty(M, N)
    h.add_bias(xd.data_ptr(), bd.data_ptr(), od.data_ptr(), M, N)
    assert np.array_equal(g.host(od), oracle.add_bias(x, b))
    cs = g.empty(N)
    h.colsum(xd.data_ptr(), M, N, N, cs.data_ptr())
    ref = oracle.colsum(x)
    if M <= 512:
        assert np.array_equal(g.host(cs), ref)  # ascending-row order, bit-identical
    else:
        scale = np.abs(x).sum(axis=0)
        assert np.max(np.abs(g.host(cs) - ref) / scale) <= 1e-5
        assert np.max(np.abs(g.host(cs) - x.astype(np.float64).sum(axis=0)) / scale) <= 1e-6
    first = g.host(cs).copy()
    h.colsum(xd.data_ptr(), M, N, N, cs.data_ptr(), beta=1.0)
    assert np.array_equal(g.host(cs), first + first)
    h.colsum(xd.data_ptr(), M, N, N, cs.data_ptr())
    assert np.array_equal(g.host(cs), first)  # run-to-run identical: the order does not depend on scheduling


# ---------------------------------------------------------------------------------------------------
# cross-entropy, SGD, accuracy
# ---------------------------------------------------------------------------------------------------
def _ce_gpu(g, logits, labels, reduction, ignore_index=-100, ls=0.0, i64=True):
    from tenmo_b200.lib import REDUCTION

    h = g.handle()
    M, C = logits.shape
    red = REDUCTION[reduction]
    ld, sm, dl = g.dev(logits), g.empty(M, C), g.empty(M, C)
    lab = g.dev(labels, np.int64 if i64 else np.int32)
    loss = g.empty(M if red == 2 else 1)
    vc = torch.zeros(1, dtype=torch.int32, device="cuda")
    h.ce_fwd(ld.data_ptr(), C, lab.data_ptr(), i64, M, C, ignore_index, ls, red, sm.data_ptr(), loss.data_ptr(),
             vc.data_ptr())
    h.ce_bwd(sm.data_ptr(), lab.data_ptr(), i64, M, C, ignore_index, ls, red, 0, vc.data_ptr(), dl.data_ptr())
    # the one-call form (one launch when the batch is small) must give the same bits, with and without an upstream value
    sm2, dl2, loss2 = g.empty(M, C), torch.full((M, C), float("nan"), device="cuda"), g.empty(M if red == 2 else 1)
    vc2 = torch.zeros(1, dtype=torch.int32, device="cuda")
    before = h.launch_count()
    h.ce_fwd_bwd(ld.data_ptr(), C, lab.data_ptr(), i64, M, C, ignore_index, ls, red, sm2.data_ptr(), loss2.data_ptr(),
                 vc2.data_ptr(), 0, dl2.data_ptr())
    assert h.launch_count() - before == (1 if (M <= 256 and M * C <= 16384) else 2)
    assert torch.equal(sm, sm2) and torch.equal(loss, loss2) and torch.equal(vc, vc2)
    assert torch.equal(dl, dl2)
    up = torch.full((M if red == 2 else 1,), 0.5, device="cuda")
    h.ce_bwd(sm.data_ptr(), lab.data_ptr(), i64, M, C, ignore_index, ls, red, up.data_ptr(), vc.data_ptr(), dl2.data_ptr())
    dl3 = torch.full((M, C), float("nan"), device="cuda")
    h.ce_fwd_bwd(ld.data_ptr(), C, lab.data_ptr(), i64, M, C, ignore_index, ls, red, sm2.data_ptr(), loss2.data_ptr(),
                 vc2.data_ptr(), up.data_ptr(), dl3.data_ptr())
    assert torch.equal(dl2, dl3)
    h.check_device_status()
    return g.host(loss), g.host(sm), int(vc.item()), g.host(dl)


def test_ce_reference_literals(g):
    c = kat.CE_IGNORE_LS
    logits = f32(c["logits"])
    kw = dict(ignore_index=c["ignore_index"], ls=c["label_smoothing"])
    loss, _, valid, grad = _ce_gpu(g, logits, c["targets"], "mean", **kw)
    assert valid == 2 and np.allclose(loss[0], c["mean_loss"], rtol=1e-5, atol=1e-8)
    assert np.allclose(grad, f32(c["mean_grad"]), rtol=1e-5, atol=1e-7)
    loss, _, _, grad = _ce_gpu(g, logits, c["targets"], "sum", **kw)
    assert np.allclose(loss[0], c["sum_loss"], rtol=1e-5) and np.allclose(grad, f32(c["sum_grad"]), rtol=1e-5, atol=1e-7)
    loss, _, _, grad = _ce_gpu(g, logits, c["targets"], "none", **kw)
    assert np.allclose(loss, f32(c["none_loss"]), rtol=1e-5, atol=1e-8)
    assert np.allclose(grad, f32(c["sum_grad"]), rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("mc", [(64, 10), (256, 10), (3, 3), (1, 1), (100, 33), (1024, 1000), (8192, 1000), (70, 2500), (16, 1000), (200, 80), (256, 64), (128, 129),
                                (5000, 7), (300, 36), (257, 64), (999, 1002), (513, 1024), (40, 2048)], ids=str)
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_ce_vs_oracle(g, oracle, mc, reduction):
    M, C = mc
    rng = np.random.default_rng(M + 31 * C)
    logits = (rng.standard_normal((M, C)) * 3).astype(np.float32)
    labels = rng.integers(0, C, M)
    labels[rng.random(M) < 0.1] = -100
    for ls in (0.0, 0.1):
        loss, sm, valid, grad = _ce_gpu(g, logits, labels, reduction, ls=ls, i64=(ls == 0.0))
        rl, rsm, rvalid = oracle.ce_fwd(logits, labels, reduction, label_smoothing=ls)
        assert valid == rvalid
        # tolerance of the reference's own GPU-vs-CPU check: rtol = atol = 1e-5 (tests/gpu/test_cross_entropy.mojo:94-113)
        assert np.allclose(sm, rsm, rtol=1e-5, atol=1e-7)
        assert np.allclose(loss if reduction == "none" else loss[0], rl, rtol=1e-5, atol=1e-5)
        rgrad = oracle.ce_bwd(rsm, labels, rvalid, reduction, label_smoothing=ls)
        assert np.allclose(grad, rgrad, rtol=1e-5, atol=1e-7)


def test_ce_bad_label_is_reported(g):
    from tenmo_b200 import TenmoError

    logits = np.zeros((4, 3), np.float32)
    with pytest.raises(TenmoError):
        _ce_gpu(g, logits, np.array([0, 1, 5, 2]), "mean")
    g.handle().check_device_status()  # the status word was cleared


@pytest.mark.parametrize("case", kat.SGD, ids=lambda c: c["name"])
def test_sgd_literals(g, case):
    h = g.handle()
    p, v = g.dev(np.ones((2, 2), np.float32)), g.dev(np.zeros((2, 2), np.float32))
    for grad, want in zip(case["grads"], case["expect"]):
        gd = g.dev(np.full((2, 2), grad, np.float32))
        h.sgd_step([p.data_ptr()], [gd.data_ptr()], [v.data_ptr()], [4], case["lr"], case["momentum"], case["wd"])
        assert np.allclose(g.host(p), want, rtol=1e-5, atol=1e-8)


def test_sgd_multi_tensor_bit_exact(g, oracle):
    h = g.handle()
    rng = np.random.default_rng(2)
    sizes = [1, 7, 128, 4097, 100352, 33] * 6  # more tensors than one launch carries
    P = [rng.standard_normal(n).astype(np.float32) for n in sizes]
    G = [rng.standard_normal(n).astype(np.float32) for n in sizes]
    V = [np.zeros(n, np.float32) for n in sizes]
    Pd, Gd, Vd = [g.dev(x) for x in P], [g.dev(x) for x in G], [g.dev(x) for x in V]
    for step in range(3):
        for mom, wd, scale in ((0.9, 0.0, 1.0), (0.9, 1e-4, 0.5), (0.0, 0.01, 1.0)):
            h.sgd_step([t.data_ptr() for t in Pd], [t.data_ptr() for t in Gd], [t.data_ptr() for t in Vd], sizes, 0.01,
                       mom, wd, scale)
            for p, gg, v in zip(P, G, V):
                oracle.sgd_step(p, gg * np.float32(scale), v, 0.01, mom, wd)
    for p, v, pd, vd in zip(P, V, Pd, Vd):
        assert np.array_equal(g.host(pd), p) and np.array_equal(g.host(vd), v)


def test_sgd_with_lo_planes_matches_update_then_split(g, oracle):
    """tenmo_sgd_step_lo_f32: the parameters come out as from tenmo_sgd_step_f32, and the lo plane written along is what
    tenmo_split_lo_f32 gives for the updated weights (only the first lo_numel elements, nothing beyond)."""
    from tenmo_b200 import make_mat

    h = g.handle()
    rng = np.random.default_rng(8)
    shapes = [(96, 64), (33, 20), (5, 4)]          # (rows, cols) of the weight part; a bias of `cols` follows it
    sizes = [r * c + (c + 3) // 4 * 4 for r, c in shapes]
    P = [rng.standard_normal(n).astype(np.float32) for n in sizes]
    G = [rng.standard_normal(n).astype(np.float32) for n in sizes]
    Pd, Gd, Vd = [g.dev(x) for x in P], [g.dev(x) for x in G], [g.dev(np.zeros(n, np.float32)) for n in sizes]
    Pd2, Vd2 = [g.dev(x) for x in P], [g.dev(np.zeros(n, np.float32)) for n in sizes]
    lo = [torch.full((r * c + 8,), 7.0, device="cuda") for r, c in shapes]
    for _ in range(2):
        h.sgd_step([t.data_ptr() for t in Pd], [t.data_ptr() for t in Gd], [t.data_ptr() for t in Vd], sizes, 0.05, 0.9, 1e-3, 0.5,
                   lo_ptrs=[t.data_ptr() for t in lo], lo_numels=[r * c for r, c in shapes])
        h.sgd_step([t.data_ptr() for t in Pd2], [t.data_ptr() for t in Gd], [t.data_ptr() for t in Vd2], sizes, 0.05, 0.9, 1e-3, 0.5)
    torch.cuda.synchronize()
    for (r, c), pd, pd2, l in zip(shapes, Pd, Pd2, lo):
        assert torch.equal(pd, pd2)
        want = g.empty(r * c)
        h.split_lo(make_mat(pd.data_ptr(), (r, c), (c, 1)), r, c, want.data_ptr(), r * c)
        torch.cuda.synchronize()
        assert torch.equal(l[:r * c], want) and bool((l[r * c:] == 7.0).all())
    h.check_device_status()


@pytest.mark.parametrize("case", kat.ACCURACY, ids=lambda c: str(c["correct"]))
def test_accuracy_literals(g, case):
    h = g.handle()
    pred = f32(case["pred"])
    pd, td = g.dev(pred), g.dev(case["target"], np.int64)
    cnt = torch.zeros(1, dtype=torch.int64, device="cuda")
    assert h.accuracy(pd.data_ptr(), pred.shape[1], td.data_ptr(), True, pred.shape[0], pred.shape[1],
                      cnt.data_ptr()) == case["correct"]


@pytest.mark.parametrize("mc", [(1000, 10), (8192, 1000), (5, 70), (3000, 33)], ids=str)
def test_accuracy_vs_oracle(g, oracle, mc):
    M, C = mc
    h = g.handle()
    rng = np.random.default_rng(M)
    pred = np.round(rng.standard_normal((M, C)), 1).astype(np.float32)  # rounded: many exact ties
    tgt = np.argmax(pred, axis=1)
    flip = rng.random(M) < 0.3
    tgt[flip] = rng.integers(0, C, flip.sum())
    pd, td = g.dev(pred), g.dev(tgt, np.int32)
    cnt = torch.zeros(1, dtype=torch.int64, device="cuda")
    assert h.accuracy(pd.data_ptr(), C, td.data_ptr(), False, M, C, cnt.data_ptr()) == oracle.accuracy(pred, tgt)
