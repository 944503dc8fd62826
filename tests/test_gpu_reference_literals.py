"""The literals the reference's own tests hold for softmax, ReLU, Sigmoid, axis-0 sums, the bias add, matrix-vector
products and Conv2d (tests/golden/reference_kat.py gives file:line), run through the CUDA entry points of the C ABI.
The same entries pin the CPU oracle in test_oracle_reference_literals.py."""
import numpy as np
import pytest

from tests.golden import reference_kat as kat
from tests.test_oracle_reference_literals import (check_conv_backward, check_conv_forward, close, conv_case_operands, f32,
                                                  softmax_upstream)

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def g():
    from tests import gpu_util

    gpu_util.handle()
    return gpu_util


def gpu_softmax(g, x):
    x = f32(x)
    xd, yd = g.dev(x), g.empty(*x.shape)
    g.handle().softmax_fwd(xd.data_ptr(), x.shape[1], yd.data_ptr(), x.shape[0], x.shape[1])
    return yd


@pytest.mark.parametrize("case", kat.SOFTMAX_FWD, ids=lambda c: c["name"])
def test_softmax_forward_literals(g, oracle, case):
    y = g.host(gpu_softmax(g, [case["x"]]))
    assert close(y[0], case["y"], 1e-6)
    assert close(y, oracle.softmax_fwd(f32([case["x"]])), 2e-7)


@pytest.mark.parametrize("rows", kat.SOFTMAX_ROWS_SUM_TO_ONE, ids=lambda r: f"{len(r)}x{len(r[0])}")
def test_softmax_rows_are_distributions(g, rows):
    y = g.host(gpu_softmax(g, rows))
    assert np.all(np.isfinite(y)) and np.all((y >= 0) & (y <= 1))
    assert np.all(np.abs(y.sum(axis=1, dtype=np.float64) - 1) < 1e-5)


@pytest.mark.parametrize("case", kat.SOFTMAX_BWD, ids=lambda c: c["name"])
def test_softmax_backward_literals(g, oracle, case):
    yd = gpu_softmax(g, case["x"])
    y = g.host(yd)
    up = softmax_upstream(case, y)
    dx = g.empty(*y.shape)
    upd = g.dev(up)
    g.handle().softmax_bwd(yd.data_ptr(), upd.data_ptr(), dx.data_ptr(), y.shape[0], y.shape[1])
    assert close(g.host(dx), case["dx"], 2e-7)
    assert close(g.host(dx), oracle.softmax_bwd(up, y), 1e-7)


@pytest.mark.parametrize("case", kat.RELU, ids=lambda c: str(len(np.ravel(c["x"]))))
def test_relu_literals(g, case):
    x = f32(case["x"])
    xd, out, mask, dx = g.dev(x), g.empty(*x.shape), g.empty(*x.shape), g.empty(*x.shape)
    h = g.handle()
    h.relu_fwd(xd.data_ptr(), out.data_ptr(), mask.data_ptr(), x.size)
    ones = g.dev(np.ones_like(x))
    h.relu_bwd(ones.data_ptr(), mask.data_ptr(), dx.data_ptr(), x.size)
    assert np.array_equal(g.host(out), f32(case["y"])) and np.array_equal(g.host(mask), f32(case["mask"]))
    assert np.array_equal(g.host(dx), f32(case["mask"]))
    # the same ReLU as the epilogue of a GEMM with the identity: out = relu(x . I), aux = mask
    x2 = x.reshape(-1, x.shape[-1]) if x.ndim > 1 else x.reshape(1, -1)
    from oracle import ref

    c, aux, _ = g.gpu_matmul(ref.View.of(x2), ref.View.of(np.eye(x2.shape[1], dtype=np.float32)), act=1, want_aux=True)
    assert np.array_equal(c.reshape(x.shape), f32(case["y"])) and np.array_equal(aux.reshape(x.shape), f32(case["mask"]))


@pytest.mark.parametrize("case", kat.SIGMOID, ids=lambda c: str(len(np.ravel(c["x"]))))
def test_sigmoid_literals(g, oracle, case):
    x = f32(case["x"])
    xd, y, dx = g.dev(x), g.empty(*x.shape), g.empty(*x.shape)
    h = g.handle()
    h.sigmoid_fwd(xd.data_ptr(), y.data_ptr(), x.size)
    ones = g.dev(np.ones_like(x))
    h.sigmoid_bwd(ones.data_ptr(), y.data_ptr(), dx.data_ptr(), x.size)
    s = f32(case["y"])
    assert close(g.host(y), s, 1e-6) and close(g.host(dx), s * (1 - s), 1e-6)
    assert close(g.host(y), oracle.sigmoid_fwd(x), 2e-7)


@pytest.mark.parametrize("case", kat.SUM_AXIS0, ids=lambda c: str(len(c["out"])))
def test_sum_axis0_literals(g, case):
    x = f32(case["x"])
    out = g.empty(x.shape[1])
    xd = g.dev(x)
    g.handle().colsum(xd.data_ptr(), x.shape[0], x.shape[1], x.shape[1], out.data_ptr())
    assert np.array_equal(g.host(out), f32(case["out"]))


def test_bias_add_broadcast_literals(g):
    c = kat.ADD_BROADCAST
    x, b = f32(c["x"]), f32(c["bias"])
    out, db = g.empty(*x.shape), g.empty(b.size)
    h = g.handle()
    xd, bd, ones = g.dev(x), g.dev(b), g.dev(np.ones_like(x))   # named: a temporary's memory may be reused by the next one
    h.add_bias(xd.data_ptr(), bd.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1])
    h.colsum(ones.data_ptr(), x.shape[0], x.shape[1], x.shape[1], db.data_ptr())
    assert np.array_equal(g.host(out), f32(c["out"])) and np.array_equal(g.host(db), f32(c["dbias"]))


# ---- Conv2d ------------------------------------------------------------------------------------------------------
def gpu_conv(g, x, k, b, stride, dilation, pad, grad=None):
    from tenmo_b200.cnn import Conv2d

    N, Cin, H, W = x.shape
    Cout, _, kh, kw = k.shape
    assert kh == kw
    conv = Conv2d(g.handle(), N, Cin, H, W, Cout, kh, stride, dilation, pad, relu=False)
    bias = b if b is not None else np.zeros(Cout, np.float32)
    xd, kd, bd = g.dev(x), g.dev(k), g.dev(bias)
    out = g.host(conv.forward(xd, kd, bd))
    if grad is None:
        return out
    dW, db = g.empty(*k.shape), g.empty(Cout)
    dx = conv.backward(g.dev(grad(out)), kd, dW, db)
    return out, g.host(dx), g.host(dW), g.host(db)


@pytest.mark.parametrize("case", kat.CONV_FWD, ids=lambda c: c["name"])
def test_conv_forward_literals(g, oracle, case):
    x, k, b = conv_case_operands(case)
    out = gpu_conv(g, x, k, b, case["stride"], case["dilation"], case["pad"])
    check_conv_forward(case, out)
    assert np.array_equal(out, oracle.conv2d_fwd(x, k, b, stride=case["stride"], dilation=case["dilation"], pad=case["pad"]))


def test_conv_batch_literals(g):
    c = kat.CONV_BATCH
    x = np.empty(c["x_shape"], np.float32)
    for b in range(x.shape[0]):
        x[b] = b + 1
    out = gpu_conv(g, x, np.ones(c["k_shape"], np.float32), None, 1, 1, 0)
    assert [float(out[b, 0, 0, 0]) for b in range(4)] == c["expect_first"]


@pytest.mark.parametrize("case", kat.CONV_BWD, ids=lambda c: c["name"])
def test_conv_backward_literals(g, case):
    x, k, b = conv_case_operands(case)
    out, dx, dk, db = gpu_conv(g, x, k, b, case["stride"], case["dilation"], case["pad"], grad=np.ones_like)
    if "out_shape" in case:
        assert out.shape == tuple(case["out_shape"])
    check_conv_backward(case, dx, dk, db)  # small integers: every summation order gives the same bits


# ---- matrix @ vector, vector @ matrix through the HBM-bound kernels -------------------------------------------------
def gpu_gemv(g, M, v, beta=0.0, y0=None, transposed_storage=False):
    """y = M . v through tenmo_gemv_f32; with transposed_storage the matrix is handed over as a stride view of its
    transpose (column-major), which takes the other kernel."""
    from tenmo_b200 import make_mat

    M, v = f32(M), f32(v)
    m, k = M.shape
    if transposed_storage:
        Md = g.dev(np.ascontiguousarray(M.T))
        mat = make_mat(Md.data_ptr(), (m, k), (1, m))
    else:
        Md = g.dev(M)
        mat = make_mat(Md.data_ptr(), (m, k), (k, 1))
    y = g.dev(y0) if y0 is not None else g.empty(m)
    vd = g.dev(v)
    g.handle().gemv(m, k, mat, vd.data_ptr(), 1, y.data_ptr(), beta)
    return g.host(y)


def gpu_vecmat(g, v, M, transposed_storage=False):
    from tenmo_b200 import make_mat

    M, v = f32(M), f32(v)
    k, n = M.shape
    if transposed_storage:
        Md = g.dev(np.ascontiguousarray(M.T))
        mat = make_mat(Md.data_ptr(), (k, n), (1, k))
    else:
        Md = g.dev(M)
        mat = make_mat(Md.data_ptr(), (k, n), (n, 1))
    y = g.empty(n)
    vd = g.dev(v)
    g.handle().vecmat(k, n, vd.data_ptr(), 1, mat, y.data_ptr())
    return g.host(y)


@pytest.mark.parametrize("case", kat.MV, ids=lambda c: c["name"])
@pytest.mark.parametrize("tr", [False, True], ids=["row_major", "col_major"])
def test_mv_literals(g, case, tr):
    M, v = f32(case["M"]), f32(case["v"])
    flat = M.reshape(-1, *M.shape[-2:])
    out = np.stack([gpu_gemv(g, Mb, v, transposed_storage=tr) for Mb in flat]).reshape(np.shape(case["out"]))
    assert np.array_equal(out, f32(case["out"]))
    # dv = sum over the batch of M_b^T . ones (matrixvector.mojo:15-201): the vecmat kernel with beta = 1 semantics
    dv = sum(gpu_vecmat(g, np.ones(Mb.shape[0], np.float32), Mb, transposed_storage=tr) for Mb in flat)
    assert np.array_equal(dv, f32(case["dv"]))


@pytest.mark.parametrize("case", kat.VM, ids=lambda c: c["name"])
@pytest.mark.parametrize("tr", [False, True], ids=["row_major", "col_major"])
def test_vm_literals(g, case, tr):
    v, M = f32(case["v"]), f32(case["M"])
    assert np.array_equal(gpu_vecmat(g, v, M, transposed_storage=tr), f32(case["out"]))
    assert np.array_equal(gpu_gemv(g, M, np.ones(M.shape[1], np.float32), transposed_storage=tr), f32(case["dv"]))


@pytest.mark.parametrize("mk", [(1, 1), (3, 5), (37, 301), (513, 64), (1000, 1027), (4096, 4096), (130, 70000)], ids=str)
@pytest.mark.parametrize("tr", [False, True], ids=["row_major", "col_major"])
def test_gemv_vecmat_vs_oracle(g, oracle, mk, tr):
    m, k = mk
    rng = np.random.default_rng(m * 7 + k)
    M = rng.standard_normal((m, k)).astype(np.float32)
    v, u = rng.standard_normal(k).astype(np.float32), rng.standard_normal(m).astype(np.float32)
    y0 = rng.standard_normal(m).astype(np.float32)
    # the oracle's chain is k-ascending, the kernels' is not: same sum to rounding, bar 1e-5 of sum |a||x|
    want = oracle.mv(M, v).astype(np.float64)
    bound = np.abs(M).astype(np.float64) @ np.abs(v).astype(np.float64) + 1e-30
    assert np.max(np.abs(gpu_gemv(g, M, v, transposed_storage=tr) - want) / bound) <= 1e-5
    acc = gpu_gemv(g, M, v, beta=1.0, y0=y0, transposed_storage=tr)
    assert np.max(np.abs(acc - (want + y0)) / (bound + np.abs(y0))) <= 1e-5
    want_t = oracle.vm(u, M).astype(np.float64)
    bound_t = np.abs(u).astype(np.float64) @ np.abs(M).astype(np.float64) + 1e-30
    assert np.max(np.abs(gpu_vecmat(g, u, M, transposed_storage=tr) - want_t) / bound_t) <= 1e-5
    # run to run the bits are the same (slab order, not arrival order)
    assert np.array_equal(gpu_vecmat(g, u, M, transposed_storage=tr), gpu_vecmat(g, u, M, transposed_storage=tr))
    g.handle().check_device_status()


def test_gemv_rejects_a_matrix_without_a_unit_stride(g):
    from tenmo_b200 import TenmoError, make_mat

    A = g.dev(np.zeros((8, 16), np.float32))
    with pytest.raises(TenmoError):
        xv, yv = g.empty(4), g.empty(4)
        g.handle().gemv(4, 4, make_mat(A.data_ptr(), (4, 4), (32, 2)), xv.data_ptr(), 1, yv.data_ptr())


# ---- the reference's own C-ABI seam (tests/test_blas.mojo) and dot (tests/test_dot.mojo) ---------------------------------
from tests.test_oracle_reference_literals import seam_views  # noqa: E402


@pytest.fixture(scope="module")
def tm():
    import tenmo_b200.tensor as tensor

    tensor.handle()
    tensor.set_gemm_algo("simt")
    return tensor


@pytest.mark.parametrize("case", kat.BLAS_SEAM, ids=lambda c: c["name"])
def test_blas_seam_literals_through_the_c_abi(g, oracle, case):
    """blas.matmul(A, B, transpose_A, transpose_B) becomes tenmo_gemm_f32 on stride views of the stored operands."""
    _, _, Av, Bv = seam_views(oracle, case)
    C, _, _ = g.gpu_matmul(Av, Bv)
    g.handle().check_device_status()
    assert np.array_equal(C, oracle.matmul(Av, Bv))
    if "C" in case:
        assert np.array_equal(C, f32(case["C"]))
    if "shape" in case:
        assert C.shape == case["shape"] and C[0, 0] == np.float32(case["C00"])


@pytest.mark.parametrize("case", [c for c in kat.BLAS_SEAM if "dA" in c], ids=lambda c: c["name"])
def test_blas_seam_gradients_through_the_host_mirror(tm, case):
    A = tm.Tensor.d2(case["A"], requires_grad=True)
    B = tm.Tensor.d2(case["B"], requires_grad=True)
    left = A.transpose() if case["ta"] else A
    right = B.transpose() if case["tb"] else B
    left.matmul(right).sum().backward()
    assert A.grad().all_close(f32(case["dA"])) and B.grad().all_close(f32(case["dB"]))


@pytest.mark.parametrize("case", kat.BLAS_SEAM_ONES, ids=lambda c: f"{c['M']}x{c['K']}x{c['N']}")
def test_blas_seam_ones(g, oracle, case):
    A, B = np.ones((case["M"], case["K"]), np.float32), np.ones((case["K"], case["N"]), np.float32)
    C, _, _ = g.gpu_matmul(oracle.View.of(A), oracle.View.of(B))
    assert C.shape == (case["M"], case["N"]) and np.all(C == np.float32(case["value"]))


def test_blas_seam_finite_difference(g, oracle):
    c = kat.BLAS_SEAM_FD
    A, B = f32(c["A"]), f32(c["B"])
    plus, minus = A.copy(), A.copy()
    plus[0, 0] += np.float32(c["eps"])
    minus[0, 0] -= np.float32(c["eps"])
    V = oracle.View
    lp = np.float32(g.gpu_matmul(V.of(plus), V.of(B))[0].sum(dtype=np.float32))
    lm = np.float32(g.gpu_matmul(V.of(minus), V.of(B))[0].sum(dtype=np.float32))
    analytic = g.gpu_matmul(V.of(np.ones((2, 2), np.float32)), V.of(B).t())[0][0, 0]
    assert analytic == np.float32(c["dA00"]) and abs(float(analytic) - float((lp - lm) / np.float32(2 * c["eps"]))) < c["tol"]


@pytest.mark.parametrize("case", kat.DOT, ids=lambda c: str(c["value"]))
def test_dot_literals(tm, case):
    a = tm.Tensor.d1(case["a"], requires_grad=True)
    b = tm.Tensor.d1(case["b"], requires_grad=True)
    d = a.matmul(b)
    assert d.item() == case["value"]
    d.backward()
    assert a.grad().all_close(f32(case["b"])) and b.grad().all_close(f32(case["a"]))   # d(a.b)/da = b, /db = a


def test_dot_gradients_accumulate_like_the_chained_case(tm):
    # tests/test_dot.mojo:148-160 uses loss = d + d; two backward passes of d accumulate the same 2 b and 2 a
    c = kat.DOT_CHAINED
    a = tm.Tensor.d1(c["a"], requires_grad=True)
    b = tm.Tensor.d1(c["b"], requires_grad=True)
    for _ in range(2):
        a.matmul(b).backward()
    assert a.grad().all_close(f32(c["da"])) and b.grad().all_close(f32(c["db"]))
