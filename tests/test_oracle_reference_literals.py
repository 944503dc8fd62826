"""Pins the oracle's softmax, ReLU, Sigmoid, column-sum, bias-add, matrix-vector and Conv2d restatements on the
literals the reference's own tests hold (tests/golden/reference_kat.py gives file:line for each).  CPU only."""
import numpy as np
import pytest

from tests.golden import reference_kat as kat


def f32(x):
    return np.asarray(x, dtype=np.float32)


def close(a, b, atol):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return a.shape == b.shape and bool(np.all(np.abs(a - b) <= atol))


# ---- softmax ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", kat.SOFTMAX_FWD, ids=lambda c: c["name"])
@pytest.mark.parametrize("simd", [8, 16])
def test_softmax_forward_literals(oracle, case, simd):
    y = oracle.softmax_fwd(f32([case["x"]]), simd_width=simd)
    assert close(y[0], case["y"], 1e-6)  # the reference asserts atol 1e-5


@pytest.mark.parametrize("rows", kat.SOFTMAX_ROWS_SUM_TO_ONE, ids=lambda r: f"{len(r)}x{len(r[0])}")
def test_softmax_rows_are_distributions(oracle, rows):
    y = oracle.softmax_fwd(f32(rows))
    assert np.all((y >= 0) & (y <= 1)) and np.all(np.abs(y.sum(axis=1, dtype=np.float64) - 1) < 1e-5)
    assert np.all(np.isfinite(y))


def softmax_upstream(case, y):
    """Gradient reaching the softmax node: 2 (y - t) / numel for the mse loss, the weights for sum(y * w)."""
    if "mse_target" in case:
        return (2.0 * (y.astype(np.float64) - np.asarray(case["mse_target"], np.float64)) / y.size).astype(np.float32)
    return f32(case["weights"])


@pytest.mark.parametrize("case", kat.SOFTMAX_BWD, ids=lambda c: c["name"])
def test_softmax_backward_literals(oracle, case):
    x = f32(case["x"])
    y = oracle.softmax_fwd(x)
    dx = oracle.softmax_bwd(softmax_upstream(case, y), y)
    assert close(dx, case["dx"], 2e-7)  # float64 literals against an fp32 restatement


def test_softmax_matches_float64_formula(oracle):
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((33, 517)) * 3).astype(np.float32)
    g = rng.standard_normal((33, 517)).astype(np.float32)
    y = oracle.softmax_fwd(x)
    x64 = x.astype(np.float64)
    e = np.exp(x64 - x64.max(axis=1, keepdims=True))
    y64 = e / e.sum(axis=1, keepdims=True)
    assert np.max(np.abs(y - y64) / y64) < 5e-6
    d64 = y64 * (g - (g * y64).sum(axis=1, keepdims=True))
    assert np.max(np.abs(oracle.softmax_bwd(g, y) - d64)) < 1e-6


# ---- ReLU / Sigmoid / sums / bias add -------------------------------------------------------------------------
@pytest.mark.parametrize("case", kat.RELU, ids=lambda c: str(len(np.ravel(c["x"]))))
def test_relu_literals(oracle, case):
    x = f32(case["x"])
    out, mask = oracle.relu_fwd(x)
    assert np.array_equal(out, f32(case["y"])) and np.array_equal(mask, f32(case["mask"]))
    # loss = sum(relu(x)): the gradient is ones * mask
    assert np.array_equal(oracle.relu_bwd(np.ones_like(x), mask), f32(case["mask"]))


@pytest.mark.parametrize("case", kat.SIGMOID, ids=lambda c: str(len(np.ravel(c["x"]))))
def test_sigmoid_literals(oracle, case):
    x = f32(case["x"])
    y = oracle.sigmoid_fwd(x)
    assert close(y, case["y"], 1e-6)
    s = f32(case["y"])
    assert close(oracle.sigmoid_bwd(np.ones_like(x), y), s * (1 - s), 1e-6)


@pytest.mark.parametrize("case", kat.SUM_AXIS0, ids=lambda c: str(len(c["out"])))
def test_sum_axis0_literals(oracle, case):
    assert np.array_equal(oracle.colsum(f32(case["x"])), f32(case["out"]))


def test_bias_add_broadcast_literals(oracle):
    c = kat.ADD_BROADCAST
    assert np.array_equal(oracle.add_bias(f32(c["x"]), f32(c["bias"])), f32(c["out"]))
    # BroadcastBackward (broadcast.mojo:66-88): the bias gradient is the upstream gradient summed over the rows
    assert np.array_equal(oracle.colsum(np.ones_like(f32(c["x"]))), f32(c["dbias"]))


# ---- matrix @ vector, vector @ matrix ----------------------------------------------------------------------------
@pytest.mark.parametrize("case", kat.MV, ids=lambda c: c["name"])
@pytest.mark.parametrize("contract", [0, 1])
def test_mv_literals(oracle, case, contract):
    M, v = f32(case["M"]), f32(case["v"])
    out = oracle.mv(M, v, contract)
    assert np.array_equal(out, f32(case["out"]))
    # MatrixVectorMulNdBackward (matrixvector.mojo:15-201): dM = g (outer) v, dv = sum over batch of M^T g, g = ones
    g = np.ones_like(out)
    dM = g[..., None] * v
    dv = sum(oracle.vm(gb, Mb, contract) for gb, Mb in zip(g.reshape(-1, g.shape[-1]), M.reshape(-1, *M.shape[-2:])))
    assert np.array_equal(dM, f32(case["dM"])) and np.array_equal(dv, f32(case["dv"]))
    # the same numbers through the GEMM restatement with a unit dimension (what the CUDA library runs for small sizes)
    flat = M.reshape(-1, *M.shape[-2:])
    as_gemm = np.stack([oracle.matmul(Mb, v.reshape(-1, 1), contract_scalar=contract)[:, 0] for Mb in flat])
    assert np.array_equal(as_gemm.reshape(out.shape), out)


@pytest.mark.parametrize("case", kat.VM, ids=lambda c: c["name"])
def test_vm_literals(oracle, case):
    v, M = f32(case["v"]), f32(case["M"])
    out = oracle.vm(v, M)
    assert np.array_equal(out, f32(case["out"]))
    g = np.ones_like(out)
    assert np.array_equal(oracle.mv(M, g), f32(case["dv"]))           # dv = M g
    assert np.array_equal(v[:, None] * g[None, :], f32(case["dM"]))  # dM = v (outer) g
    assert np.array_equal(oracle.matmul(v.reshape(1, -1), M)[0], out)


def test_mv_vm_are_single_ascending_chains(oracle):
    rng = np.random.default_rng(9)
    M, v = rng.standard_normal((37, 301)).astype(np.float32), rng.standard_normal(301).astype(np.float32)
    want = np.zeros(37, np.float32)
    for j in range(301):
        want = np.float32(M[:, j].astype(np.float64) * np.float64(v[j]) + want.astype(np.float64))
    got = oracle.mv(M, v, 1)
    assert np.mean(got == want) > 0.9 and np.max(np.abs(got - want)) <= np.max(np.abs(want)) * 2.0 ** -22
    assert np.array_equal(oracle.vm(v, M.T.copy(), 1), got)


# ---- Conv2d ----------------------------------------------------------------------------------------------------
def conv_operand(spec, shape):
    if isinstance(spec, list):
        return f32(spec)
    if spec == "arange1":
        return np.arange(1, int(np.prod(shape)) + 1, dtype=np.float32).reshape(shape)
    if spec == "filter_index_plus_1":
        k = np.empty(shape, np.float32)
        for i in range(shape[0]):
            k[i] = i + 1
        return k
    return np.full(shape, spec, np.float32)


def conv_case_operands(case):
    k = conv_operand(case["k"], case.get("k_shape"))
    x = conv_operand(case["x"], case["x_shape"])
    b = f32(case["bias"]) if case["bias"] is not None else None
    return x, k, b


def check_conv_forward(case, out):
    if "full" in case:
        assert np.array_equal(out, f32(case["full"]))
    if "out_shape" in case:
        assert out.shape == tuple(case["out_shape"])
    if "fill" in case:
        assert np.all(out == np.float32(case["fill"]))
    if "channel_fill" in case:
        for c, val in enumerate(case["channel_fill"]):
            assert np.all(out[:, c] == np.float32(val))


@pytest.mark.parametrize("case", kat.CONV_FWD, ids=lambda c: c["name"])
def test_conv_forward_literals(oracle, case):
    x, k, b = conv_case_operands(case)
    check_conv_forward(case, oracle.conv2d_fwd(x, k, b, stride=case["stride"], dilation=case["dilation"], pad=case["pad"]))


def test_conv_batch_literals(oracle):
    c = kat.CONV_BATCH
    x = np.empty(c["x_shape"], np.float32)
    for b in range(x.shape[0]):
        x[b] = b + 1
    out = oracle.conv2d_fwd(x, np.ones(c["k_shape"], np.float32), None)
    assert out.shape == (4, 1, 2, 2) and [float(out[b, 0, 0, 0]) for b in range(4)] == c["expect_first"]


def check_conv_backward(case, dx, dk, db):
    assert np.array_equal(db, f32(case["dbias"]))
    if "dx" in case:
        assert np.array_equal(dx, f32(case["dx"]))
    if "dk" in case:
        assert np.array_equal(dk, f32(case["dk"]))
    if "dk_plane" in case:
        for o in range(dk.shape[0]):
            for i in range(dk.shape[1]):
                assert np.array_equal(dk[o, i], f32(case["dk_plane"]))


@pytest.mark.parametrize("case", kat.CONV_BWD, ids=lambda c: c["name"])
def test_conv_backward_literals(oracle, case):
    x, k, b = conv_case_operands(case)
    kw = dict(stride=case["stride"], dilation=case["dilation"], pad=case["pad"])
    out = oracle.conv2d_fwd(x, k, b, **kw)
    if "out_shape" in case:
        assert out.shape == tuple(case["out_shape"])
    dx, dk, db = oracle.conv2d_bwd(np.ones_like(out), x, k, **kw)
    check_conv_backward(case, dx, dk, db)


# ---- the reference's own C-ABI seam (BLASHandle.matmul) and dot -------------------------------------------------------
def seam_views(oracle, case):
    """Operands of a BLAS-seam case as the views the call multiplies: a transpose flag is a stride view, as in the
    backward GEMMs."""
    A, B = f32(case["A"]), f32(case["B"])
    Av, Bv = oracle.View.of(A), oracle.View.of(B)
    return A, B, (Av.t() if case["ta"] else Av), (Bv.t() if case["tb"] else Bv)


def seam_gradients(oracle, case):
    """Gradients of sum(op(A) @ op(B)) with respect to the STORED A and B (matmul.mojo:24-54 applied to the views)."""
    A, B, Av, Bv = seam_views(oracle, case)
    M, N = Av.shape[-2], Bv.shape[-1]
    G = oracle.View.of(np.ones((M, N), np.float32))
    d_opA = oracle.matmul(G, Bv.t())   # gradient of the view op(A)
    d_opB = oracle.matmul(Av.t(), G)
    return (d_opA.T if case["ta"] else d_opA), (d_opB.T if case["tb"] else d_opB)


@pytest.mark.parametrize("case", kat.BLAS_SEAM, ids=lambda c: c["name"])
def test_blas_seam_literals(oracle, case):
    _, _, Av, Bv = seam_views(oracle, case)
    C = oracle.matmul(Av, Bv)
    if "C" in case:
        assert np.array_equal(C, f32(case["C"]))
    if "shape" in case:
        assert C.shape == case["shape"] and C[0, 0] == np.float32(case["C00"])
    if "dA" in case:
        dA, dB = seam_gradients(oracle, case)
        assert np.array_equal(dA, f32(case["dA"])) and np.array_equal(dB, f32(case["dB"]))


@pytest.mark.parametrize("case", kat.BLAS_SEAM_ONES, ids=lambda c: f"{c['M']}x{c['K']}x{c['N']}")
def test_blas_seam_ones(oracle, case):
    C = oracle.matmul(np.ones((case["M"], case["K"]), np.float32), np.ones((case["K"], case["N"]), np.float32))
    assert C.shape == (case["M"], case["N"]) and np.all(C == np.float32(case["value"]))


def test_blas_seam_finite_difference(oracle):
    c = kat.BLAS_SEAM_FD
    A, B = f32(c["A"]), f32(c["B"])
    plus, minus = A.copy(), A.copy()
    plus[0, 0] += np.float32(c["eps"])
    minus[0, 0] -= np.float32(c["eps"])
    fd = (np.float32(oracle.matmul(plus, B).sum(dtype=np.float32)) - np.float32(oracle.matmul(minus, B).sum(dtype=np.float32))) / np.float32(2 * c["eps"])
    analytic = oracle.matmul(np.ones((2, 2), np.float32), oracle.View.of(B).t())[0, 0]
    assert analytic == np.float32(c["dA00"]) and abs(float(analytic) - float(fd)) < c["tol"]


@pytest.mark.parametrize("case", kat.DOT, ids=lambda c: str(c["value"]))
def test_dot_literals(oracle, case):
    a, b = f32(case["a"]), f32(case["b"])
    d = oracle.matmul(a[None, :], b[:, None])   # dot as the (1,k) @ (k,1) product the GPU path runs
    assert d.shape == (1, 1) and d[0, 0] == np.float32(case["value"])
