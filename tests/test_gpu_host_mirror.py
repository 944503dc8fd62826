"""The host-side mirror (Tensor / Linear / CrossEntropyLoss / SGD / Accuracy) over the C ABI, written the
way the reference's own tests are: build tensors, call matmul / backward / step, compare with the
literals the reference holds or with the CPU oracle on the same seeded inputs."""
import numpy as np
import pytest

from tests.golden import reference_kat as kat

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def tm():
    import tenmo_b200.crossentropy as ce
    import tenmo_b200.net as net
    import tenmo_b200.optim as optim
    import tenmo_b200.tensor as tensor

    tensor.handle()
    tensor.set_gemm_algo("simt")

    class NS:
        Tensor, NDBuffer = tensor.Tensor, tensor.NDBuffer
        Linear, ReLU, Sigmoid, Sequential = net.Linear, net.ReLU, net.Sigmoid, net.Sequential
        CrossEntropyLoss, Accuracy, SGD = ce.CrossEntropyLoss, ce.Accuracy, optim.SGD
        set_gemm_algo = staticmethod(tensor.set_gemm_algo)

    return NS


def validate_matmul_2d_grads(A, B, C):
    """tests/test_mm2d.mojo:39-100: after C.backward(ones), dA == ones.B^T and dB == A^T.ones."""
    a, b = A.numpy(), B.numpy()
    ones = np.ones(C.shape(), np.float32)
    assert A.grad().all_close(ones @ b.T) and B.grad().all_close(a.T @ ones)


@pytest.mark.parametrize("case", kat.MM2D, ids=lambda c: c["name"])
def test_matmul_2d_with_grads(tm, case):
    A = tm.Tensor.d2(case["A"], requires_grad=True)
    B = tm.Tensor.d2(case["B"], requires_grad=True)
    C = A.matmul(B)
    assert C.all_close(np.asarray(case["C"], np.float32))
    C.backward()
    validate_matmul_2d_grads(A, B, C)


@pytest.mark.parametrize("case", kat.MM2D_VIEWS, ids=lambda c: c["name"])
def test_matmul_2d_views(tm, case):
    base = tm.Tensor.d1(case["A_base"])
    A1 = base.view(case["A_shape"], case["A_strides"], case["A_offset"])
    C = A1.matmul(tm.Tensor.d2(case["B"]))
    assert C.all_close(np.asarray(case["C"], np.float32))


@pytest.mark.parametrize("case", kat.MMND_GRADS, ids=lambda c: c["name"])
def test_matmul_nd_with_grads(tm, case):
    A = tm.Tensor.d3(case["A"], requires_grad=True)
    B = tm.Tensor.d3(case["B"], requires_grad=True)
    C = A.matmul(B)
    if "C" in case:
        assert C.all_close(np.asarray(case["C"], np.float32), atol=1e-5)
    loss = C.sum()
    loss.backward()
    assert A.grad().all_close(np.asarray(case["dA"], np.float32))
    assert B.grad().all_close(np.asarray(case["dB"], np.float32))


def test_matrix_vector_and_vector_matrix(tm):
    # tests/test_mv.mojo:14-45: M[m,k] @ v[k]
    M = tm.Tensor.d2([[1, 2, 3], [4, 5, 6]], requires_grad=True)
    v = tm.Tensor.d1([1, 2, 3], requires_grad=True)
    r = M.matmul(v, mode="mv")
    r.sum().backward()
    assert r.all_close(np.asarray([14, 32], np.float32))
    assert M.grad().all_close(np.asarray([[1, 2, 3], [1, 2, 3]], np.float32))
    assert v.grad().all_close(np.asarray([5, 7, 9], np.float32))
    # tests/test_mv.mojo:48-82: M[m,k] @ v[batch,k] -> [batch,m], gradients summed over the batch for M
    M = tm.Tensor.d2([[1, 2], [3, 4]], requires_grad=True)
    v = tm.Tensor.d2([[1, 0], [0, 1]], requires_grad=True)
    r = M.matmul(v, mode="mv")
    r.sum().backward()
    assert r.all_close(np.asarray([[1, 3], [2, 4]], np.float32))
    assert M.grad().all_close(np.ones((2, 2), np.float32))
    assert v.grad().all_close(np.asarray([[4, 6], [4, 6]], np.float32))
    # tests/test_vm.mojo:14-48: v[k] @ M[k,n]
    v = tm.Tensor.d1([1, 2, 3], requires_grad=True)
    M = tm.Tensor.d2([[1, 2], [3, 4], [5, 6]], requires_grad=True)
    r = v.matmul(M)  # rank-based classification picks vm
    r.sum().backward()
    assert r.all_close(np.asarray([22, 28], np.float32))
    assert v.grad().all_close(np.asarray([3, 7, 11], np.float32))
    assert M.grad().all_close(np.asarray([[1, 1], [2, 2], [3, 3]], np.float32))
    # dot
    a = tm.Tensor.d1([1, 2, 3], requires_grad=True)
    b = tm.Tensor.d1([4, 5, 6], requires_grad=True)
    d = a.matmul(b)
    d.backward()
    assert d.item() == 32.0 and a.grad().all_close(b.numpy()) and b.grad().all_close(a.numpy())


def test_gradient_accumulation_over_two_backward_passes(tm):
    # Gradbox accumulates across backward calls until zero_grad (tests/test_matmul.mojo: gradient accumulation)
    A = tm.Tensor.d2([[1, 2], [3, 4]], requires_grad=True)
    B = tm.Tensor.d2([[5, 6], [7, 8]], requires_grad=True)
    for _ in range(2):
        A.matmul(B).backward()
    assert A.grad().all_close(2 * (np.ones((2, 2), np.float32) @ np.asarray([[5, 6], [7, 8]], np.float32).T))
    A.zero_grad()
    assert not A.grad().numpy().any()


def test_matmul_errors_are_host_errors(tm):
    A, B = tm.Tensor.zeros(2, 3), tm.Tensor.zeros(4, 5)
    with pytest.raises(RuntimeError, match="incompatible shapes"):
        A.matmul(B)
    with pytest.raises(RuntimeError, match="not broadcastable"):
        tm.Tensor.zeros(2, 2, 3).matmul(tm.Tensor.zeros(3, 3, 4))
    lin = tm.Linear(4, 2)
    with pytest.raises(RuntimeError, match="input dim mismatch"):
        lin(tm.Tensor.zeros(3, 5))


def test_cross_entropy_reference_literals(tm):
    c = kat.CE_IGNORE_LS
    targets = tm.Tensor.labels(c["targets"])
    for red, want_loss, want_grad in (("mean", c["mean_loss"], c["mean_grad"]), ("sum", c["sum_loss"], c["sum_grad"]),
                                      ("none", c["none_loss"], c["sum_grad"])):
        logits = tm.Tensor.d2(c["logits"], requires_grad=True)
        crit = tm.CrossEntropyLoss(reduction=red, ignore_index=c["ignore_index"], label_smoothing=c["label_smoothing"])
        loss = crit(logits, targets)
        assert loss.all_close(np.asarray(want_loss, np.float32))
        loss.backward()
        assert logits.grad().all_close(np.asarray(want_grad, np.float32), atol=1e-7)


def test_cross_entropy_rejects_bad_labels(tm):
    from tenmo_b200 import TenmoError

    logits = tm.Tensor.zeros(2, 3, requires_grad=True)
    with pytest.raises(TenmoError):
        tm.CrossEntropyLoss()(logits, tm.Tensor.labels([0, 7]))


@pytest.mark.parametrize("case", kat.SGD, ids=lambda c: c["name"])
def test_sgd_literals(tm, case):
    param = tm.Tensor.ones(2, 2, requires_grad=True)
    opt = tm.SGD([param], lr=case["lr"], momentum=case["momentum"], weight_decay=case["wd"])
    for g, want in zip(case["grads"], case["expect"]):
        param.seed_grad(g)
        opt.step()
        assert param.all_close(np.full((2, 2), want, np.float32))
        opt.zero_grad()
        assert not param.grad().numpy().any()


@pytest.mark.parametrize("case", kat.ACCURACY, ids=lambda c: str(c["correct"]))
def test_accuracy_literals(tm, case):
    assert tm.Accuracy.compute(tm.Tensor.d2(case["pred"]), tm.Tensor.labels(case["target"])) == case["correct"]


def _build_mlp(tm, dims, Ws, act="relu"):
    layers = []
    for i in range(len(dims) - 1):
        lin = tm.Linear(dims[i], dims[i + 1])
        lin.weight = tm.Tensor.from_numpy(Ws[i], requires_grad=True)
        lin.bias = tm.Tensor.from_numpy(np.zeros(dims[i + 1], np.float32), requires_grad=True)
        layers.append(lin)
        if i + 2 < len(dims):
            layers.append(tm.ReLU() if act == "relu" else tm.Sigmoid())
    return tm.Sequential(*layers)


def test_mnist_shaped_mlp_training_is_bit_consistent_with_the_oracle(tm, oracle):
    """Config 1 shapes (784-128-32-10, batch 64, Xavier-uniform, zero bias, SGD lr 0.01 momentum 0.9), synthetic
    pixels and labels from a seed.  Free-running for 30 steps: the strict-fp32 GEMM, the sequential-order
    small reductions and the unfused SGD arithmetic make logits, losses and parameters IDENTICAL to the
    oracle's except for exp/log (libm vs CUDA), so argmax / accuracy must be bit-identical every step and
    the parameters must stay within 1e-6."""
    rng = np.random.default_rng(2024)
    dims = [784, 128, 32, 10]
    Ws = [rng.uniform(-1, 1, (dims[i], dims[i + 1])).astype(np.float32) * np.float32(np.sqrt(6.0 / (dims[i] + dims[i + 1])))
          for i in range(3)]
    model = _build_mlp(tm, dims, Ws)
    ref = oracle.MLP(Ws, [np.zeros(d, np.float32) for d in dims[1:]])
    opt = tm.SGD(model.parameters(), lr=0.01, momentum=0.9)
    crit = tm.CrossEntropyLoss()
    for step in range(30):
        X = rng.uniform(0, 1, (64, 784)).astype(np.float32)
        y = rng.integers(0, 10, 64)
        xs, ys = tm.Tensor.from_numpy(X), tm.Tensor.labels(y)
        opt.zero_grad()
        logits = model(xs)
        loss = crit(logits, ys)
        loss.backward()
        opt.step()
        r_loss, r_logits = ref.step(X, y, lr=0.01, momentum=0.9)
        got = logits.numpy()
        assert np.array_equal(np.argmax(got, 1), np.argmax(r_logits, 1)), f"argmax differs at step {step}"
        assert tm.Accuracy.compute(logits, ys) == oracle.accuracy(r_logits, y)
        assert np.max(np.abs(got - r_logits)) <= 1e-5 * max(1.0, np.max(np.abs(r_logits)))
        assert abs(loss.item() - r_loss) <= 1e-5
    for p, w in zip([m.weight for m in model.modules if isinstance(m, tm.Linear)], ref.W):
        assert np.max(np.abs(p.numpy() - w)) <= 1e-6


def test_first_step_of_the_mlp_is_bit_identical(tm, oracle):
    """Before exp/log differences can feed back (first forward), the logits are bit-for-bit the oracle's."""
    rng = np.random.default_rng(5)
    dims = [784, 128, 32, 10]
    Ws = [rng.uniform(-0.08, 0.08, (dims[i], dims[i + 1])).astype(np.float32) for i in range(3)]
    model = _build_mlp(tm, dims, Ws)
    ref = oracle.MLP(Ws, [np.zeros(d, np.float32) for d in dims[1:]])
    X = rng.uniform(0, 1, (64, 784)).astype(np.float32)
    y = rng.integers(0, 10, 64)
    logits = model(tm.Tensor.from_numpy(X))
    _, r_logits = ref.step(X, y, update=False)
    assert np.array_equal(logits.numpy(), r_logits)


def test_sigmoid_mlp_and_3xtf32_path(tm, oracle):
    """Sigmoid epilogue neighbours + the tensor-core GEMM through the same host API (tolerance 1e-4)."""
    rng = np.random.default_rng(6)
    X = rng.standard_normal((256, 512)).astype(np.float32)
    W = (rng.standard_normal((512, 256)) * 0.05).astype(np.float32)
    tm.set_gemm_algo("3xtf32")
    try:
        xs = tm.Tensor.from_numpy(X, requires_grad=True)
        ws = tm.Tensor.from_numpy(W, requires_grad=True)
        out = xs.matmul(ws).sigmoid()
        out.sum().backward()
    finally:
        tm.set_gemm_algo("simt")
    z = oracle.matmul(X, W, threads=4)
    yref = oracle.sigmoid_fwd(z)
    assert np.allclose(out.numpy(), yref, rtol=1e-4, atol=1e-5)
    dz = oracle.sigmoid_bwd(np.ones_like(yref), yref)
    assert np.allclose(ws.grad().numpy(), oracle.matmul(oracle.View.of(X).t(), oracle.View.of(dz)), rtol=1e-4, atol=1e-3)
    assert np.allclose(xs.grad().numpy(), oracle.matmul(oracle.View.of(dz), oracle.View.of(W).t()), rtol=1e-4, atol=1e-3)


def test_interior_broadcast_batch_gradients(tm):
    """(2,1,m,k) @ (1,3,k,n): each operand is broadcast along an INTERIOR batch axis; the backward pass sums the batched
    gradients back over that axis (sum_over_broadcasted_axes, sum_mean_reduction.mojo:184-211)."""
    rng = np.random.default_rng(17)
    a = rng.standard_normal((2, 1, 5, 4)).astype(np.float32)
    b = rng.standard_normal((1, 3, 4, 6)).astype(np.float32)
    A, B = tm.Tensor.from_numpy(a, requires_grad=True), tm.Tensor.from_numpy(b, requires_grad=True)
    C = A.matmul(B)
    assert C.shape() == (2, 3, 5, 6) and C.all_close(a @ b, rtol=1e-5, atol=1e-6)
    up = rng.standard_normal((2, 3, 5, 6)).astype(np.float32)
    C.backward(tm.Tensor.from_numpy(up))
    dA = (up @ np.swapaxes(b, -1, -2)).sum(axis=1, keepdims=True)
    dB = (np.swapaxes(a, -1, -2) @ up).sum(axis=0, keepdims=True)
    assert A.grad().shape() == a.shape and A.grad().all_close(dA, rtol=1e-5, atol=1e-5)
    assert B.grad().shape() == b.shape and B.grad().all_close(dB, rtol=1e-5, atol=1e-5)


def test_sum_backward_keeps_the_upstream_on_the_device(tm):
    A = tm.Tensor.d2([[1, 2], [3, 4]], requires_grad=True)
    s = A.sum()
    s.backward(3.0)
    assert A.grad().all_close(np.full((2, 2), 3.0, np.float32))
    assert s.gradbox is None or not s.gradbox.numpy().any()   # zeroed like every other backward (retain_graph=False)
