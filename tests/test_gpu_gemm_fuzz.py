"""Seeded random sweeps of the GEMM entry point: shapes (ragged and aligned, small and one-tile-per-SM large), all four
transpose layouts as stride views, bias / ReLU (+ mask) / beta = 1 in the epilogue.  Strict fp32 must match the oracle
bit for bit whichever kernel the library picks; 3xTF32 must stay within 1e-4 of sum |a||b| (split-K shapes included)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def g():
    from tests import gpu_util

    gpu_util.handle()
    return gpu_util


def _case(rng, oracle, M, N, K):
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    Av, Bv = oracle.View.of(A), oracle.View.of(B)
    if rng.random() < 0.5:
        Av = oracle.View.of(np.ascontiguousarray(A.T)).t()
    if rng.random() < 0.5:
        Bv = oracle.View.of(np.ascontiguousarray(B.T)).t()
    kw, bias, init = {}, None, None
    if rng.random() < 0.4:
        bias = rng.standard_normal(N).astype(np.float32)
        kw["bias"] = bias
    kw["act"] = int(rng.integers(0, 2))
    if kw["act"] == 1 and rng.random() < 0.5:
        kw["want_aux"] = True
    if rng.random() < 0.3:
        init = rng.standard_normal((M, N)).astype(np.float32)
        kw.update(beta=1.0, c_init=init)
    return A, B, Av, Bv, kw, bias, init


@pytest.mark.parametrize("seed", [11, 12])
def test_strict_fp32_random_shapes_bit_exact(g, oracle, seed):
    rng = np.random.default_rng(seed)
    kernels = set()
    for it in range(160):
        if it % 8 == 0:   # enough 128 x 128 tiles for every SM: the TMA-staged kernel when the strides allow it
            M, N, K = int(rng.integers(410, 550)) * 4, int(rng.integers(410, 550)) * 4, int(rng.integers(16, 40)) * 4
        else:
            M, N, K = (int(rng.integers(1, 300)) for _ in range(3))
        A, B, Av, Bv, kw, bias, init = _case(rng, oracle, M, N, K)
        C, aux, _ = g.gpu_matmul(Av, Bv, algo=0, **kw)
        kernels.add(g.handle().gemm_last_kernel())
        z = oracle.matmul(Av, Bv, contract_scalar=1, threads=8)
        if bias is not None:
            z = oracle.add_bias(z, bias)
        if kw["act"] == 1:
            z, mask = oracle.relu_fwd(z)
            if kw.get("want_aux"):
                assert np.array_equal(aux, mask), (M, N, K)
        if init is not None:
            z = init + z
        assert np.array_equal(C, z), (M, N, K, Av.strides, Bv.strides, sorted(kw))
    assert kernels == {"gemm_simt_kernel", "gemm_simt_tma_kernel"}
    g.handle().check_device_status()


def test_3xtf32_random_shapes_within_bar(g, oracle):
    rng = np.random.default_rng(21)
    for it in range(120):
        M, N, K = (int(rng.integers(1, 180)) * 4 for _ in range(3))
        if it % 6 == 0:   # small output, long k: the split-K path
            M, N, K = int(rng.integers(1, 40)) * 4, int(rng.integers(1, 40)) * 4, int(rng.integers(1024, 3000)) * 4
        A, B, Av, Bv, kw, bias, init = _case(rng, oracle, M, N, K)
        C, _, _ = g.gpu_matmul(Av, Bv, algo=1, **kw)
        z = A.astype(np.float64) @ B.astype(np.float64)
        if bias is not None:
            z = z + bias
        pre = z.copy()
        if kw["act"] == 1:
            z = np.maximum(z, 0)
        if init is not None:
            z = init + z
        scale = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64) + 1e-30
        err = np.abs(C.astype(np.float64) - z) / scale
        if kw["act"] == 1:
            err[np.abs(pre) / scale < 1e-4] = 0  # a pre-activation within rounding of zero may land on either side
        assert np.max(err) <= 1e-4, (M, N, K, Av.strides, Bv.strides, sorted(kw))
    g.handle().check_device_status()
