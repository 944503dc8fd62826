"""The asynchronously staged (TMA + cp.async) strict-fp32 GEMM kernel (problems of at least one 128 x 128 tile per SM whose operands a
tensor map can describe): bit-identical to the CPU oracle and to the register-staged kernel in all four
transpose layouts, at ragged edges, batched, and through every epilogue option."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

SIMT = 0


@pytest.fixture(scope="module")
def g():
    from tests import gpu_util

    gpu_util.handle()
    return gpu_util


def _views(oracle, A, B, layout):
    Av, Bv = oracle.View.of(A), oracle.View.of(B)
    if layout in ("tn", "tt"):
        Av = oracle.View.of(np.ascontiguousarray(A.T)).t()
    if layout in ("nt", "tt"):
        Bv = oracle.View.of(np.ascontiguousarray(B.T)).t()
    return Av, Bv


def _register_staged(fn):
    """Run fn with the TMA-staged kernel switched off (the library reads the variable at every launch)."""
    os.environ["TENMO_SIMT_TMA"] = "0"
    try:
        return fn()
    finally:
        del os.environ["TENMO_SIMT_TMA"]


# every M, N gives >= 148 tiles of 128 x 128; ragged edges in M, N and K (K = 204: a 12-wide last k-tile)
SHAPES = [(1536, 256, 1664), (1540, 204, 1668), (2048, 64, 1280), (1284, 1000, 2052)]


@pytest.mark.parametrize("mkn", SHAPES, ids=str)
@pytest.mark.parametrize("layout", ["nn", "tn", "nt", "tt"])
def test_bit_exact_vs_oracle_and_register_staged(g, oracle, mkn, layout):
    M, K, N = mkn
    rng = np.random.default_rng(M + 7 * K + 13 * N)
    A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32)
    Av, Bv = _views(oracle, A, B, layout)
    launches = g.handle().launch_count()
    C, _, _ = g.gpu_matmul(Av, Bv, algo=SIMT)
    assert g.handle().launch_count() == launches + 1 and g.handle().gemm_last_kernel() == "gemm_simt_tma_kernel"
    ref = oracle.matmul(Av, Bv, contract_scalar=1, threads=8)
    assert np.array_equal(C, ref), f"max abs diff {np.max(np.abs(C - ref))}"
    C_old, _, _ = _register_staged(lambda: g.gpu_matmul(Av, Bv, algo=SIMT))
    assert g.handle().gemm_last_kernel() == "gemm_simt_kernel" and np.array_equal(C, C_old)
    g.handle().check_device_status()


def test_epilogue_options(g, oracle):
    from tenmo_b200 import make_mat

    h = g.handle()
    M, K, N = 1536, 96, 1664
    rng = np.random.default_rng(9)
    A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32) * 0.1
    bias = rng.standard_normal(N).astype(np.float32)
    Av, Bv = oracle.View.of(A), oracle.View.of(B)
    z = oracle.add_bias(oracle.matmul(A, B, threads=8), bias)
    C, aux, _ = g.gpu_matmul(Av, Bv, algo=SIMT, bias=bias, act=1, want_aux=True)
    out, mask = oracle.relu_fwd(z)
    assert np.array_equal(C, out) and np.array_equal(aux, mask)
    init = rng.standard_normal((M, N), np.float32)
    C, _, _ = g.gpu_matmul(Av, Bv, algo=SIMT, beta=1.0, c_init=init)
    assert np.array_equal(C, init + oracle.matmul(A, B, threads=8))
    # the same with B as a transposed view (scattered 4-byte copies instead of the bulk copy)
    Bt = oracle.View.of(np.ascontiguousarray(B.T)).t()
    C, aux, _ = g.gpu_matmul(Av, Bt, algo=SIMT, bias=bias, act=1, want_aux=True)
    assert np.array_equal(C, out) and np.array_equal(aux, mask)
    # extended options: mask multiply, lo plane of the result, per-row bias as the accumulator's start
    Ad, Bd = g.dev(A), g.dev(B)
    mA, mB = make_mat(Ad.data_ptr(), (M, K), (K, 1)), make_mat(Bd.data_ptr(), (K, N), (N, 1))
    keep = (rng.random((M, N)) < 0.5).astype(np.float32)
    bias_m = rng.standard_normal(M).astype(np.float32)
    C1, c_lo, want_lo = g.empty(M, N), g.empty(M * N), g.empty(M * N)
    h.gemm_ex(M, N, K, mA, mB, C1.data_ptr(), algo=SIMT, mul_mask=g.dev(keep).data_ptr(), c_lo=c_lo.data_ptr(),
              bias_m=g.dev(bias_m).data_ptr())
    torch.cuda.synchronize()
    C_old = g.empty(M, N)
    _register_staged(lambda: h.gemm_ex(M, N, K, mA, mB, C_old.data_ptr(), algo=SIMT, mul_mask=g.dev(keep).data_ptr(),
                                       bias_m=g.dev(bias_m).data_ptr()))
    torch.cuda.synchronize()
    assert np.array_equal(g.host(C1), g.host(C_old))
    assert not g.host(C1)[keep == 0].any()
    h.split_lo(make_mat(C1.data_ptr(), (M, N), (N, 1)), M, N, want_lo.data_ptr(), M * N)
    assert np.array_equal(g.host(c_lo), g.host(want_lo))
    h.check_device_status()


def test_batched_and_broadcast(g, oracle):
    rng = np.random.default_rng(17)
    # (B, M, K) @ (1, K, N): B broadcast, 3 x 8 x 8 = 192 tiles
    A = rng.standard_normal((3, 1024, 80), np.float32)
    B = rng.standard_normal((1, 80, 1024), np.float32)
    C, _, _ = g.gpu_matmul(oracle.View.of(A), oracle.View.of(B), algo=SIMT)
    assert np.array_equal(C, oracle.matmul(A, B, threads=8))
    # attention-shaped with K^T as a stride-permuted view: (B*H, S, D) @ (B*H, D, S)
    Q, Kt = (rng.standard_normal((40, 256, 64), np.float32) * 0.125 for _ in range(2))
    Kv = oracle.View.of(Kt).t()
    S, _, _ = g.gpu_matmul(oracle.View.of(Q), Kv, algo=SIMT)
    assert g.handle().gemm_last_kernel() == "gemm_simt_tma_kernel"
    assert np.array_equal(S, oracle.matmul(oracle.View.of(Q), Kv, threads=8))
    g.handle().check_device_status()
