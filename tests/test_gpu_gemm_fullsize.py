"""The GEMMs at the full sizes of the benchmark configurations (square 4096 and 8192, skinny 65536 x 784 x 128),
forward and both backward products with transposed views, checked through properties that do not need the whole CPU
result:

  * sampled rows: every output element is an independent k-chain, so a handful of rows of the full-size result must
    equal the oracle's result for just those rows -- bit for bit on the strict-fp32 kernel, within 1e-4 of
    sum_k |a||b| on the 3xTF32 kernel;
  * checksum: the row sums of C against A.(B.1) in float64;
  * scaling by two is exact in binary floating point: (2A).B == 2(A.B) bit for bit, on both kernels;
  * the same call twice gives the same bits.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

SIMT, TC = 0, 1
TOL = {SIMT: 2e-5, TC: 1e-4}  # checksum / sampled-row bar, relative to sum |a||b|


@pytest.fixture(scope="module")
def g():
    from tests import gpu_util

    gpu_util.handle()
    return gpu_util


def _gemm(h, algo, M, N, K, a_mat, b_mat):
    out = torch.empty(M, N, dtype=torch.float32, device="cuda")
    h.gemm(M, N, K, a_mat, b_mat, out.data_ptr(), algo=algo)
    return out


@pytest.mark.parametrize("mkn", [(4096, 4096, 4096), (8192, 8192, 8192), (65536, 784, 128)], ids=str)
@pytest.mark.parametrize("algo", [SIMT, TC], ids=["simt", "3xtf32"])
def test_forward_backward_fullsize(g, oracle, mkn, algo):
    from tenmo_b200 import make_mat

    h = g.handle()
    M, K, N = mkn
    gen = torch.Generator(device="cuda").manual_seed(M + K + N + algo)
    A = torch.randn(M, K, generator=gen, device="cuda")
    B = torch.randn(K, N, generator=gen, device="cuda")
    dC = torch.randn(M, N, generator=gen, device="cuda")
    mA, mB, mdC = (make_mat(t.data_ptr(), tuple(t.shape), (t.shape[1], 1)) for t in (A, B, dC))
    mBt = make_mat(B.data_ptr(), (N, K), (1, N))   # B^T as a stride view
    mAt = make_mat(A.data_ptr(), (K, M), (1, K))   # A^T as a stride view

    C = _gemm(h, algo, M, N, K, mA, mB)            # C  = A . B
    assert h.gemm_last_kernel() == {SIMT: "gemm_simt_tma_kernel", TC: "gemm_tc_kernel"}[algo]
    dA = _gemm(h, algo, M, K, N, mdC, mBt)         # dA = dC . B^T
    dB = _gemm(h, algo, K, N, M, mAt, mdC)         # dB = A^T . dC
    torch.cuda.synchronize()
    h.check_device_status()

    Ah, Bh, dCh = A.cpu().numpy(), B.cpu().numpy(), dC.cpu().numpy()
    rng = np.random.default_rng(7)

    def check_rows(got, left_rows, right_view, rows):
        """got[rows] against the oracle's product of the sampled left rows with the whole right operand."""
        ref = oracle.matmul(left_rows, right_view, threads=8)
        res = got[torch.as_tensor(rows, device="cuda")].cpu().numpy()
        if algo == SIMT:
            assert np.array_equal(res, ref)
        else:
            scale = np.abs(left_rows.numpy()).astype(np.float64) @ np.abs(right_view.numpy()).astype(np.float64)
            assert np.max(np.abs(res.astype(np.float64) - ref) / np.maximum(scale, 1e-30)) <= TOL[TC]

    V = oracle.View
    rows = np.sort(rng.choice(M, 8, replace=False))
    check_rows(C, V.of(np.ascontiguousarray(Ah[rows])), V.of(Bh), rows)
    check_rows(dA, V.of(np.ascontiguousarray(dCh[rows])), V.of(Bh).t(), rows)
    krows = np.sort(rng.choice(K, 8, replace=False))
    check_rows(dB, V.of(np.ascontiguousarray(Ah[:, krows])).t(), V.of(dCh), krows)

    # checksum of the whole result: rowsum(C) = A . (B . 1), in float64, against the bar scaled by |A| . (|B| . 1)
    rs = C.double().sum(dim=1).cpu().numpy()
    want = Ah.astype(np.float64) @ Bh.astype(np.float64).sum(axis=1)
    scale = np.abs(Ah).astype(np.float64) @ np.abs(Bh).astype(np.float64).sum(axis=1)
    assert np.max(np.abs(rs - want) / scale) <= TOL[algo]

    # exact scaling and repeatability
    A2 = A * 2.0
    C2 = _gemm(h, algo, M, N, K, make_mat(A2.data_ptr(), (M, K), (K, 1)), mB)
    assert torch.equal(C2, C * 2.0)
    assert torch.equal(_gemm(h, algo, M, N, K, mA, mB), C)
    h.check_device_status()
