"""Parity of the tcgen05 3xTF32 GEMM with the CPU oracle.

Bar: max relative error <= 1e-4, measured per element against the oracle's fp32 result and normalised by
sum_k |a_ik||b_kj| (the scale every backward-stable GEMM error bound is stated in); the fp64 product is
checked at the same bar so that the oracle's own rounding does not mask anything.  In practice the kernel
lands near 1e-6.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

TC = 1
TOL = 1e-4


@pytest.fixture(scope="module")
def g():
    from tests import gpu_util

    gpu_util.handle()
    return gpu_util


def rel_err(C, ref, absA, absB):
    scale = absA.astype(np.float64) @ absB.astype(np.float64)
    return float(np.max(np.abs(C.astype(np.float64) - ref) / np.maximum(scale, 1e-30)))


def layouts(oracle, A, B, layout):
    Av, Bv = oracle.View.of(A), oracle.View.of(B)
    if layout in ("tn", "tt"):
        Av = oracle.View.of(np.ascontiguousarray(A.T)).t()
    if layout in ("nt", "tt"):
        Bv = oracle.View.of(np.ascontiguousarray(B.T)).t()
    return Av, Bv


SHAPES = [(128, 32, 256), (128, 64, 128), (256, 128, 512), (384, 96, 640), (200, 100, 300), (1000, 260, 132),
          (129, 36, 260), (512, 784, 128), (2048, 512, 1024), (640, 2052, 388),
          (2048, 96, 2048), (1024, 160, 1000)]  # 128 x 256 tiles; the 1000-class layer on 128 x 64 tiles


@pytest.mark.parametrize("mkn", SHAPES, ids=str)
@pytest.mark.parametrize("layout", ["nn", "nt", "tn", "tt"])
def test_tc_matches_oracle(g, oracle, mkn, layout):
    M, K, N = mkn
    if layout in ("tn", "tt") and M % 4:
        pytest.skip("transposed A needs a 16-byte aligned leading stride")
    rng = np.random.default_rng(M * 31 + K * 7 + N)
    A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32)
    Av, Bv = layouts(oracle, A, B, layout)
    C, _, _ = g.gpu_matmul(Av, Bv, algo=TC)
    assert g.handle().gemm_last_algo() == TC
    g.handle().check_device_status()
    ref32 = oracle.matmul(Av, Bv, threads=4)
    e32 = rel_err(C, ref32.astype(np.float64), np.abs(A), np.abs(B))
    e64 = rel_err(C, A.astype(np.float64) @ B.astype(np.float64), np.abs(A), np.abs(B))
    assert e32 <= TOL and e64 <= TOL, (e32, e64)
    assert e64 <= 4e-6, f"3xTF32 should be close to fp32 accuracy, got {e64}"


def test_tc_epilogue_and_accumulate(g, oracle):
    M, K, N = 384, 200, 512
    rng = np.random.default_rng(9)
    A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32) * 0.1
    bias = rng.standard_normal(N).astype(np.float32)
    Av, Bv = oracle.View.of(A), oracle.View.of(B)
    z = oracle.add_bias(oracle.matmul(A, B), bias)
    C, aux, _ = g.gpu_matmul(Av, Bv, algo=TC, bias=bias, act=1, want_aux=True)
    out, mask = oracle.relu_fwd(z)
    near_zero = np.abs(z) < 1e-4  # the sign of a pre-activation within rounding of 0 is not defined
    assert np.allclose(C, out, rtol=1e-5, atol=1e-4)
    assert np.array_equal(aux[~near_zero], mask[~near_zero])
    C, _, _ = g.gpu_matmul(Av, Bv, algo=TC, bias=bias, act=2)
    assert np.allclose(C, oracle.sigmoid_fwd(z), rtol=1e-5, atol=1e-5)
    init = rng.standard_normal((M, N), np.float32)
    C, _, cs = g.gpu_matmul(Av.t(), oracle.View.of(init), algo=TC, beta=1.0, c_init=np.ones((K, N), np.float32),
                            colsum=True)
    ref = 1.0 + A.T.astype(np.float64) @ init.astype(np.float64)
    assert rel_err(C - 1.0, ref - 1.0, np.abs(A.T), np.abs(init)) <= TOL
    assert np.allclose(cs, 0.0 + oracle.colsum(init), rtol=1e-5, atol=1e-4)


def test_tc_batched(g, oracle):
    rng = np.random.default_rng(4)
    # (B,M,K) @ (1,K,N): broadcast right operand
    A = rng.standard_normal((6, 256, 64), np.float32)
    B = rng.standard_normal((1, 64, 128), np.float32)
    C, _, _ = g.gpu_matmul(oracle.View.of(A), oracle.View.of(B), algo=TC)
    ref = A.astype(np.float64) @ B.astype(np.float64)
    assert np.max(np.abs(C - ref)) <= TOL * 64 * 4
    # attention-shaped with a stride-permuted K^T, then P @ V
    BH, S, D = 8, 256, 64
    Q, Kt, V = (rng.standard_normal((BH, S, D), np.float32) * 0.125 for _ in range(3))
    Kv = oracle.View.of(Kt).t()
    scores, _, _ = g.gpu_matmul(oracle.View.of(Q), Kv, algo=TC)
    ref = Q.astype(np.float64) @ np.swapaxes(Kt, 1, 2).astype(np.float64)
    assert np.max(np.abs(scores - ref)) <= 1e-5
    assert np.max(np.abs(scores - oracle.matmul(oracle.View.of(Q), Kv, threads=4))) <= 1e-5
    ctx, _, _ = g.gpu_matmul(oracle.View.of(scores), oracle.View.of(V), algo=TC)
    assert np.max(np.abs(ctx - scores.astype(np.float64) @ V.astype(np.float64))) <= 1e-4
    # 4-D batch that collapses to one stride
    A4 = rng.standard_normal((2, 3, 128, 32), np.float32)
    B4 = rng.standard_normal((2, 3, 32, 64), np.float32)
    C4, _, _ = g.gpu_matmul(oracle.View.of(A4), oracle.View.of(B4), algo=TC)
    assert np.max(np.abs(C4 - A4.astype(np.float64) @ B4.astype(np.float64))) <= 1e-4


def test_tc_refuses_what_it_cannot_take_and_auto_falls_back(g, oracle):
    from tenmo_b200 import TenmoError

    rng = np.random.default_rng(1)
    A, B = rng.standard_normal((128, 30), np.float32), rng.standard_normal((30, 64), np.float32)  # ld 30: rows not 16-byte aligned
    with pytest.raises(TenmoError) as e:
        g.gpu_matmul(oracle.View.of(A), oracle.View.of(B), algo=TC)
    assert e.value.status == -3
    C, _, _ = g.gpu_matmul(oracle.View.of(A), oracle.View.of(B), algo=-1)  # auto -> SIMT on the GPU, never the CPU
    assert g.handle().gemm_last_algo() == 0 and np.array_equal(C, oracle.matmul(A, B))
    # auto picks the tensor-core kernel for a large aligned problem
    A, B = rng.standard_normal((1024, 1024), np.float32), rng.standard_normal((1024, 1024), np.float32)
    C, _, _ = g.gpu_matmul(oracle.View.of(A), oracle.View.of(B), algo=-1)
    assert g.handle().gemm_last_algo() == 1
    assert rel_err(C, A.astype(np.float64) @ B.astype(np.float64), np.abs(A), np.abs(B)) <= TOL


@pytest.mark.parametrize("algo", [0, 1], ids=["simt", "3xtf32"])
def test_gemm_ex_lo_planes_and_mask(g, oracle, algo):
    """tenmo_gemm_f32_ex: supplied lo planes give the same bits as the in-call split, c_lo is the lo plane of
    what was stored, mul_mask multiplies the result (fused ReLU backward)."""
    from tenmo_b200 import make_mat

    h = g.handle()
    M, K, N = 256, 192, 320
    rng = np.random.default_rng(12)
    A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32)
    mask = (rng.random((M, N)) < 0.5).astype(np.float32)
    Ad, Bd, Md = g.dev(A), g.dev(B), g.dev(mask)
    mA, mB = make_mat(Ad.data_ptr(), (M, K), (K, 1)), make_mat(Bd.data_ptr(), (K, N), (N, 1))
    a_lo, b_lo = g.empty(M * K), g.empty(K * N)
    h.split_lo(mA, M, K, a_lo.data_ptr(), M * K)
    h.split_lo(mB, K, N, b_lo.data_ptr(), K * N)
    # lo = x - trunc_tf32(x), rounded to tf32: exact check on the host
    hi = (A.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)
    lo_ref = A - hi
    got_lo = g.host(a_lo).reshape(M, K)
    assert np.max(np.abs(got_lo - lo_ref)) <= 2.0 ** -11 * np.max(np.abs(lo_ref)) and not (got_lo.view(np.uint32) & 0x1FFF).any()
    C0, C1, c_lo = g.empty(M, N), g.empty(M, N), g.empty(M * N)
    h.gemm_ex(M, N, K, mA, mB, C0.data_ptr(), algo=algo, mul_mask=Md.data_ptr())
    h.gemm_ex(M, N, K, mA, mB, C1.data_ptr(), algo=algo, mul_mask=Md.data_ptr(), a_lo=a_lo.data_ptr(), b_lo=b_lo.data_ptr(),
              c_lo=c_lo.data_ptr())
    torch.cuda.synchronize()
    c0, c1 = g.host(C0), g.host(C1)
    assert np.array_equal(c0, c1)
    ref = oracle.matmul(A, B, threads=4) * mask
    if algo == 0:
        assert np.array_equal(c1, ref)
    else:
        assert rel_err(c1, ref.astype(np.float64), np.abs(A), np.abs(B)) <= TOL
    assert not c1[mask == 0].any()
    want_lo = g.empty(M * N)
    h.split_lo(make_mat(C1.data_ptr(), (M, N), (N, 1)), M, N, want_lo.data_ptr(), M * N)
    assert np.array_equal(g.host(c_lo), g.host(want_lo))
    # the transposed view of a matrix shares its storage's lo plane (what the backward GEMMs rely on)
    Ct = g.empty(K, N)
    G = g.dev(rng.standard_normal((M, N), np.float32))
    g_lo = g.empty(M * N)
    mG = make_mat(G.data_ptr(), (M, N), (N, 1))
    h.split_lo(mG, M, N, g_lo.data_ptr(), M * N)
    h.gemm_ex(K, N, M, make_mat(Ad.data_ptr(), (K, M), (1, K)), mG, Ct.data_ptr(), algo=algo, a_lo=a_lo.data_ptr(),
              b_lo=g_lo.data_ptr())
    torch.cuda.synchronize()
    want = A.T.astype(np.float64) @ g.host(G).astype(np.float64)
    assert rel_err(g.host(Ct), want, np.abs(A.T), np.abs(g.host(G))) <= TOL


def test_tc_run_to_run_identical(g, oracle):
    rng = np.random.default_rng(8)
    A, B = rng.standard_normal((512, 512), np.float32), rng.standard_normal((512, 768), np.float32)
    C1, _, _ = g.gpu_matmul(oracle.View.of(A), oracle.View.of(B), algo=TC)
    C2, _, _ = g.gpu_matmul(oracle.View.of(A), oracle.View.of(B), algo=TC)
    assert np.array_equal(C1, C2)


@pytest.mark.parametrize("mkn", [(784, 65536, 128), (200, 8192, 96), (128, 16384, 256)], ids=str)
@pytest.mark.parametrize("layout", ["nn", "tn"])
def test_tc_split_k_for_small_outputs_with_long_k(g, oracle, mkn, layout):
    """A small output with a very long k (dW of a narrow layer at a large batch) is cut along k into the batches of one
    batched launch plus an ordered sum: same bar as the unsplit kernel, beta = 1 honoured, repeatable."""
    M, K, N = mkn
    rng = np.random.default_rng(M + N)
    A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32)
    Av, Bv = layouts(oracle, A, B, layout)
    launches = g.handle().launch_count()
    C, _, _ = g.gpu_matmul(Av, Bv, algo=TC)
    assert g.handle().launch_count() - launches == 4  # two lo-plane splits, the batched GEMM, the ordered sum
    ref64 = A.astype(np.float64) @ B.astype(np.float64)
    assert rel_err(C, ref64, np.abs(A), np.abs(B)) <= TOL
    init = rng.standard_normal((M, N), np.float32)
    C1, _, _ = g.gpu_matmul(Av, Bv, algo=TC, beta=1.0, c_init=init)
    assert rel_err(C1, init.astype(np.float64) + ref64, np.abs(A), np.abs(B)) <= TOL
    C2, _, _ = g.gpu_matmul(Av, Bv, algo=TC)
    assert np.array_equal(C, C2)
    g.handle().check_device_status()


# (M, K, N): tile counts that leave the last wave of a 148-SM machine partly empty in different ways -- less than one wave
# (pieces shorter than a tile), 3.46 waves (the last 1.46 cut into pieces), 1.73 waves (only the last .73), ragged
# edges in m, n and k, a batch
STREAM_K_SHAPES = [(1024, 2048, 1024), (1024, 4096, 4096), (2048, 2048, 2048), (4096, 2048, 4096), (2048, 4096, 4096),
                   (1000, 2052, 1000), (3, 640, 2048, 512)]


@pytest.mark.parametrize("mkn", STREAM_K_SHAPES, ids=str)
@pytest.mark.parametrize("layout", ["nn", "nt", "tn"])
def test_tc_stream_k_tail(g, oracle, mkn, layout, monkeypatch):
    """The stream-K tail (pieces of the k-range of the last tiles, partial accumulators added by the piece that ends a
    tile): same bar as whole tiles, epilogue options honoured by the completing piece, repeatable bit for bit, and the
    flags are back to zero after every launch (three launches in a row with different inputs)."""
    monkeypatch.setenv("TENMO_TC_PAIR", "0")   # the single-CTA kernel: the pair form has no stream-K tail
    batch = 1
    if len(mkn) == 4:
        batch, M, K, N = mkn
        if layout != "nn":
            pytest.skip("the batched case is run once")
    else:
        M, K, N = mkn
    h = g.handle()
    if h.device_info()["sm_count"] != 148:
        pytest.skip("shapes chosen for 148 SMs")
    rng = np.random.default_rng(M + K + N)
    shape_a, shape_b = ((batch, M, K), (batch, K, N)) if batch > 1 else ((M, K), (K, N))
    A, B = rng.standard_normal(shape_a, np.float32), rng.standard_normal(shape_b, np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    if batch > 1:
        Av, Bv = oracle.View.of(A), oracle.View.of(B)
    else:
        Av, Bv = layouts(oracle, A, B, layout)
    ref64 = A.astype(np.float64) @ B.astype(np.float64)
    absA, absB = np.abs(A), np.abs(B)

    def bar(C, want):
        scale = np.matmul(absA.astype(np.float64), absB.astype(np.float64)) + 1e-30
        return float(np.max(np.abs(C.astype(np.float64) - want) / scale))

    C, _, _ = g.gpu_matmul(Av, Bv, algo=TC)
    assert h.gemm_last_kernel() == "gemm_tc_kernel" and h.gemm_last_stream_k() == 148
    assert bar(C, ref64) <= TOL
    C2, _, _ = g.gpu_matmul(Av, Bv, algo=TC)
    assert np.array_equal(C, C2)
    monkeypatch.setenv("TENMO_TC_STREAMK", "0")
    C0, _, _ = g.gpu_matmul(Av, Bv, algo=TC)
    assert h.gemm_last_stream_k() == 0
    monkeypatch.delenv("TENMO_TC_STREAMK")
    assert bar(C0, ref64) <= TOL and bar(C, C0.astype(np.float64)) <= TOL
    if batch == 1:
        # bias + ReLU + mask + accumulate, applied once, by the completing piece
        init = rng.standard_normal((M, N), np.float32)
        C3, aux, _ = g.gpu_matmul(Av, Bv, algo=TC, bias=bias, act=1, want_aux=True, beta=1.0, c_init=init)
        assert h.gemm_last_stream_k() == 148
        pre = ref64 + bias
        want = init + np.maximum(pre, 0)
        scale = absA.astype(np.float64) @ absB.astype(np.float64) + 1e-30
        err = np.abs(C3.astype(np.float64) - want) / scale
        near0 = np.abs(pre) / scale < 1e-4
        err[near0] = 0
        assert float(err.max()) <= TOL
        assert np.array_equal(aux[~near0], (pre > 0).astype(np.float32)[~near0])
    # other inputs straight after: nothing of the previous launch may be picked up
    A2 = rng.standard_normal(shape_a, np.float32)
    absA = np.abs(A2)
    Av2 = oracle.View.of(A2) if (batch > 1 or layout[0] == "n") else oracle.View.of(np.ascontiguousarray(A2.T)).t()
    C4, _, _ = g.gpu_matmul(Av2, Bv, algo=TC)
    assert bar(C4, A2.astype(np.float64) @ B.astype(np.float64)) <= TOL
    h.check_device_status()


def test_tc_stream_k_replays_in_a_graph(g):
    """A captured launch with a stream-K tail is replayed with new inputs: the kernel re-arms its own counters, so each
    replay equals the eager call on the same inputs bit for bit."""
    from tenmo_b200 import make_mat

    h = g.handle()
    if h.device_info()["sm_count"] != 148:
        pytest.skip("shape chosen for 148 SMs")
    M, K, N = 1024, 2048, 1024
    gen = torch.Generator(device="cuda").manual_seed(5)
    A, B = torch.randn(M, K, generator=gen, device="cuda"), torch.randn(K, N, generator=gen, device="cuda")
    C, Ce = g.empty(M, N), g.empty(M, N)
    mA, mB = make_mat(A.data_ptr(), (M, K), (K, 1)), make_mat(B.data_ptr(), (K, N), (N, 1))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    try:
        with torch.cuda.stream(side):
            h.set_stream(side.cuda_stream)
            h.gemm(M, N, K, mA, mB, C.data_ptr(), algo=TC)  # grows the workspace before the capture
            assert h.gemm_last_stream_k() == 148
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                h.gemm(M, N, K, mA, mB, C.data_ptr(), algo=TC)
        torch.cuda.current_stream().wait_stream(side)
    finally:
        h.set_stream(torch.cuda.current_stream().cuda_stream)
    for _ in range(3):
        A.copy_(torch.randn(M, K, generator=gen, device="cuda"))
        C.fill_(float("nan"))
        graph.replay()
        h.gemm(M, N, K, mA, mB, Ce.data_ptr(), algo=TC)
        torch.cuda.synchronize()
        assert torch.equal(C, Ce)
        ref = A.double() @ B.double()
        scale = A.double().abs() @ B.double().abs()
        assert float(((C.double() - ref).abs() / scale).max()) <= TOL
    h.check_device_status()


# ---- the CTA-pair form (tcgen05.mma.cta_group::2: two SMs share a 256 x 256 tile) ------------------------------------
@pytest.fixture
def force_pair(monkeypatch):
    monkeypatch.setenv("TENMO_TC_PAIR", "1")   # read by the library at every launch
    monkeypatch.setenv("TENMO_TC_BN", "256")   # the pair form exists for 256-wide tiles; small products would pick narrower ones


PAIR_SHAPES = [(256, 64, 256), (512, 96, 512), (1000, 260, 388), (129, 36, 260), (640, 2052, 516), (2048, 512, 1024),
               (300, 4096, 257 * 4)]  # whole tiles, ragged rows / columns, a row tile whose second CTA is empty, long k


@pytest.mark.parametrize("mkn", PAIR_SHAPES, ids=str)
@pytest.mark.parametrize("layout", ["nn", "nt", "tn", "tt"])
def test_tc_pair_matches_oracle(g, oracle, force_pair, mkn, layout):
    M, K, N = mkn
    if layout in ("tn", "tt") and M % 4:
        pytest.skip("transposed A needs a 16-byte aligned leading stride")
    rng = np.random.default_rng(M * 13 + K * 5 + N)
    A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32)
    Av, Bv = layouts(oracle, A, B, layout)
    C, _, _ = g.gpu_matmul(Av, Bv, algo=TC)
    h = g.handle()
    assert h.gemm_last_algo() == TC and h.gemm_last_pair() and h.gemm_last_stream_k() == 0   # too few k-blocks to cut here
    h.check_device_status()
    e32 = rel_err(C, oracle.matmul(Av, Bv, threads=4).astype(np.float64), np.abs(A), np.abs(B))
    e64 = rel_err(C, A.astype(np.float64) @ B.astype(np.float64), np.abs(A), np.abs(B))
    assert e32 <= TOL and e64 <= 4e-6, (e32, e64)
    # the pair form and the single-CTA form add the same products in the same order inside a tile: identical bits
    import os

    os.environ["TENMO_TC_PAIR"] = "0"
    C1, _, _ = g.gpu_matmul(Av, Bv, algo=TC)
    assert not h.gemm_last_pair()
    os.environ["TENMO_TC_STREAMK"] = "0"
    C1, _, _ = g.gpu_matmul(Av, Bv, algo=TC)
    del os.environ["TENMO_TC_STREAMK"]
    assert np.array_equal(C, C1)


def test_tc_pair_epilogue_batches_and_planes(g, oracle, force_pair):
    """Bias, ReLU with its mask, the accumulate, a row bias, a multiplier and the result's lo plane through the pair
    kernel; a broadcast-batched product; the same call twice gives the same bits."""
    import torch as T

    from tenmo_b200 import make_mat

    h = g.handle()
    M, K, N = 520, 200, 772
    rng = np.random.default_rng(19)
    A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32) * 0.1
    bias = rng.standard_normal(N).astype(np.float32)
    Av, Bv = oracle.View.of(A), oracle.View.of(B)
    z = oracle.add_bias(oracle.matmul(A, B), bias)
    C, aux, _ = g.gpu_matmul(Av, Bv, algo=TC, bias=bias, act=1, want_aux=True)
    assert h.gemm_last_pair()
    out, mask = oracle.relu_fwd(z)
    near_zero = np.abs(z) < 1e-4
    assert np.allclose(C, out, rtol=1e-5, atol=1e-4) and np.array_equal(aux[~near_zero], mask[~near_zero])
    init = rng.standard_normal((M, N), np.float32)
    C2, _, _ = g.gpu_matmul(Av, Bv, algo=TC, beta=1.0, c_init=init)
    assert np.allclose(C2, init + oracle.matmul(A, B), rtol=1e-5, atol=1e-4)
    # extended options: multiplier (fused ReLU backward) and the lo plane of the stored result
    Ad, Bd, mul = g.dev(A), g.dev(B), g.dev((rng.random((M, N)) > 0.5).astype(np.float32))
    Cd, clo = g.empty(M, N), g.empty(M * N)
    h.gemm_ex(M, N, K, make_mat(Ad.data_ptr(), (M, K), (K, 1)), make_mat(Bd.data_ptr(), (K, N), (N, 1)), Cd.data_ptr(), algo=TC,
              mul_mask=mul.data_ptr(), c_lo=clo.data_ptr())
    assert h.gemm_last_pair()
    want = oracle.matmul(A, B) * g.host(mul)
    got = g.host(Cd)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-4)
    hi = (got.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)
    assert np.allclose(g.host(clo).reshape(M, N), got - hi, rtol=0, atol=np.abs(got).max() * 2.0 ** -21)
    Cd2 = g.empty(M, N)
    h.gemm_ex(M, N, K, make_mat(Ad.data_ptr(), (M, K), (K, 1)), make_mat(Bd.data_ptr(), (K, N), (N, 1)), Cd2.data_ptr(), algo=TC,
              mul_mask=mul.data_ptr())
    assert T.equal(Cd, Cd2)
    # (B, M, K) @ (1, K, N)
    Ab = rng.standard_normal((5, 300, 64), np.float32)
    Bb = rng.standard_normal((1, 64, 512), np.float32)
    Cb, _, _ = g.gpu_matmul(oracle.View.of(Ab), oracle.View.of(Bb), algo=TC)
    assert h.gemm_last_pair()
    assert np.max(np.abs(Cb - Ab.astype(np.float64) @ Bb.astype(np.float64))) <= TOL * 64 * 4
    h.check_device_status()


@pytest.mark.parametrize("mkn", [(2048, 4096, 4096), (768, 4096, 4096), (2048, 4096, 4000)], ids=str)
@pytest.mark.parametrize("layout", ["nn", "tn"])
def test_tc_pair_stream_k_tail(g, oracle, force_pair, mkn, layout):
    """The CTA-pair kernel with its stream-K tail (one piece per pair, two parked halves per piece): same bar as whole tiles,
    epilogue options honoured by the completing piece, repeatable bit for bit, flags back to zero after every launch."""
    M, K, N = mkn
    h = g.handle()
    if h.device_info()["sm_count"] != 148:
        pytest.skip("shapes chosen for 148 SMs")
    rng = np.random.default_rng(M + K + N + 1)
    A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    Av, Bv = layouts(oracle, A, B, layout)
    ref64 = A.astype(np.float64) @ B.astype(np.float64)
    scale = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64) + 1e-30
    C, _, _ = g.gpu_matmul(Av, Bv, algo=TC)
    assert h.gemm_last_pair() and h.gemm_last_stream_k() == 74
    h.check_device_status()
    assert float(np.max(np.abs(C - ref64) / scale)) <= 1e-5   # the bar is 1e-4; partial accumulators add a rounding each
    for _ in range(2):  # the flags were re-armed: the same bits again
        C2, _, _ = g.gpu_matmul(Av, Bv, algo=TC)
        assert np.array_equal(C, C2)
    Cb, aux, _ = g.gpu_matmul(Av, Bv, algo=TC, bias=bias, act=1, want_aux=True)
    z = ref64 + bias
    assert float(np.max(np.abs(Cb - np.maximum(z, 0)) / scale)) <= 1e-5
    near_zero = np.abs(z) < 1e-5 * scale
    assert np.array_equal(aux[~near_zero], (z > 0).astype(np.float32)[~near_zero])
    h.check_device_status()


# ---- long accumulation chains are cut into sub-ranges that the epilogue warps add up --------------------------------
CHUNK_SHAPES = [(256, 512, 256), (200, 516, 300), (1000, 772, 132), (129, 640, 262), (640, 2052, 388)]


@pytest.mark.parametrize("pair", [0, 1])
@pytest.mark.parametrize("mkn", CHUNK_SHAPES, ids=str)
@pytest.mark.parametrize("layout", ["nn", "nt", "tn"])
def test_tc_cut_accumulation_matches_oracle(g, oracle, monkeypatch, mkn, layout, pair):
    """TENMO_TC_CHUNK=4 makes every k-range above six k-blocks travel as several carried segments: plain result, result
    with every epilogue option, accumulate into C (the old C is the first carry), a column count that is not a multiple
    of four (scalar stores), both kernel forms."""
    M, K, N = mkn
    if layout == "tn" and M % 4:
        pytest.skip("transposed A needs a 16-byte aligned leading stride")
    if layout != "nt" and N % 4:
        pytest.skip("row-major B needs a 16-byte aligned leading stride")
    monkeypatch.setenv("TENMO_TC_CHUNK", "4")
    monkeypatch.setenv("TENMO_TC_PAIR", str(pair))
    if pair:
        monkeypatch.setenv("TENMO_TC_BN", "256")
    h = g.handle()
    rng = np.random.default_rng(M * 3 + K * 11 + N)
    A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    init = rng.standard_normal((M, N), np.float32)
    Av, Bv = layouts(oracle, A, B, layout)
    ref64 = A.astype(np.float64) @ B.astype(np.float64)
    scale = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64) + 1e-30
    C, _, _ = g.gpu_matmul(Av, Bv, algo=TC)
    assert h.gemm_last_algo() == TC and h.gemm_last_pair() == bool(pair)
    h.check_device_status()
    assert float(np.max(np.abs(C - ref64) / scale)) <= 1e-5
    Cb, aux, _ = g.gpu_matmul(Av, Bv, algo=TC, bias=bias, act=1, want_aux=True)
    z = ref64 + bias
    assert float(np.max(np.abs(Cb - np.maximum(z, 0)) / scale)) <= 1e-5
    near_zero = np.abs(z) < 1e-5 * scale
    assert np.array_equal(aux[~near_zero], (z > 0).astype(np.float32)[~near_zero])
    Ca, _, _ = g.gpu_matmul(Av, Bv, algo=TC, beta=1.0, c_init=init, bias=bias)
    assert float(np.max(np.abs(Ca - (init + z)) / (scale + np.abs(init)))) <= 1e-5
    # accumulate after an activation: C cannot hold the running sum, the range is summed in one chain as before
    Cr, _, _ = g.gpu_matmul(Av, Bv, algo=TC, beta=1.0, c_init=init, act=1)
    assert float(np.max(np.abs(Cr - (init + np.maximum(ref64, 0))) / (scale + np.abs(init)))) <= 1e-5
    h.check_device_status()
    monkeypatch.setenv("TENMO_TC_CHUNK", "0")
    C0, _, _ = g.gpu_matmul(Av, Bv, algo=TC)
    assert float(np.max(np.abs(C - C0) / scale)) <= 4e-6


@pytest.mark.parametrize("pair", [0, 1])
def test_tc_cut_accumulation_with_stream_k(g, oracle, monkeypatch, pair):
    """Pieces of the stream-K tail that are themselves cut: parked partials carry their sum in the slot, completing pieces
    in C."""
    h = g.handle()
    if h.device_info()["sm_count"] != 148:
        pytest.skip("shape chosen for 148 SMs")
    monkeypatch.setenv("TENMO_TC_CHUNK", "16")
    monkeypatch.setenv("TENMO_TC_PAIR", str(pair))
    monkeypatch.setenv("TENMO_TC_BN", "256")
    M, K, N = 2048, 4096, 4096
    rng = np.random.default_rng(77 + pair)
    A, B = rng.standard_normal((M, K), np.float32), rng.standard_normal((K, N), np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    Av, Bv = oracle.View.of(A), oracle.View.of(B)
    ref64 = A.astype(np.float64) @ B.astype(np.float64) + bias
    scale = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64) + 1e-30
    C, _, _ = g.gpu_matmul(Av, Bv, algo=TC, bias=bias)
    assert h.gemm_last_stream_k() > 0 and h.gemm_last_pair() == bool(pair)
    h.check_device_status()
    assert float(np.max(np.abs(C - ref64) / scale)) <= 1e-5
    C2, _, _ = g.gpu_matmul(Av, Bv, algo=TC, bias=bias)
    assert np.array_equal(C, C2)


@pytest.mark.parametrize("pair", [0, 1])
def test_tc_long_chain_of_same_signed_products(g, monkeypatch, pair):
    """The tensor core adds into its accumulator with truncation, so a chain of same-signed products drifts in proportion to
    its length (K = 8192 in one chain: about 1e-4 of sum |a||b|, the bar itself).  The kernel cuts chains above 96 k-blocks
    and adds the sub-sums in fp32 with rounding: a weight gradient of post-ReLU activations against one-sided gradients
    stays well inside the bar."""
    monkeypatch.setenv("TENMO_TC_PAIR", str(pair))
    monkeypatch.setenv("TENMO_TC_STREAMK", "0")
    monkeypatch.setenv("TENMO_TC_BN", "256")
    M, K, N = 2048, 8192, 1024
    rng = np.random.default_rng(5)
    A = np.maximum(rng.standard_normal((K, M), np.float32), 0)      # activations, stored (batch, features): used transposed
    B = np.abs(rng.standard_normal((K, N), np.float32)) * np.float32(1e-4)
    from oracle.ref import View

    Av, Bv = View.of(A).t(), View.of(B)
    C, _, _ = g.gpu_matmul(Av, Bv, algo=TC)
    h = g.handle()
    assert h.gemm_last_algo() == TC and h.gemm_last_pair() == bool(pair) and h.gemm_last_stream_k() == 0
    h.check_device_status()
    ref64 = A.T.astype(np.float64) @ B.astype(np.float64)   # all terms >= 0: sum |a||b| is the result itself
    cut = float(np.max(np.abs(C - ref64) / ref64))
    assert cut <= 8e-5, cut
    monkeypatch.setenv("TENMO_TC_CHUNK", "0")
    C1, _, _ = g.gpu_matmul(Av, Bv, algo=TC)
    one_chain = float(np.max(np.abs(C1 - ref64) / ref64))
    assert cut < 0.6 * one_chain, (cut, one_chain)
