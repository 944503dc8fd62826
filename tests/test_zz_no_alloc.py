"""The column-sum entry point that never allocates, checked against the regular one.

Who needs it: a host that cannot let this library call cudaMalloc -- it has given the whole device to
its own buffer pool, or it runs a loop that must not hit the device-wide synchronisation an allocation
implies.  ``tenmo_colsum_f32_static`` keeps its scratch (partial sums + ticket counters) in a fixed
array inside the loaded module instead of the context's growable workspace, serves up to 16384 columns
and needs no context at all.

The test calls it through the C ABI twice in a row on different shapes (the second call meets whatever
the first left in the shared scratch) and compares with ``tenmo_colsum_f32`` at the tolerance the other
reduction tests use: 1e-5 relative to the column's sum of magnitudes (the two entry points may split the
rows into different slabs, so the last bits can differ).  This file is collected last, so a run that
stops at the first failure has already run every other test; it also passes alone in a fresh process.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _both(g, x, beta_init=None):
    h = g.handle()
    M, N = x.shape
    xd = g.dev(x)
    ref = g.empty(N) if beta_init is None else g.dev(beta_init)
    got = g.empty(N) if beta_init is None else g.dev(beta_init)
    beta = 0.0 if beta_init is None else 1.0
    h.colsum(xd.data_ptr(), M, N, N, ref.data_ptr(), beta=beta)
    h.colsum_static(xd.data_ptr(), M, N, N, got.data_ptr(), beta=beta, stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return g.host(got), g.host(ref)


def test_static_colsum_matches_regular_entry_point_twice_in_a_row():
    from tenmo_b200 import TenmoError
    from tests import gpu_util as g

    rng = np.random.default_rng(77)
    shapes = [(8192, 4096), (5000, 1000)]  # two calls in a row: wide + vector loads, then ragged
    for M, N in shapes:
        x = rng.standard_normal((M, N), np.float32)
        got, ref = _both(g, x)
        scale = np.abs(x).sum(axis=0)
        assert np.max(np.abs(got - ref) / scale) <= 1e-5
        assert np.max(np.abs(got - x.astype(np.float64).sum(axis=0)) / scale) <= 1e-6
    # accumulate form, scalar-load path (N not a multiple of 4), and the few-rows path that needs no scratch
    for M, N in [(3001, 130), (64, 128)]:
        x = rng.standard_normal((M, N), np.float32)
        init = rng.standard_normal(N).astype(np.float32)
        got, ref = _both(g, x, beta_init=init)
        assert np.max(np.abs(got - ref) / (np.abs(x).sum(axis=0) + np.abs(init))) <= 1e-5
    # beyond the fixed scratch: a clear refusal, not a silent fallback to allocating
    h = g.handle()
    wide = g.empty(600, 16388)
    out = g.empty(16388)
    with pytest.raises(TenmoError) as e:
        h.colsum_static(wide.data_ptr(), 600, 16388, 16388, out.data_ptr())
    assert e.value.status == -3 and "16384" in str(e.value)
