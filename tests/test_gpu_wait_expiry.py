"""The expiry path of the device-side bounded waits, exercised without a fault: a probe kernel waits (with the wait
routine and status word of the GEMM kernels, limit 2 ms) on a barrier nothing arrives on, gives up and returns; the
host reads the status as an error and the context keeps working."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_wait_expiry_is_reported_and_the_context_survives(oracle):
    from tenmo_b200 import TenmoError
    from tests import gpu_util as g

    h = g.handle()
    h.check_device_status()
    h.wait_probe(2000)
    with pytest.raises(TenmoError) as err:
        h.check_device_status()
    assert "bounded wait" in str(err.value)
    h.check_device_status()  # the status word was cleared by the failed check
    rng = np.random.default_rng(0)
    A, B = rng.standard_normal((300, 200), np.float32), rng.standard_normal((200, 260), np.float32)
    for algo in (0, 1):
        C, _, _ = g.gpu_matmul(oracle.View.of(A), oracle.View.of(B), algo=algo)
        ref = oracle.matmul(A, B)
        assert np.array_equal(C, ref) if algo == 0 else np.allclose(C, ref, rtol=1e-4, atol=1e-4)
    h.check_device_status()


def test_wait_probe_rejects_unbounded_limits():
    from tenmo_b200 import TenmoError
    from tests import gpu_util as g

    for bad in (0, -5, 2_000_000):
        with pytest.raises(TenmoError):
            g.handle().wait_probe(bad)
