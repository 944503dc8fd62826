"""Data-parallel training, over NCCL and over the library's own peer-memory kernel: two ranks on two GPUs equal one
rank on the global batch.

Runs as child processes, one per GPU (skipped with fewer than two GPUs).  NVLS is switched off and every
rank leaves only between steps, as this pool asks of multi-process GPU tests.
"""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _problem(classes=10):
    rng = np.random.default_rng(31)
    dims = [256, 192, 128, classes]
    Ws = [rng.uniform(-1, 1, (dims[i], dims[i + 1])).astype(np.float32) * np.float32(np.sqrt(6.0 / dims[i])) for i in range(3)]
    bs = [np.zeros(d, np.float32) for d in dims[1:]]
    X = rng.standard_normal((4, 128, 256)).astype(np.float32)  # 4 steps of a 128-row global batch
    y = rng.integers(0, 10, (4, 128))
    return Ws, bs, X, y


def _worker(rank, world, port, out_dir, mode):
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    import torch.distributed as dist

    from tenmo_b200 import TenmoCuda
    from tenmo_b200.parallel import exchange_unique_id, shard_rows, torch_all_gather_bytes, torch_broadcast_bytes
    from tenmo_b200.trainer import MLPTrainer

    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # mode = exchange[+tc][+graph]: "+tc" runs the 3xTF32 kernel (the sharded optimiser then also writes the weights'
        # lo planes), "+graph" replays the captured step instead of enqueueing it
        exchange, *flags = mode.split("+")
        algo = "3xtf32" if "tc" in flags else "simt"
        h = TenmoCuda(rank).require()
        uid = exchange_unique_id(h.dp_get_unique_id, rank, world, torch_broadcast_bytes()) if exchange == "nccl" else None
        Ws, bs, X, y = _problem(16 if "tc" in flags else 10)   # the tensor-core kernel wants 16-byte aligned rows
        lo, hi = shard_rows(128, rank, world)
        tr = MLPTrainer(Ws, bs, batch=hi - lo, lr=0.05, momentum=0.9, algo=algo, handle=h, rank=rank, world=world,
                        unique_id=uid, device=rank, exchange=exchange, all_gather_bytes=torch_all_gather_bytes())
        if exchange.startswith("p2p") and not flags:
            # the collective on its own: ragged ranges, every rank ends with the same bits = the sum in rank order
            g = torch.Generator(device="cpu").manual_seed(5 + rank)
            mine = torch.randn(tr.numel, generator=g)
            for off, cnt in ((0, tr.numel), (4, 1001), (8, 3), (12, 0), (256, 4096)):
                tr.G.copy_(mine)
                torch.cuda.synchronize()
                dist.barrier()
                h.dp_p2p_allreduce_sum(off, cnt)
                torch.cuda.synchronize()
                h.check_device_status()
                parts = [torch.randn(tr.numel, generator=torch.Generator(device="cpu").manual_seed(5 + r)) for r in range(world)]
                want = mine.clone()
                acc = parts[0][off:off + cnt].clone()
                for r in range(1, world):
                    acc += parts[r][off:off + cnt]
                want[off:off + cnt] = acc
                assert torch.equal(tr.G.cpu(), want), (off, cnt)
                dist.barrier()
            tr.G.zero_()
            torch.cuda.synchronize()
            dist.barrier()
        losses = []
        if "graph" in flags:
            tr.load_batch(X[0, lo:hi], y[0, lo:hi])
            dist.barrier()
            tr.capture()     # two warm-up steps and the capture itself: every rank makes the same calls
            torch.cuda.synchronize()
            dist.barrier()
        for s in range(4):
            if "graph" in flags:
                tr.load_batch(X[s, lo:hi], y[s, lo:hi])
                tr.replay()
            else:
                tr.step(X[s, lo:hi], y[s, lo:hi])
            losses.append(tr.loss_value())
        torch.cuda.synchronize()
        h.check_device_status()
        vel = tr.state_dict()["__velocity__"]   # gathers the sharded momentum: every rank calls it
        np.save(os.path.join(out_dir, f"v{rank}.npy"), vel)
        np.save(os.path.join(out_dir, f"w{rank}.npy"), np.concatenate([w.reshape(-1) for w in tr.weights() + tr.biases()]))
        np.save(os.path.join(out_dir, f"l{rank}.npy"), np.array(losses))
        dist.barrier()  # leave only between steps, with nothing in flight
        tr.close()
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["nccl", "p2p", "p2p_allreduce", "p2p+tc", "p2p+graph"])
def test_two_ranks_equal_one_rank_on_the_global_batch(tmp_path, mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from tenmo_b200.trainer import MLPTrainer

    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), mode), nprocs=2, join=True)
    Ws, bs, X, y = _problem(16 if "+tc" in mode else 10)
    single = MLPTrainer(Ws, bs, batch=128, lr=0.05, momentum=0.9, algo="3xtf32" if "+tc" in mode else "simt")
    losses = []
    for s in range(4):
        single.step(X[s], y[s])
        losses.append(single.loss_value())
    ref = np.concatenate([w.reshape(-1) for w in single.weights() + single.biases()])
    w0, w1 = np.load(tmp_path / "w0.npy"), np.load(tmp_path / "w1.npy")
    assert np.array_equal(w0, w1), "replicas diverged"
    # summation order differs (two half-batch sums added by NCCL vs one full-batch chain): 1e-5 relative
    bar = 5e-5 if "+tc" in mode else 1e-5   # 3xTF32 products of half batches round differently from the full batch's
    assert np.max(np.abs(w0 - ref)) <= bar * np.max(np.abs(ref))
    l0, l1 = np.load(tmp_path / "l0.npy"), np.load(tmp_path / "l1.npy")
    assert np.allclose((l0 + l1) / 2, losses, rtol=10 * bar, atol=1e-6)  # mean of rank means == global mean
    # the momentum buffers, gathered from the ranks that own them, are the single rank's
    v0, v1 = np.load(tmp_path / "v0.npy"), np.load(tmp_path / "v1.npy")
    vref = single.state_dict()["__velocity__"]
    assert np.array_equal(v0, v1) and np.max(np.abs(v0 - vref)) <= 10 * bar * np.max(np.abs(vref))


def test_sharded_optimiser_kernel_single_rank_matches_sgd_kernel():
    """tenmo_dp_p2p_sgd_step_f32 with a world of one is SGD-momentum on the whole range: the parameters, velocities and
    lo plane it leaves equal tenmo_sgd_step_lo_f32's bit for bit, on aligned and ragged ranges, over two steps."""
    from tenmo_b200 import TenmoCuda
    from tenmo_b200.parallel import DeviceFloats

    h = TenmoCuda(0).require()
    h.set_stream(torch.cuda.current_stream().cuda_stream)
    n = 300_000
    ptr, handles = h.dp_p2p_alloc(2 * n)
    try:
        h.dp_p2p_connect(0, 1, handles)
        bucket = torch.as_tensor(DeviceFloats(ptr, 2 * n), device="cuda:0")
        G, P = bucket[:n], bucket[n:]
        gen = torch.Generator(device="cuda").manual_seed(3)
        for off, cnt, lo_cnt in ((0, n, n), (1024, 70_001, 40_000), (4, 3, 3), (8, 100_003, 0)):
            p0 = torch.randn(n, generator=gen, device="cuda")
            v0 = torch.randn(n, generator=gen, device="cuda") * 0.1
            P.copy_(p0)
            V, lo = v0.clone(), torch.zeros(n, device="cuda")
            rp, rv, rlo = p0.clone(), v0.clone(), torch.zeros(n, device="cuda")
            for step in range(2):
                g = torch.randn(n, generator=gen, device="cuda")
                G.copy_(g)
                h.dp_p2p_sgd_step(off, n + off, cnt, V.data_ptr() + 4 * off, lo.data_ptr() + 4 * off, lo_cnt, 0.05, 0.9, 0.01, 0.5)
                h.sgd_step([rp.data_ptr() + 4 * off], [g.data_ptr() + 4 * off], [rv.data_ptr() + 4 * off], [cnt], 0.05, 0.9, 0.01, 0.5,
                           lo_ptrs=[rlo.data_ptr() + 4 * off], lo_numels=[lo_cnt])
                torch.cuda.synchronize()
                assert torch.equal(P, rp) and torch.equal(V, rv) and torch.equal(lo, rlo), (off, cnt, step)
                assert torch.equal(G, g)   # the gradient range is left alone
        with pytest.raises(Exception):
            h.dp_p2p_sgd_step(0, 10, 100, V.data_ptr(), 0, 0, 0.1, 0.9)   # overlapping ranges
        h.check_device_status()
    finally:
        h.dp_p2p_close()


def test_p2p_single_rank_and_argument_errors():
    """The peer-memory exchange's entry points on one GPU: state and range errors, world = 1 as a no-op."""
    from tenmo_b200 import TenmoCuda, TenmoError

    h = TenmoCuda(0).require()
    with pytest.raises(TenmoError):
        h.dp_p2p_allreduce_sum(0, 10)          # nothing allocated or connected
    ptr, handles = h.dp_p2p_alloc(1000)
    assert ptr != 0 and len(handles) == 128
    with pytest.raises(TenmoError):
        h.dp_p2p_alloc(10)                     # one bucket per context
    with pytest.raises(TenmoError):
        h.dp_p2p_connect(0, 9, handles * 9)    # at most 8 ranks
    with pytest.raises(TenmoError):
        h.dp_p2p_connect(1, 1, handles)        # rank outside the world
    h.dp_p2p_connect(0, 1, handles)
    h.dp_p2p_allreduce_sum(0, 1000)            # a single rank: nothing to exchange
    with pytest.raises(TenmoError):
        h.dp_p2p_allreduce_sum(900, 200)       # range outside the bucket
    h.check_device_status()
    h.dp_p2p_close()
    h.dp_p2p_close()                           # closing twice is harmless
