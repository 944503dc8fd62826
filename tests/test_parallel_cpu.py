"""Data-parallel host logic on CPU: two gloo ranks, the CPU oracle standing in for the GPU kernels.

Checks that (a) the row sharding covers the global batch exactly once, (b) the NCCL unique id reaches every
rank unchanged through the broadcast helper, (c) shard gradients summed over ranks and scaled by 1/world
equal the global-batch gradients, so the data-parallel SGD step equals the single-process step.
"""
import os
import socket

import numpy as np
import pytest

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tenmo_b200.parallel import (DeviceFloats, averaged_gradients, connect_peer_buckets, exchange_unique_id, shard_rows,
                                 torch_all_gather_bytes, torch_broadcast_bytes)


def test_shard_rows():
    assert [shard_rows(8192, r, 8) for r in range(8)] == [(r * 1024, (r + 1) * 1024) for r in range(8)]
    assert shard_rows(64, 0, 1) == (0, 64)
    with pytest.raises(ValueError):
        shard_rows(10, 0, 4)
    with pytest.raises(ValueError):
        shard_rows(8, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    from oracle import ref

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # (b) unique id broadcast
        uid = exchange_unique_id(lambda: bytes(range(128)), rank, world, torch_broadcast_bytes())
        assert uid == bytes(range(128))

        # (b') the peer-memory exchange's setup: every rank's handle block reaches every rank, rank-major
        class FakeHandle:
            def dp_p2p_alloc(self, count):
                self.count = count
                return 0x1000 * (rank + 1), bytes([rank]) * 128

            def dp_p2p_connect(self, r, w, blob):
                self.connected = (r, w, blob)

        fake = FakeHandle()
        ptr = connect_peer_buckets(fake, 77, rank, world, torch_all_gather_bytes())
        assert ptr == 0x1000 * (rank + 1) and fake.count == 77
        assert fake.connected == (rank, world, b"".join(bytes([r]) * 128 for r in range(world)))

        # (c) one data-parallel step == one global-batch step
        rng = np.random.default_rng(99)  # same stream on every rank: identical replicas and global batch
        dims = [40, 24, 12, 6]
        Ws = [rng.uniform(-0.3, 0.3, (dims[i], dims[i + 1])).astype(np.float32) for i in range(3)]
        bs = [np.zeros(d, np.float32) for d in dims[1:]]
        X = rng.standard_normal((32, 40)).astype(np.float32)
        y = rng.integers(0, 6, 32)
        lo, hi = shard_rows(32, rank, world)
        local = ref.MLP(Ws, bs)
        local.step(X[lo:hi], y[lo:hi], update=False)  # fills dW / db with the shard-mean gradients

        def allreduce_sum(a):
            t = torch.from_numpy(a.copy())
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            return t.numpy()

        flat = np.concatenate([g.reshape(-1) for pair in zip(local.dW, local.db) for g in pair])
        avg = averaged_gradients(flat, allreduce_sum, world)
        full = ref.MLP(Ws, bs)
        full.step(X, y, update=False)
        flat_full = np.concatenate([g.reshape(-1) for pair in zip(full.dW, full.db) for g in pair])
        np.save(os.path.join(out_dir, f"diff{rank}.npy"), np.array([np.max(np.abs(avg - flat_full)), np.max(np.abs(flat_full))]))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_match_single_process(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        err, scale = np.load(tmp_path / f"diff{r}.npy")
        assert err <= 1e-6 * max(1.0, scale), (err, scale)


def test_device_floats_interface():
    d = DeviceFloats(0xABC000, 12)
    iface = d.__cuda_array_interface__
    assert iface["shape"] == (12,) and iface["typestr"] == "<f4" and iface["data"] == (0xABC000, False)
