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

from tenmo_b200.parallel import (DeviceFloats, averaged_gradients, connect_peer_buckets, exchange_unique_id, optimizer_shard,
                                 shard_rows, torch_all_gather_bytes, torch_broadcast_bytes)


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


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("count", [0, 1, 3, 4, 10, 1000, 4096 * 1000, 16777216, 16777219])
def test_optimizer_shards_tile_the_layer(count, world):
    """The shards of the sharded-optimiser exchange cover [0, count) once, in rank order, every boundary but the end a
    multiple of four floats (16-byte accesses), sizes differing by less than one rounded shard."""
    spans = [optimizer_shard(count, r, world) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == count
    for (lo, hi), (nlo, _) in zip(spans, spans[1:]):
        assert lo <= hi == nlo and hi % 4 == 0 or hi == count
    assert all(lo % 4 == 0 or lo == count for lo, _ in spans)
    sz = max(hi - lo for lo, hi in spans)
    assert sz <= (count + world - 1) // world + 3
    with pytest.raises(ValueError):
        optimizer_shard(8, 2, 2)


def _sharded_worker(rank, world, port, out_dir):
    """The algorithm of tenmo_dp_p2p_sgd_step_f32 on the host: every rank holds its own gradient copy; the owner of a
    shard adds the W copies in rank order, applies SGD-momentum with grad_scale = 1/world to its shard of the parameters
    (its velocities never leave the rank) and the updated shards are gathered by everyone."""
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    from oracle import ref

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        count, lr, mom = 1003, 0.05, 0.9
        rng = np.random.default_rng(7)
        p0 = rng.standard_normal(count).astype(np.float32)                    # identical replicas
        grads = [rng.standard_normal(count).astype(np.float32) for _ in range(world)]   # rank r computed grads[r]
        vel_full = np.zeros(count, np.float32)
        p_ref = p0.copy()
        p_mine, v_mine = p0.copy(), np.zeros(count, np.float32)              # v_mine: only the own shard is ever touched
        scale = np.float32(1.0 / world)
        for step in range(3):
            # reference: sum in rank order, scaled, one SGD step over everything (the all-reduce + SGD form)
            total = grads[0].copy()
            for g in grads[1:]:
                total = total + g
            ref.sgd_step(p_ref, total * scale, vel_full, lr, mom)
            # sharded: gather every rank's copy of MY shard (the peer loads), sum in rank order, update my shard
            lo, hi = optimizer_shard(count, rank, world)
            mine = torch.from_numpy(grads[rank].copy())
            copies = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(copies, mine)
            s = copies[0].numpy()[lo:hi].copy()
            for c in copies[1:]:
                s = s + c.numpy()[lo:hi]
            shard_p, shard_v = p_mine[lo:hi].copy(), v_mine[lo:hi].copy()
            ref.sgd_step(shard_p, s * scale, shard_v, lr, mom)
            v_mine[lo:hi] = shard_v
            # the push of the updated parameters: every rank receives every shard
            padded = np.zeros(count, np.float32)
            padded[lo:hi] = shard_p
            t = torch.from_numpy(padded)
            dist.all_reduce(t, op=dist.ReduceOp.SUM)                          # disjoint shards: the sum is the gather
            p_mine = t.numpy().copy()
            grads = [g * np.float32(0.5) + np.float32(0.1) for g in grads]    # next step's gradients
        # the checkpoint's gather of the sharded momentum
        tv = torch.from_numpy(v_mine.copy())
        dist.all_reduce(tv, op=dist.ReduceOp.SUM)
        np.save(os.path.join(out_dir, f"sh{rank}.npy"),
                np.array([float(np.array_equal(p_mine, p_ref)), float(np.array_equal(tv.numpy(), vel_full)),
                          float(np.count_nonzero(np.delete(v_mine, np.arange(lo, hi))))]))
    finally:
        dist.destroy_process_group()


def test_sharded_optimiser_equals_allreduce_then_sgd(tmp_path):
    world = 2
    mp.spawn(_sharded_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        same_params, same_velocity, stray = np.load(tmp_path / f"sh{r}.npy")
        assert same_params == 1.0 and same_velocity == 1.0 and stray == 0.0
