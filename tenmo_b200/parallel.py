"""Host-side logic of batch-sharded data-parallel training (one process per GPU).

The reference has no distributed layer (its README lists it as future work), so there is nothing to
mirror here; this is the plumbing around ``tenmo_dp_*``: which rows a rank owns, how the NCCL unique id
travels from rank 0 to the others, and the gradient-averaging rule.  Everything in this module runs
without a GPU (the collective is passed in), so it is tested with gloo ranks on CPU.
"""
from __future__ import annotations

import numpy as np


def shard_rows(global_batch: int, rank: int, world: int) -> tuple[int, int]:
    """[begin, end) of the consecutive rows rank ``rank`` owns.  The global batch must divide evenly:
    with equal shards the mean of the per-rank mean losses is the global mean, and a sum all-reduce
    scaled by 1/world is the global-batch gradient."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world {world}")
    if global_batch % world != 0:
        raise ValueError(f"global batch {global_batch} does not split evenly over {world} ranks")
    per = global_batch // world
    return rank * per, (rank + 1) * per


def optimizer_shard(count: int, rank: int, world: int) -> tuple[int, int]:
    """[lo, hi) of the `count` floats of a layer whose gradients rank `rank` sums and whose optimiser state it owns in
    the sharded exchange (tenmo_dp_p2p_sgd_step_f32): equal shards rounded up to four floats, the last ones short or
    empty.  The same arithmetic as the kernel's, so that checkpoints can gather and re-deal the momentum."""
    if not 0 <= rank < world or count < 0:
        raise ValueError(f"rank {rank} / world {world} / count {count}")
    sz = ((count + world - 1) // world + 3) // 4 * 4
    lo = min(count, rank * sz)
    return lo, min(count, lo + sz)


def exchange_unique_id(get_unique_id, rank: int, world: int, broadcast_bytes) -> bytes | None:
    """Rank 0 draws the 128-byte NCCL id (``get_unique_id()``), everyone receives it through
    ``broadcast_bytes(buf: bytearray, src=0)`` -- any out-of-band channel (a torch.distributed gloo / nccl
    broadcast, a file, a TCP store).  Returns None when world == 1."""
    if world == 1:
        return None
    buf = bytearray(128)
    if rank == 0:
        uid = get_unique_id()
        if len(uid) != 128:
            raise ValueError("unique id must be 128 bytes")
        buf[:] = uid
    broadcast_bytes(buf, 0)
    return bytes(buf)


def torch_broadcast_bytes(device=None):
    """A ``broadcast_bytes`` built on the default torch.distributed process group."""
    import torch
    import torch.distributed as dist

    def bcast(buf: bytearray, src: int):
        t = torch.tensor(list(buf), dtype=torch.uint8, device=device)
        dist.broadcast(t, src)
        buf[:] = bytes(t.cpu().tolist())

    return bcast


def torch_all_gather_bytes(device=None):
    """An ``all_gather_bytes(data) -> [bytes per rank]`` built on the default torch.distributed process group (every
    rank passes the same length)."""
    import torch
    import torch.distributed as dist

    def gather(data: bytes):
        mine = torch.tensor(list(data), dtype=torch.uint8, device=device)
        out = [torch.empty_like(mine) for _ in range(dist.get_world_size())]
        dist.all_gather(out, mine)
        return [bytes(t.cpu().tolist()) for t in out]

    return gather


def connect_peer_buckets(handle, count: int, rank: int, world: int, all_gather_bytes):
    """The peer-memory exchange's setup: allocate this rank's gradient bucket inside the library, share its CUDA IPC
    handles with the other ranks through ``all_gather_bytes`` and map theirs.  Returns the device pointer of the
    bucket (``count`` floats, zeroed)."""
    ptr, handles = handle.dp_p2p_alloc(count)
    blocks = all_gather_bytes(handles)
    if len(blocks) != world or any(len(b) != len(handles) for b in blocks):
        raise ValueError("all_gather_bytes must return one handle block per rank")
    handle.dp_p2p_connect(rank, world, b"".join(blocks))
    return ptr


class DeviceFloats:
    """Device memory owned by someone else, exposed through __cuda_array_interface__ so that torch.as_tensor wraps it
    without a copy."""

    def __init__(self, ptr: int, count: int):
        self.__cuda_array_interface__ = {"shape": (int(count),), "typestr": "<f4", "data": (int(ptr), False), "version": 2}


def averaged_gradients(local_grads: np.ndarray, allreduce_sum, world: int) -> np.ndarray:
    """sum over ranks, then 1/world: what the fused SGD kernel applies through ``grad_scale``."""
    total = allreduce_sum(np.ascontiguousarray(local_grads, np.float32))
    return total * np.float32(1.0 / world)
