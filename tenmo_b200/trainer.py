"""A whole Linear/ReLU/softmax-CE/SGD training step as one pre-planned sequence of C-ABI calls.

This is the call sequence tenmo's host makes for ``Sequential(Linear, ReLU, ..., Linear)`` +
``CrossEntropyLoss`` + ``SGD`` (net.mojo:1085-1092, crossentropy.mojo:1360-1391, tensor.mojo:3154-3247,
optim.mojo:405-543) with the host round trips taken out so that it can be replayed as a CUDA graph:

  forward   per layer ONE GEMM with the bias add, ReLU and the 0/1 mask in its epilogue
  loss      fused cross-entropy forward + backward, loss and valid count stay on the device
  backward  per layer dW = X^T . dY (db rides along as the column sum of dY) and dX = dY . W^T on
            transposed stride views, then the ReLU mask multiply
  exchange  (data parallel) per layer, on a side stream, as soon as that layer's gradients exist: an NCCL sum
            all-reduce followed by SGD on the layer's slice, or ONE kernel of this library that reduce-scatters the
            gradients over NVLink peer memory, applies SGD to this rank's 1/world shard and all-gathers the
            updated weights.  The backward pass runs every dX first and the dW of the lowest layers last-but-
            early, so that no exchange is left to finish after the last GEMM; the next step's forward of layer l
            waits for layer l's update only.
  update    (one GPU) ONE SGD-momentum launch over the flat parameter / gradient / velocity buffers
  feed      two sets of input buffers and a copy stream: the upload of the next batch overlaps the current step

All parameters live in one flat buffer (weights and biases back to back), and so do gradients and
velocities, which is what makes the single all-reduce and the single optimizer launch possible.
"""
from __future__ import annotations

import numpy as np
import torch

from . import lib as _lib
from .lib import TenmoCuda, make_mat
from .parallel import optimizer_shard, shard_rows


class BatchFeed:
    """Two sets of input buffers and a copy stream (the pinned-memory batch upload of examples/mnist_gpu.mojo:174-175,
    double-buffered): ``load_batch`` uploads into the set the running step does not read, so the host-to-device copy
    of the next batch overlaps the current step; ``_begin_step`` switches to the uploaded set and makes the compute
    stream wait for its copy, ``_end_step`` marks the set free once every reader has been queued."""

    def _feed_init(self, x_shape, dev: int):
        f32 = dict(dtype=torch.float32, device=f"cuda:{dev}")
        self._Xs = [torch.zeros(*x_shape, **f32) for _ in range(2)]
        self._ys = [torch.zeros(x_shape[0], dtype=torch.int64, device=f"cuda:{dev}") for _ in range(2)]
        self._set = 0            # the set the next step reads
        self._loaded = None      # a set uploaded by load_batch that no step has consumed yet
        self._copy_stream = None
        self._set_ready = [None, None]   # recorded on the copy stream after an upload
        self._set_free = [None, None]    # recorded on the compute stream after the last reader of a set
        self.X, self.y = self._Xs[0], self._ys[0]
        self.graph = None

    def _use_set(self, k: int):
        self._set = k
        self.X, self.y = self._Xs[k], self._ys[k]

    def load_batch(self, X, y):
        """Upload a batch and its int64 labels for the NEXT step.  Host arrays and pinned tensors are copied
        asynchronously on a copy stream into the set of input buffers the running step does not read.  A trainer whose
        step has been captured into a CUDA graph has fixed input addresses: it copies into the captured set on the
        current stream."""
        if not torch.is_tensor(X):
            X = torch.from_numpy(np.ascontiguousarray(X, np.float32))
        if not torch.is_tensor(y):
            y = torch.from_numpy(np.ascontiguousarray(y, np.int64))
        if self.graph is not None:
            self.X.copy_(X, non_blocking=True)
            self.y.copy_(y, non_blocking=True)
            return
        main = torch.cuda.current_stream(self.dev)
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(self.dev)
        k = self._loaded if self._loaded is not None else 1 - self._set
        cs = self._copy_stream
        if X.is_cuda or y.is_cuda:  # device-resident sources may still be being produced on the compute stream
            ev = torch.cuda.Event()
            ev.record(main)
            cs.wait_event(ev)
        if self._set_free[k] is not None:
            cs.wait_event(self._set_free[k])
        with torch.cuda.stream(cs):
            self._Xs[k].copy_(X, non_blocking=True)
            self._ys[k].copy_(y, non_blocking=True)
        for t in (X, y):
            if t.is_cuda:
                t.record_stream(cs)
        ready = torch.cuda.Event()
        ready.record(cs)
        self._set_ready[k] = ready
        self._loaded = k

    def _begin_step(self, X=None, y=None):
        main = torch.cuda.current_stream(self.dev)
        self.h.set_stream(main.cuda_stream)
        if X is not None:
            self.load_batch(X, y)
        if self._loaded is not None:
            self._use_set(self._loaded)
            self._loaded = None
            main.wait_event(self._set_ready[self._set])

    def _end_step(self):
        if self._copy_stream is not None:
            free = torch.cuda.Event()
            free.record(torch.cuda.current_stream(self.dev))  # every reader of this set has been queued before this point
            self._set_free[self._set] = free


class MLPTrainer(BatchFeed):
    def __init__(self, weights, biases, batch: int, lr: float = 0.01, momentum: float = 0.9, weight_decay: float = 0.0,
                 algo: str = "auto", handle: TenmoCuda | None = None, rank: int = 0, world: int = 1,
                 unique_id: bytes | None = None, device: int | None = None, overlap: bool | None = None,
                 reserve_sms: int = 0, exchange: str = "nccl", all_gather_bytes=None):
        """exchange: "nccl" (tenmo_dp_allreduce_sum_f32, then SGD on every rank; needs unique_id), "p2p" (the library's
        own kernel over NVLink peer memory with the optimiser sharded over the ranks, tenmo_dp_p2p_sgd_step_f32) or
        "p2p_allreduce" (the peer-memory all-reduce, then SGD on every rank).  The p2p forms need
        all_gather_bytes(data) -> [bytes per rank] to share the IPC handles of the bucket.
        overlap: run each layer's exchange on a side stream beside the remaining backward GEMMs.  None picks what measured
        best on 2 to 8 B200s: on for NCCL up to 4 ranks, off otherwise -- at 1024 rows per rank every GEMM is a single wave
        of CTAs, and anything that shares the SMs or the memory system with it costs more than the exchange it hides."""
        self.dev = torch.cuda.current_device() if device is None else device
        self.h = handle or TenmoCuda(self.dev).require()
        self.algo = {"auto": _lib.ALGO_AUTO, "simt": _lib.ALGO_SIMT_FP32, "3xtf32": _lib.ALGO_TC_3XTF32}[algo]
        self.rank, self.world = rank, world
        self.lr, self.momentum, self.wd = float(lr), float(momentum), float(weight_decay)
        self.batch = int(batch)
        self.dims = [int(weights[0].shape[0])] + [int(w.shape[1]) for w in weights]
        self.L = len(weights)
        f32 = dict(dtype=torch.float32, device=f"cuda:{self.dev}")
        # flat parameter / gradient / velocity buffers; every slice starts on a 16-byte boundary
        sizes, offs, off = [], [], 0
        for l in range(self.L):
            for n in (self.dims[l] * self.dims[l + 1], self.dims[l + 1]):
                offs.append(off)
                sizes.append(n)
                off += (n + 3) // 4 * 4
        self.numel = off
        self.exchange = exchange if world > 1 else "none"
        if self.exchange not in ("none", "nccl", "p2p", "p2p_allreduce"):
            raise ValueError(f"unknown exchange {exchange!r}")
        self.sharded = self.exchange == "p2p"
        if self.exchange in ("p2p", "p2p_allreduce"):
            # gradients AND parameters live in memory the library allocated and every peer has mapped: the peers read
            # each other's gradient shards and (sharded optimiser) each other's updated parameter shards
            from .parallel import DeviceFloats, connect_peer_buckets

            ptr = connect_peer_buckets(self.h, 2 * off, rank, world, all_gather_bytes)
            bucket = torch.as_tensor(DeviceFloats(ptr, 2 * off), device=f"cuda:{self.dev}")
            self.G, self.P = bucket[:off], bucket[off:]
            self._bucket = bucket
        else:
            self.P = torch.zeros(off, **f32)
            self.G = torch.zeros(off, **f32)
        self.V = torch.zeros(off, **f32)
        self.W = [self.P[offs[2 * l]:offs[2 * l] + sizes[2 * l]].view(self.dims[l], self.dims[l + 1]) for l in range(self.L)]
        self.b = [self.P[offs[2 * l + 1]:offs[2 * l + 1] + sizes[2 * l + 1]] for l in range(self.L)]
        self.dW = [self.G[offs[2 * l]:offs[2 * l] + sizes[2 * l]].view(self.dims[l], self.dims[l + 1]) for l in range(self.L)]
        self.db = [self.G[offs[2 * l + 1]:offs[2 * l + 1] + sizes[2 * l + 1]] for l in range(self.L)]
        for l in range(self.L):
            self.W[l].copy_(torch.from_numpy(np.ascontiguousarray(weights[l], np.float32)))
            self.b[l].copy_(torch.from_numpy(np.ascontiguousarray(biases[l], np.float32)))
        B = self.batch
        self._feed_init((B, self.dims[0]), self.dev)   # two sets of input buffers (BatchFeed)
        self.act = [self.X] + [torch.empty(B, d, **f32) for d in self.dims[1:]]
        self.mask = [torch.empty(B, d, **f32) for d in self.dims[1:-1]]
        self.gout = [torch.empty(B, d, **f32) for d in self.dims[1:]]     # dL/d(pre-activation) of layer l
        # 3xTF32 lo planes, each produced once per tensor per step: weights after the update, activations and
        # gradients by the epilogue of the GEMM that writes them (only the tensor-core path uses them)
        self.fused_lo = self.algo == _lib.ALGO_TC_3XTF32
        r4 = lambda n: (n + 3) // 4 * 4
        if self.fused_lo:
            self.W_lo = [torch.empty(self.dims[l] * r4(self.dims[l + 1]), **f32) for l in range(self.L)]
            self.act_lo = [torch.empty(B * r4(d), **f32) for d in self.dims[:-1]]
            self._x_lo = [self.act_lo[0], torch.empty_like(self.act_lo[0])]
            self.gout_lo = [torch.empty(B * r4(d), **f32) for d in self.dims[1:]]
        self.softmax = torch.empty(B, self.dims[-1], **f32)
        self.loss = torch.zeros(1, **f32)
        self.valid = torch.zeros(1, dtype=torch.int32, device=f"cuda:{self.dev}")
        self.correct = torch.zeros(1, dtype=torch.int64, device=f"cuda:{self.dev}")
        self._stream = None
        # [start, count) of each layer's weight + bias inside the flat buffers
        self.layer_span = [(offs[2 * l], offs[2 * l + 1] + (sizes[2 * l + 1] + 3) // 4 * 4 - offs[2 * l])
                           for l in range(self.L)]
        if overlap is None:
            overlap = self.exchange == "nccl" and world <= 4
        self.overlap = bool(overlap) and world > 1
        self._side = torch.cuda.Stream(self.dev) if self.overlap else None
        self._upd_ev = [None] * self.L   # per layer: recorded on the side stream after the layer's update
        self._join_each_step = False     # a captured step must end with the side stream joined
        self.reserve_sms = int(reserve_sms) if self.overlap else 0
        if self.exchange == "nccl":
            self.h.dp_init(rank, world, unique_id)
        elif self.exchange in ("p2p", "p2p_allreduce"):
            self.h.dp_p2p_set_coresident(self.overlap)
        if self.fused_lo:
            self.h.set_stream(torch.cuda.current_stream(self.dev).cuda_stream)
            for l in range(self.L):
                self._split_weight(l)
        torch.cuda.synchronize(self.dev)

    # ------------------------------------------------------------------------------------------------
    def _m(self, t: torch.Tensor, transpose: bool = False):
        r, c = t.shape
        if transpose:
            return make_mat(t.data_ptr(), (c, r), (1, c))
        return make_mat(t.data_ptr(), (r, c), (c, 1))

    def _enqueue(self, update: bool = True):
        """Queue one step on the context's current stream (no host synchronisation anywhere)."""
        self._forward()
        if update and self.overlap:
            # per-layer all-reduce + SGD on the side stream, under the backward GEMMs, which leave a few SMs
            # free for the collective's CTAs
            self.h.reserve_sms(self.reserve_sms)
            self._backward(exchange=True)
            self.h.reserve_sms(0)
        else:
            self._backward()
            if update:
                self._update()

    def _split_weight(self, l: int):
        w = self.W[l]
        self.h.split_lo(self._m(w), w.shape[0], w.shape[1], self.W_lo[l].data_ptr(), self.W_lo[l].numel())

    def _forward(self):
        h, L, B = self.h, self.L, self.batch
        lo = self.fused_lo
        if lo:  # the input's lo plane: the only activation no GEMM epilogue produces
            h.split_lo(self._m(self.X), B, self.dims[0], self.act_lo[0].data_ptr(), self.act_lo[0].numel())
        main = torch.cuda.current_stream(self.dev)
        for l in range(L):
            last = l == L - 1
            if self._upd_ev[l] is not None:  # the previous step's update of THIS layer (side stream) must have landed
                main.wait_event(self._upd_ev[l])
                self._upd_ev[l] = None
            h.gemm_ex(B, self.dims[l + 1], self.dims[l], self._m(self.act[l]), self._m(self.W[l]), self.act[l + 1].data_ptr(),
                      algo=self.algo, bias=self.b[l].data_ptr(), act=_lib.ACT_NONE if last else _lib.ACT_RELU,
                      aux=0 if last else self.mask[l].data_ptr(),
                      a_lo=self.act_lo[l].data_ptr() if lo else 0, b_lo=self.W_lo[l].data_ptr() if lo else 0,
                      c_lo=self.act_lo[l + 1].data_ptr() if (lo and not last) else 0)
        C = self.dims[-1]
        # loss and dlogits together: the loss is the root of the backward pass (one launch for a small batch)
        h.ce_fwd_bwd(self.act[L].data_ptr(), C, self.y.data_ptr(), True, B, C, -100, 0.0, 0, self.softmax.data_ptr(),
                     self.loss.data_ptr(), self.valid.data_ptr(), 0, self.gout[L - 1].data_ptr())

    def _allreduce(self, start: int, count: int):
        """Sum G[start, start + count) over the ranks on the library's current stream."""
        if self.exchange in ("p2p", "p2p_allreduce"):
            self.h.dp_p2p_allreduce_sum(start, count)
        else:
            self.h.dp_allreduce_sum(self.G.data_ptr() + 4 * start, count)

    def close(self):
        """Release the data-parallel resources (every rank, after a host barrier)."""
        if self.exchange in ("p2p", "p2p_allreduce"):
            torch.cuda.synchronize(self.dev)
            self.G = self.P = self._bucket = None
            self.dW = self.db = self.W = self.b = None
            self.h.dp_p2p_close()
        elif self.exchange == "nccl":
            self.h.dp_finalize()
        self.exchange = "none"

    def _sgd_layers(self, layers):
        """SGD on the flat slices of these layers (weight + bias each) in one launch.  On the 3xTF32 path the kernel
        also writes the weights' lo planes (a weight row that is a multiple of 4 long has the plane's layout as it
        stands; any other width is split separately)."""
        h = self.h
        spans = [self.layer_span[l] for l in layers]
        ptr = lambda buf, s: buf.data_ptr() + 4 * s
        kw = {}
        if self.fused_lo:
            fusable = [self.dims[l + 1] % 4 == 0 for l in layers]
            kw = dict(lo_ptrs=[self.W_lo[l].data_ptr() if ok else 0 for l, ok in zip(layers, fusable)],
                      lo_numels=[self.dims[l] * self.dims[l + 1] if ok else 0 for l, ok in zip(layers, fusable)])
        h.sgd_step([ptr(self.P, s) for s, _ in spans], [ptr(self.G, s) for s, _ in spans], [ptr(self.V, s) for s, _ in spans],
                   [c for _, c in spans], self.lr, self.momentum, self.wd, 1.0 / self.world, **kw)
        if self.fused_lo:
            for l, ok in zip(layers, fusable):
                if not ok:
                    self._split_weight(l)

    def _update_layers(self, layers):
        """Exchange + optimiser for these layers on the library's current stream."""
        h = self.h
        if self.sharded:
            # one kernel per layer: reduce-scatter, SGD on this rank's shard, all-gather of the updated weights
            for l in layers:
                start, count = self.layer_span[l]
                n_w = self.dims[l] * self.dims[l + 1]
                fusable = self.fused_lo and self.dims[l + 1] % 4 == 0
                h.dp_p2p_sgd_step(start, self.numel + start, count, self.V.data_ptr() + 4 * start,
                                  self.W_lo[l].data_ptr() if fusable else 0, n_w if fusable else 0, self.lr, self.momentum,
                                  self.wd, 1.0 / self.world)
                if self.fused_lo and not fusable:
                    self._split_weight(l)
            return
        if self.world > 1:
            if len(layers) == self.L:
                self._allreduce(0, self.numel)
            else:
                for l in layers:
                    self._allreduce(*self.layer_span[l])
        self._sgd_layers(layers)

    def _exchange_layer(self, l: int):
        """Side stream: wait for layer l's gradients (and for every GEMM that still reads W[l]), exchange them over
        the ranks and update that layer's slice.  The main stream goes on meanwhile; the next forward pass of layer
        l waits for the event recorded here."""
        main = torch.cuda.current_stream(self.dev)
        ev = torch.cuda.Event()
        ev.record(main)
        self._side.wait_event(ev)
        h = self.h
        h.set_stream(self._side.cuda_stream)
        self._update_layers([l])
        done = torch.cuda.Event()
        done.record(self._side)
        self._upd_ev[l] = done
        h.set_stream(main.cuda_stream)

    def _dW(self, l: int):
        """dW = X^T . dY, db = column sum of dY (same call)."""
        lo = self.fused_lo
        self.h.gemm_ex(self.dims[l], self.dims[l + 1], self.batch, self._m(self.act[l], transpose=True), self._m(self.gout[l]),
                       self.dW[l].data_ptr(), algo=self.algo, colsum=self.db[l].data_ptr(),
                       a_lo=self.act_lo[l].data_ptr() if lo else 0, b_lo=self.gout_lo[l].data_ptr() if lo else 0)

    def _dX(self, l: int):
        """dX = (dY . W^T) * mask: the ReLU backward rides in the epilogue, and so does the lo plane of the result,
        which is the layer below's dY."""
        lo = self.fused_lo
        self.h.gemm_ex(self.batch, self.dims[l], self.dims[l + 1], self._m(self.gout[l]), self._m(self.W[l], transpose=True),
                       self.gout[l - 1].data_ptr(), algo=self.algo, mul_mask=self.mask[l - 1].data_ptr(),
                       a_lo=self.gout_lo[l].data_ptr() if lo else 0, b_lo=self.W_lo[l].data_ptr() if lo else 0,
                       c_lo=self.gout_lo[l - 1].data_ptr() if lo else 0)

    def _backward(self, exchange: bool = False):
        h, L, B = self.h, self.L, self.batch
        C = self.dims[-1]  # gout[L - 1] = dlogits was written with the loss
        if self.fused_lo:
            h.split_lo(self._m(self.gout[L - 1]), B, C, self.gout_lo[L - 1].data_ptr(), self.gout_lo[L - 1].numel())
        if not exchange:
            for l in range(L - 1, -1, -1):
                self._dW(l)
                if l > 0:  # the network input needs no gradient (matmul.mojo:34)
                    self._dX(l)
            return
        # Data parallel: the layer whose gradients are produced LAST is the one whose exchange nothing can hide.  In
        # the textbook order that is layer 0 -- the first the next forward pass needs.  So: the top layer's dW and
        # the whole dX chain first, then dW from the bottom layer up; the exchange left for last belongs to the
        # second-highest layer, which the next forward pass reaches only after the layers below it.
        self._dW(L - 1)
        for l in range(L - 1, 0, -1):
            self._dX(l)
            if l == L - 1:
                self._exchange_layer(L - 1)   # after dX has read W[L-1]
        if L == 1:
            self._exchange_layer(0)
        for l in range(0, L - 1):
            self._dW(l)
            self._exchange_layer(l)
        if self._join_each_step:
            torch.cuda.current_stream(self.dev).wait_stream(self._side)
            self._upd_ev = [None] * L

    def _update(self):
        self._update_layers(list(range(self.L)))

    # ------------------------------------------------------------------------------------------------
    def _use_set(self, k: int):
        super()._use_set(k)
        self.act[0] = self.X
        if self.fused_lo:
            self.act_lo[0] = self._x_lo[k]

    def step(self, X=None, y=None, update: bool = True):
        """One training step, eagerly enqueued.  Returns nothing; read ``loss`` / ``logits()`` afterwards."""
        self._begin_step(X, y)
        self._enqueue(update)
        self._end_step()

    def capture(self):
        """Record the step once into a CUDA graph; ``replay()`` then costs one launch per step."""
        if self._loaded is not None:  # a batch uploaded for the next step becomes the captured set
            torch.cuda.current_stream(self.dev).wait_event(self._set_ready[self._loaded])
            self._use_set(self._loaded)
            self._loaded = None
        self._join_each_step = True
        side = torch.cuda.Stream(self.dev)
        side.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(side):
            self.h.set_stream(side.cuda_stream)
            snap = (self.P.clone(), self.V.clone())
            for _ in range(2):  # warm up: grow the workspace and load every kernel before capture
                self._enqueue(True)
            side.synchronize()
            self.P.copy_(snap[0])
            self.V.copy_(snap[1])
            self._refresh_weight_lo()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                self._enqueue(True)
        torch.cuda.current_stream(self.dev).wait_stream(side)
        self.P.copy_(snap[0])  # the capture itself does not run, but keep the state explicit
        self.V.copy_(snap[1])
        self.h.set_stream(torch.cuda.current_stream(self.dev).cuda_stream)
        self._refresh_weight_lo()

    def _refresh_weight_lo(self):
        """The weights changed behind the step's back (restore, checkpoint load): redo their lo planes."""
        if self.fused_lo:
            for l in range(self.L):
                self._split_weight(l)

    def replay(self):
        self.graph.replay()

    # ------------------------------------------------------------------------------------------------
    def logits(self) -> np.ndarray:
        return self.act[self.L].detach().cpu().numpy()

    def loss_value(self) -> float:
        return float(self.loss.item())

    def accuracy(self) -> int:
        self.h.set_stream(torch.cuda.current_stream(self.dev).cuda_stream)
        C = self.dims[-1]
        return self.h.accuracy(self.act[self.L].data_ptr(), C, self.y.data_ptr(), True, self.batch, C, self.correct.data_ptr())

    def weights(self):
        return [w.detach().cpu().numpy() for w in self.W]

    def biases(self):
        return [b.detach().cpu().numpy() for b in self.b]

    def flops_per_step(self) -> float:
        """Algorithmic flop of one step on this rank: forward + dW for every layer, dX for layers 2..L."""
        f = 0.0
        for l in range(self.L):
            mnk = self.batch * self.dims[l] * self.dims[l + 1]
            f += 2.0 * mnk * (3 if l > 0 else 2)
        return f

    def state_dict(self) -> dict:
        """Parameters under the reference's checkpoint names ("<idx>.weight"/"<idx>.bias" with the module
        index of Sequential(Linear, ReLU, ...), numpy_interop.mojo:166-196) plus the SGD velocities."""
        out = {}
        for l in range(self.L):
            out[f"{2 * l}.weight"] = self.W[l].detach().cpu().numpy()
            out[f"{2 * l}.bias"] = self.b[l].detach().cpu().numpy()
        out["__velocity__"] = self._full_velocity().cpu().numpy()
        return out

    def _full_velocity(self) -> torch.Tensor:
        """With the optimiser sharded over the ranks each rank holds the momentum of its own shards only (zeros
        elsewhere): the sum over the ranks is the whole buffer.  Every rank must call this together; the gradient
        bucket, idle between steps, carries the sum."""
        if not self.sharded:
            return self.V.detach().clone()
        torch.cuda.synchronize(self.dev)
        self.h.set_stream(torch.cuda.current_stream(self.dev).cuda_stream)
        self.G.copy_(self.V)
        self.h.dp_p2p_allreduce_sum(0, self.numel)
        full = self.G.detach().clone()
        torch.cuda.synchronize(self.dev)
        return full

    def _own_shard_mask(self) -> torch.Tensor:
        """1.0 where this rank owns the optimiser state (the shards tenmo_dp_p2p_sgd_step_f32 deals per layer)."""
        m = torch.zeros(self.numel, dtype=torch.float32, device=f"cuda:{self.dev}")
        for start, count in self.layer_span:
            lo, hi = optimizer_shard(count, self.rank, self.world)
            m[start + lo:start + hi] = 1.0
        return m

    def load_state_dict(self, sd: dict):
        for l in range(self.L):
            self.W[l].copy_(torch.from_numpy(np.ascontiguousarray(sd[f"{2 * l}.weight"], np.float32)))
            self.b[l].copy_(torch.from_numpy(np.ascontiguousarray(sd[f"{2 * l}.bias"], np.float32)))
        if "__velocity__" in sd:
            self.V.copy_(torch.from_numpy(np.ascontiguousarray(sd["__velocity__"], np.float32)))
            if self.sharded:  # keep the momentum of the own shards only
                self.V.mul_(self._own_shard_mask())
        self.h.set_stream(torch.cuda.current_stream(self.dev).cuda_stream)
        self._refresh_weight_lo()


__all__ = ["MLPTrainer", "shard_rows"]
