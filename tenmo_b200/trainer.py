"""A whole Linear/ReLU/softmax-CE/SGD training step as one pre-planned sequence of C-ABI calls.

This is the call sequence tenmo's host makes for ``Sequential(Linear, ReLU, ..., Linear)`` +
``CrossEntropyLoss`` + ``SGD`` (net.mojo:1085-1092, crossentropy.mojo:1360-1391, tensor.mojo:3154-3247,
optim.mojo:405-543) with the host round trips taken out so that it can be replayed as a CUDA graph:

  forward   per layer ONE GEMM with the bias add, ReLU and the 0/1 mask in its epilogue
  loss      fused cross-entropy forward + backward, loss and valid count stay on the device
  backward  per layer dW = X^T . dY (db rides along as the column sum of dY) and dX = dY . W^T on
            transposed stride views, then the ReLU mask multiply
  exchange  (data parallel) one NCCL sum all-reduce of the flat gradient bucket
  update    ONE SGD-momentum launch over the flat parameter / gradient / velocity buffers,
            1/world folded into it

All parameters live in one flat buffer (weights and biases back to back), and so do gradients and
velocities, which is what makes the single all-reduce and the single optimizer launch possible.
"""
from __future__ import annotations

import numpy as np
import torch

from . import lib as _lib
from .lib import TenmoCuda, make_mat
from .parallel import shard_rows


class MLPTrainer:
    def __init__(self, weights, biases, batch: int, lr: float = 0.01, momentum: float = 0.9, weight_decay: float = 0.0,
                 algo: str = "auto", handle: TenmoCuda | None = None, rank: int = 0, world: int = 1,
                 unique_id: bytes | None = None, device: int | None = None, overlap: bool = True,
                 reserve_sms: int = 0, exchange: str = "nccl", all_gather_bytes=None):
        """exchange: "nccl" (tenmo_dp_allreduce_sum_f32; needs unique_id) or "p2p" (the library's own kernel over NVLink
        peer memory; needs all_gather_bytes(data) -> [bytes per rank] to share the IPC handles of the gradient bucket)."""
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
        if self.exchange not in ("none", "nccl", "p2p"):
            raise ValueError(f"unknown exchange {exchange!r}")
        self.P = torch.zeros(off, **f32)
        if self.exchange == "p2p":
            # the gradient bucket lives in memory the library allocated and every peer has mapped
            from .parallel import DeviceFloats, connect_peer_buckets

            ptr = connect_peer_buckets(self.h, off, rank, world, all_gather_bytes)
            self.G = torch.as_tensor(DeviceFloats(ptr, off), device=f"cuda:{self.dev}")
        else:
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
        self.X = torch.zeros(B, self.dims[0], **f32)
        self.y = torch.zeros(B, dtype=torch.int64, device=f"cuda:{self.dev}")
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
            self.gout_lo = [torch.empty(B * r4(d), **f32) for d in self.dims[1:]]
        self.softmax = torch.empty(B, self.dims[-1], **f32)
        self.loss = torch.zeros(1, **f32)
        self.valid = torch.zeros(1, dtype=torch.int32, device=f"cuda:{self.dev}")
        self.correct = torch.zeros(1, dtype=torch.int64, device=f"cuda:{self.dev}")
        self.graph = None
        self._stream = None
        # [start, count) of each layer's weight + bias inside the flat buffers
        self.layer_span = [(offs[2 * l], offs[2 * l + 1] + (sizes[2 * l + 1] + 3) // 4 * 4 - offs[2 * l])
                           for l in range(self.L)]
        self.overlap = overlap and world > 1
        self._side = torch.cuda.Stream(self.dev) if self.overlap else None
        self.reserve_sms = int(reserve_sms) if self.overlap else 0
        if self.exchange == "nccl":
            self.h.dp_init(rank, world, unique_id)
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
        for l in range(L):
            last = l == L - 1
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
        if self.exchange == "p2p":
            self.h.dp_p2p_allreduce_sum(start, count)
        else:
            self.h.dp_allreduce_sum(self.G.data_ptr() + 4 * start, count)

    def close(self):
        """Release the data-parallel resources (every rank, after a host barrier)."""
        if self.exchange == "p2p":
            torch.cuda.synchronize(self.dev)
            self.G = None
            self.dW = self.db = None
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

    def _exchange_layer(self, l: int):
        """Side stream: wait for layer l's gradients (and for the dX GEMM that still reads W[l]), sum them over
        the ranks, apply SGD to that layer's slice.  The main stream goes on with layer l-1 meanwhile."""
        main = torch.cuda.current_stream(self.dev)
        ev = torch.cuda.Event()
        ev.record(main)
        self._side.wait_event(ev)
        start, count = self.layer_span[l]
        h = self.h
        h.set_stream(self._side.cuda_stream)
        self._allreduce(start, count)
        self._sgd_layers([l])
        h.set_stream(main.cuda_stream)

    def _backward(self, exchange: bool = False):
        h, L, B = self.h, self.L, self.batch
        C = self.dims[-1]  # gout[L - 1] = dlogits was written with the loss
        lo = self.fused_lo
        if lo:
            h.split_lo(self._m(self.gout[L - 1]), B, C, self.gout_lo[L - 1].data_ptr(), self.gout_lo[L - 1].numel())
        for l in range(L - 1, -1, -1):
            g = self.gout[l]
            g_lo = self.gout_lo[l].data_ptr() if lo else 0
            # dW = X^T . dY, db = column sum of dY (same call)
            h.gemm_ex(self.dims[l], self.dims[l + 1], B, self._m(self.act[l], transpose=True), self._m(g),
                      self.dW[l].data_ptr(), algo=self.algo, colsum=self.db[l].data_ptr(),
                      a_lo=self.act_lo[l].data_ptr() if lo else 0, b_lo=g_lo)
            if l > 0:  # the network input needs no gradient (matmul.mojo:34)
                # dX = (dY . W^T) * mask: the ReLU backward rides in the epilogue, and so does the lo plane of
                # the result, which is the next layer's dY
                h.gemm_ex(B, self.dims[l], self.dims[l + 1], self._m(g), self._m(self.W[l], transpose=True),
                          self.gout[l - 1].data_ptr(), algo=self.algo, mul_mask=self.mask[l - 1].data_ptr(),
                          a_lo=g_lo, b_lo=self.W_lo[l].data_ptr() if lo else 0,
                          c_lo=self.gout_lo[l - 1].data_ptr() if lo else 0)
            if exchange:
                self._exchange_layer(l)
        if exchange:  # the next step's forward reads the updated parameters
            torch.cuda.current_stream(self.dev).wait_stream(self._side)

    def _update(self):
        h = self.h
        if self.world > 1:
            self._allreduce(0, self.numel)
        self._sgd_layers(list(range(self.L)))

    # ------------------------------------------------------------------------------------------------
    def load_batch(self, X, y):
        """Copy a (batch, in) fp32 array and (batch,) int64 labels into the step's static input buffers
        (host arrays / pinned tensors are copied asynchronously on the current stream)."""
        if not torch.is_tensor(X):
            X = torch.from_numpy(np.ascontiguousarray(X, np.float32))
        if not torch.is_tensor(y):
            y = torch.from_numpy(np.ascontiguousarray(y, np.int64))
        self.X.copy_(X, non_blocking=True)
        self.y.copy_(y, non_blocking=True)

    def step(self, X=None, y=None, update: bool = True):
        """One training step, eagerly enqueued.  Returns nothing; read ``loss`` / ``logits()`` afterwards."""
        self.h.set_stream(torch.cuda.current_stream(self.dev).cuda_stream)
        if X is not None:
            self.load_batch(X, y)
        self._enqueue(update)

    def capture(self):
        """Record the step once into a CUDA graph; ``replay()`` then costs one launch per step."""
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
        out["__velocity__"] = self.V.detach().cpu().numpy()
        return out

    def load_state_dict(self, sd: dict):
        for l in range(self.L):
            self.W[l].copy_(torch.from_numpy(np.ascontiguousarray(sd[f"{2 * l}.weight"], np.float32)))
            self.b[l].copy_(torch.from_numpy(np.ascontiguousarray(sd[f"{2 * l}.bias"], np.float32)))
        if "__velocity__" in sd:
            self.V.copy_(torch.from_numpy(np.ascontiguousarray(sd["__velocity__"], np.float32)))
        self.h.set_stream(torch.cuda.current_stream(self.dev).cuda_stream)
        self._refresh_weight_lo()


__all__ = ["MLPTrainer", "shard_rows"]
