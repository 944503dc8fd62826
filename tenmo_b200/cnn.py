"""Conv2d (as an implicit GEMM) and MaxPool2d over the C ABI, NCHW, plus the CIFAR-shaped CNN training step.

The reference's Conv2D (tenmo/cnn.mojo:18-271, net.mojo) pads, then runs a direct convolution; its backward uses an
explicit im2col + matmul for the kernel gradient and a scatter for the input gradient.  Here each direction is one
call whose kernel gathers the patch operand from a shared-memory copy of the image region it needs, so no patch
matrix ever exists in device memory:

  forward   out = relu(conv(x, W) + b) with the bias as the accumulators' start value and the 0/1 mask from the epilogue
  backward  dW, db = conv2d_bwd_weight(x, g * mask);  dx = conv2d_bwd_input(g * mask, W)   (the mask multiply rides in
            the kernels' loads)
"""
from __future__ import annotations

import numpy as np
import torch

from . import lib as _lib
from .lib import TenmoCuda, make_mat
from .trainer import BatchFeed


def out_size(n: int, k: int, stride: int, dilation: int, pad: int) -> int:
    return (n + 2 * pad - ((k - 1) * dilation + 1)) // stride + 1


class Conv2d:
    """One convolution layer with pre-planned buffers for a fixed batch."""

    def __init__(self, h: TenmoCuda, N, Cin, H, W, Cout, k, stride=1, dilation=1, pad=0, relu=False, device=0,
                 need_dx=True):
        self.h, self.N, self.Cin, self.H, self.W, self.Cout, self.k = h, N, Cin, H, W, Cout, k
        self.stride, self.dil, self.pad, self.relu, self.need_dx = stride, dilation, pad, relu, need_dx
        self.Ho, self.Wo = out_size(H, k, stride, dilation, pad), out_size(W, k, stride, dilation, pad)
        f32 = dict(dtype=torch.float32, device=f"cuda:{device}")
        self.out = torch.empty(N, Cout, self.Ho, self.Wo, **f32)
        self.mask = torch.empty(N, Cout, self.Ho, self.Wo, **f32) if relu else None
        self.dx = torch.empty(N, Cin, H, W, **f32) if need_dx else None
        self.x = None

    def _geom(self):
        return (self.N, self.Cin, self.H, self.W), (self.Cout, self.k, self.k, self.stride, self.dil, self.pad)

    def forward(self, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
        (N, Cin, H, W), (Cout, kh, kw, stride, dil, pad) = self._geom()
        self.x = x  # the kernel gradient reads the layer input again
        self.h.conv2d_fwd(x.data_ptr(), N, Cin, H, W, weight.data_ptr(), bias.data_ptr() if bias is not None else 0, Cout, kh, kw,
                          stride, dil, pad, _lib.ACT_RELU if self.relu else _lib.ACT_NONE, self.out.data_ptr(),
                          self.mask.data_ptr() if self.relu else 0)
        return self.out

    def backward(self, g: torch.Tensor, weight: torch.Tensor, dW: torch.Tensor, db: torch.Tensor):
        """g is dL/d(out) AFTER the activation; with relu=True the kernels multiply it by the mask as they load it."""
        (N, Cin, H, W), (Cout, kh, kw, stride, dil, pad) = self._geom()
        mask = self.mask.data_ptr() if self.relu else 0
        self.h.conv2d_bwd_weight(self.x.data_ptr(), g.data_ptr(), mask, N, Cin, H, W, Cout, kh, kw, stride, dil, pad,
                                 dW.data_ptr(), db.data_ptr())
        if self.need_dx:
            self.h.conv2d_bwd_input(g.data_ptr(), mask, weight.data_ptr(), N, Cin, H, W, Cout, kh, kw, stride, dil, pad,
                                    self.dx.data_ptr())
        return self.dx


class MaxPool2d:
    def __init__(self, h: TenmoCuda, N, C, H, W, k=2, stride=2, pad=0, device=0):
        self.h, self.N, self.C, self.H, self.W, self.k, self.stride, self.pad = h, N, C, H, W, k, stride, pad
        self.Ho, self.Wo = (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1
        dev = f"cuda:{device}"
        self.out = torch.empty(N, C, self.Ho, self.Wo, dtype=torch.float32, device=dev)
        self.argmax = torch.empty(N, C, self.Ho, self.Wo, dtype=torch.int64, device=dev)
        self.dx = torch.empty(N, C, H, W, dtype=torch.float32, device=dev)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        self.h.maxpool2d_fwd(x.data_ptr(), self.N, self.C, self.H, self.W, self.k, self.stride, self.pad, self.out.data_ptr(),
                             self.argmax.data_ptr())
        return self.out

    def backward(self, g: torch.Tensor) -> torch.Tensor:
        self.h.maxpool2d_bwd(g.data_ptr(), self.argmax.data_ptr(), self.N, self.C, self.H, self.W, self.Ho, self.Wo,
                             self.dx.data_ptr())
        return self.dx


class CNNTrainer(BatchFeed):
    """The CIFAR-shaped CNN of the reference's examples as one planned step: conv3x3(3->32, pad 1) + ReLU,
    maxpool 2, conv3x3(32->64, pad 1) + ReLU, maxpool 2, flatten (NCHW order), Linear 4096->10, softmax
    cross-entropy, SGD momentum.  Parameters, gradients and velocities live in flat buffers so that the
    data-parallel exchange is one all-reduce and the update one launch."""

    def __init__(self, params: dict, batch: int, hw: int = 32, lr: float = 0.01, momentum: float = 0.9,
                 handle: TenmoCuda | None = None, rank: int = 0, world: int = 1, unique_id: bytes | None = None,
                 device: int | None = None, exchange: str = "nccl", all_gather_bytes=None):
        """exchange: "nccl" (needs unique_id) or "p2p" (the library's peer-memory kernel; needs all_gather_bytes)."""
        self.dev = torch.cuda.current_device() if device is None else device
        self.h = handle or TenmoCuda(self.dev).require()
        self.rank, self.world, self.lr, self.momentum, self.batch = rank, world, float(lr), float(momentum), int(batch)
        f32 = dict(dtype=torch.float32, device=f"cuda:{self.dev}")
        names = ["conv1.weight", "conv1.bias", "conv2.weight", "conv2.bias", "fc.weight", "fc.bias"]
        shapes = [tuple(np.shape(params[n])) for n in names]
        offs, off = [], 0
        for s in shapes:
            offs.append(off)
            off += (int(np.prod(s)) + 3) // 4 * 4
        self.numel = off
        self.exchange = exchange if world > 1 else "none"
        self.P, self.V = (torch.zeros(off, **f32) for _ in range(2))
        if self.exchange == "p2p":
            from .parallel import DeviceFloats, connect_peer_buckets

            ptr = connect_peer_buckets(self.h, off, rank, world, all_gather_bytes)
            self.G = torch.as_tensor(DeviceFloats(ptr, off), device=f"cuda:{self.dev}")
        else:
            self.G = torch.zeros(off, **f32)
        view = lambda buf, i: buf[offs[i]:offs[i] + int(np.prod(shapes[i]))].view(*shapes[i])
        self.p = {n: view(self.P, i) for i, n in enumerate(names)}
        self.g = {n: view(self.G, i) for i, n in enumerate(names)}
        for n in names:
            self.p[n].copy_(torch.from_numpy(np.ascontiguousarray(params[n], np.float32)))
        B, C1, C2 = self.batch, shapes[0][0], shapes[2][0]
        h = self.h
        self.conv1 = Conv2d(h, B, shapes[0][1], hw, hw, C1, shapes[0][2], pad=1, relu=True, device=self.dev, need_dx=False)
        self.pool1 = MaxPool2d(h, B, C1, hw, hw, device=self.dev)
        self.conv2 = Conv2d(h, B, C1, hw // 2, hw // 2, C2, shapes[2][2], pad=1, relu=True, device=self.dev)
        self.pool2 = MaxPool2d(h, B, C2, hw // 2, hw // 2, device=self.dev)
        self.feat = C2 * (hw // 4) * (hw // 4)
        self.classes = shapes[4][1]
        assert shapes[4][0] == self.feat, "fc.weight rows must equal the flattened feature count"
        self._feed_init((B, shapes[0][1], hw, hw), self.dev)   # two sets of input buffers (BatchFeed)
        self.logits = torch.empty(B, self.classes, **f32)
        self.softmax = torch.empty(B, self.classes, **f32)
        self.dlogits = torch.empty(B, self.classes, **f32)
        self.dfeat = torch.empty(B, self.feat, **f32)
        self.loss = torch.zeros(1, **f32)
        self.valid = torch.zeros(1, dtype=torch.int32, device=f"cuda:{self.dev}")
        self.correct = torch.zeros(1, dtype=torch.int64, device=f"cuda:{self.dev}")
        if self.exchange == "nccl":
            self.h.dp_init(rank, world, unique_id)
        torch.cuda.synchronize(self.dev)

    def step(self, X=None, y=None, update: bool = True):
        h, B, C = self.h, self.batch, self.classes
        self._begin_step(X, y)
        p, g = self.p, self.g
        a1 = self.pool1.forward(self.conv1.forward(self.X, p["conv1.weight"], p["conv1.bias"]))
        a2 = self.pool2.forward(self.conv2.forward(a1, p["conv2.weight"], p["conv2.bias"]))
        flat = make_mat(a2.data_ptr(), (B, self.feat), (self.feat, 1))            # Flatten: NCHW order, a view
        mWfc = make_mat(p["fc.weight"].data_ptr(), (self.feat, C), (C, 1))
        h.gemm_ex(B, C, self.feat, flat, mWfc, self.logits.data_ptr(), algo=_lib.ALGO_SIMT_FP32, bias=p["fc.bias"].data_ptr())
        h.ce_fwd_bwd(self.logits.data_ptr(), C, self.y.data_ptr(), True, B, C, -100, 0.0, 0, self.softmax.data_ptr(),
                     self.loss.data_ptr(), self.valid.data_ptr(), 0, self.dlogits.data_ptr())
        mdl = make_mat(self.dlogits.data_ptr(), (B, C), (C, 1))
        h.gemm_ex(self.feat, C, B, make_mat(a2.data_ptr(), (self.feat, B), (1, self.feat)), mdl, g["fc.weight"].data_ptr(),
                  algo=_lib.ALGO_SIMT_FP32, colsum=g["fc.bias"].data_ptr())
        h.gemm_ex(B, self.feat, C, mdl, make_mat(p["fc.weight"].data_ptr(), (C, self.feat), (1, C)), self.dfeat.data_ptr(),
                  algo=_lib.ALGO_SIMT_FP32)
        d2 = self.pool2.backward(self.dfeat)                                       # (B, C2, 16, 16)
        d1p = self.conv2.backward(d2, p["conv2.weight"], g["conv2.weight"], g["conv2.bias"])
        d1 = self.pool1.backward(d1p)
        self.conv1.backward(d1, p["conv1.weight"], g["conv1.weight"], g["conv1.bias"])
        if update:
            if self.exchange == "p2p":
                h.dp_p2p_allreduce_sum(0, self.numel)
            elif self.exchange == "nccl":
                h.dp_allreduce_sum(self.G.data_ptr(), self.numel)
            h.sgd_step([self.P.data_ptr()], [self.G.data_ptr()], [self.V.data_ptr()], [self.numel], self.lr, self.momentum,
                       0.0, 1.0 / self.world)
        self._end_step()

    def close(self):
        """Release the data-parallel resources (every rank, after a host barrier)."""
        if self.exchange == "p2p":
            torch.cuda.synchronize(self.dev)
            self.G = None
            self.g = None
            self.h.dp_p2p_close()
        elif self.exchange == "nccl":
            self.h.dp_finalize()
        self.exchange = "none"

    def loss_value(self) -> float:
        return float(self.loss.item())

    def accuracy(self) -> int:
        return self.h.accuracy(self.logits.data_ptr(), self.classes, self.y.data_ptr(), True, self.batch, self.classes,
                               self.correct.data_ptr())

    def params(self) -> dict:
        return {n: t.detach().cpu().numpy() for n, t in self.p.items()}

    def grads(self) -> dict:
        return {n: t.detach().cpu().numpy() for n, t in self.g.items()}

    # Module index of each parameterised layer inside Sequential(Conv2D, ReLU, MaxPool2d, Conv2D, ReLU, MaxPool2d, Flatten,
    # Linear): the reference names checkpoint entries "<index>.weight" / "<index>.bias" (numpy_interop.mojo:166-196;
    # tests/test_checkpoint.mojo:41-54 shows the numbering skipping layers without parameters).
    _CKPT_INDEX = {"conv1": 0, "conv2": 3, "fc": 7}

    def state_dict(self) -> dict:
        """Parameters under the reference's checkpoint names plus the SGD velocities (flat, in parameter order)."""
        torch.cuda.synchronize(self.dev)
        out = {}
        for n, t in self.p.items():
            layer, kind = n.split(".")
            out[f"{self._CKPT_INDEX[layer]}.{kind}"] = t.detach().cpu().numpy().copy()
        out["__velocity__"] = self.V.detach().cpu().numpy().copy()
        return out

    def load_state_dict(self, sd: dict):
        for n, t in self.p.items():
            layer, kind = n.split(".")
            src = np.ascontiguousarray(sd[f"{self._CKPT_INDEX[layer]}.{kind}"], np.float32)
            if src.shape != tuple(t.shape):
                raise ValueError(f"checkpoint entry for {n} has shape {src.shape}, the model holds {tuple(t.shape)}")
            t.copy_(torch.from_numpy(src))
        if "__velocity__" in sd:
            self.V.copy_(torch.from_numpy(np.ascontiguousarray(sd["__velocity__"], np.float32)))
        torch.cuda.synchronize(self.dev)
