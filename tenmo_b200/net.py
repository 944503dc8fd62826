"""Linear / ReLU / Sigmoid / Sequential (tenmo/net.mojo:49-216, 692-698, 1069-1181)."""
from __future__ import annotations

import math

import numpy as np

from .tensor import Tensor, panic


class Linear:
    """Fully connected layer ``y = x W + b`` with W of shape (in_features, out_features) (net.mojo:49-216).
    The reference draws weights from Mojo's own random stream, which cannot be reproduced elsewhere, so
    the initialisers take a NumPy generator seeded with ``init_seed``; tests pass explicit arrays instead."""

    def __init__(self, in_features: int, out_features: int, init_seed=None, init_method: str = "standard",
                 bias: bool = True, bias_zero: bool = True):
        self.in_features, self.out_features = in_features, out_features
        self.training = True
        rng = np.random.default_rng(init_seed)
        if init_method == "xavier":  # net.mojo:87-116
            limit = math.sqrt(6.0 / (in_features + out_features))
            w = rng.uniform(-limit, limit, (in_features, out_features))
            b = rng.uniform(-limit, limit, out_features)
        elif init_method == "he":  # net.mojo:118-147
            std = math.sqrt(2.0 / in_features)
            w = rng.normal(0.0, std, (in_features, out_features))
            b = rng.normal(0.0, std * 0.01, out_features)
        else:  # "standard": U(-0.1, 0.1)
            w = rng.uniform(-0.1, 0.1, (in_features, out_features))
            b = rng.uniform(-0.1, 0.1, out_features)
        self.weight = Tensor.from_numpy(w.astype(np.float32), requires_grad=True)
        self.bias = None
        if bias:
            self.bias = Tensor.from_numpy((np.zeros(out_features) if bias_zero else b).astype(np.float32),
                                          requires_grad=True)

    def __call__(self, xs: Tensor) -> Tensor:
        if xs.shape()[-1] != self.weight.shape()[0]:
            panic("Linear forward: input dim mismatch: input shape ->", xs.shape(), "and weights shape ->",
                  self.weight.shape())
        out = xs.matmul(self.weight, track_grad=self.training)
        if self.bias is not None:
            out = out.add_bias(self.bias, track_grad=self.training)
        return out

    def parameters(self):
        return [self.weight] + ([self.bias] if self.bias is not None else [])


class ReLU:
    training = True

    def __call__(self, xs: Tensor) -> Tensor:
        return xs.relu(track_grad=self.training)

    def parameters(self):
        return []


class Sigmoid:
    training = True

    def __call__(self, xs: Tensor) -> Tensor:
        return xs.sigmoid(track_grad=self.training)

    def parameters(self):
        return []


class Sequential:
    def __init__(self, *modules):
        self.modules = list(modules)

    def __call__(self, xs: Tensor) -> Tensor:
        for m in self.modules:
            xs = m(xs)
        return xs

    def parameters(self):
        return [p for m in self.modules for p in m.parameters()]

    def train(self):
        for m in self.modules:
            m.training = True

    def eval(self):
        for m in self.modules:
            m.training = False

    def named_parameters(self, prefix: str = ""):
        """Names as the reference's checkpoints use them: "<idx>.weight", "<idx>.bias" (net.mojo:235-244,1102-1109)."""
        out = {}
        for i, m in enumerate(self.modules):
            if isinstance(m, Linear):
                out[f"{prefix}{i}.weight"] = m.weight
                if m.bias is not None:
                    out[f"{prefix}{i}.bias"] = m.bias
        return out
