"""CrossEntropyLoss for class-index targets (tenmo/crossentropy.mojo:1360-1391, 937-1083, 664-823)."""
from __future__ import annotations

import numpy as np
import torch

from .lib import REDUCTION
from .tensor import (BACKWARD_CE_CLASS_INDICES_INT32, BACKWARD_CE_CLASS_INDICES_INT64, Ancestry, NDBuffer, Tensor,
                     handle, panic)


class CrossEntropyLoss:
    """``criterion(logits, targets)`` with ``reduction`` in {"mean","sum","none"} (or 0/1/2), ``ignore_index``
    (default -100) and ``label_smoothing``.  Logits are (M, C); targets are int64 or int32 class indices."""

    def __init__(self, reduction="mean", ignore_index: int = -100, label_smoothing: float = 0.0):
        if isinstance(reduction, int):
            reduction = {0: "mean", 1: "sum", 2: "none"}[reduction]
        if reduction not in REDUCTION:
            panic("CrossEntropyLoss: unknown reduction", reduction)
        self.reduction = reduction
        self.ignore_index = ignore_index
        self.label_smoothing = float(label_smoothing)
        self.training = True

    def __call__(self, logits: Tensor, target: Tensor, validate: bool = True) -> Tensor:
        if len(logits.shape()) != 2:
            panic("CrossEntropyLoss: logits must be (M, C) on this path, got", logits.shape())
        M, C = logits.shape()
        if target.shape() != (M,):
            panic("CrossEntropyLoss: target shape", target.shape(), "does not match logits", logits.shape())
        tdt = target.buffer.storage.dtype
        if tdt not in (torch.int64, torch.int32):
            panic("CrossEntropyLoss: class-index targets must be int64 or int32")
        is_i64 = tdt == torch.int64
        x = logits.buffer.contiguous()
        track = self.training and logits.requires_grad
        softmax = NDBuffer.empty((M, C)) if track else None
        red = REDUCTION[self.reduction]
        loss = NDBuffer.empty((M,) if red == 2 else ())
        valid = torch.zeros(1, dtype=torch.int32, device="cuda")
        h = handle()
        h.ce_fwd(x.data_ptr(), C, target.buffer.data_ptr(), is_i64, M, C, self.ignore_index, self.label_smoothing, red,
                 softmax.data_ptr() if track else 0, loss.data_ptr(), valid.data_ptr())
        if validate:
            # the reference validates labels on the host before the kernel (crossentropy.mojo:114-134);
            # here the kernel flags a bad label and the host reads one status word
            h.check_device_status()
        out = Tensor(loss)
        if track:
            out.requires_grad = True
            code = BACKWARD_CE_CLASS_INDICES_INT64 if is_i64 else BACKWARD_CE_CLASS_INDICES_INT32
            out.ancestry = Ancestry(code, [logits], arg=dict(softmax=softmax, target=target.buffer, valid=valid,
                                                              reduction=red, ignore_index=self.ignore_index,
                                                              ls=self.label_smoothing, M=M, C=C, is_i64=is_i64))
        return out


def ce_class_indices_backward(output: Tensor, retain_graph: bool):
    """CEClassIndicesBackward (crossentropy.mojo:664-823): one fused kernel, valid count read on the device."""
    a = output.ancestry.arg
    (logits,) = output.ancestry.parents
    g = NDBuffer.empty((a["M"], a["C"]))
    handle().ce_bwd(a["softmax"].data_ptr(), a["target"].data_ptr(), a["is_i64"], a["M"], a["C"], a["ignore_index"],
                    a["ls"], a["reduction"], output.gradbox.data_ptr(), a["valid"].data_ptr(), g.data_ptr())
    if logits.requires_grad:
        logits.update_grad(g)
    if not retain_graph:
        output.gradbox.fill(0.0)
    return [logits]


class Accuracy:
    """Accuracy.compute (tenmo/accuracy.mojo:7-85): count of rows whose first-index argmax equals the label."""

    @staticmethod
    def compute(pred: Tensor, target: Tensor) -> int:
        M, C = pred.shape()
        x = pred.buffer.contiguous()
        cnt = torch.zeros(1, dtype=torch.int64, device="cuda")
        is_i64 = target.buffer.storage.dtype == torch.int64
        return handle().accuracy(x.data_ptr(), C, target.buffer.data_ptr(), is_i64, M, C, cnt.data_ptr())
