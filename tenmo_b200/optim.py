"""SGD with momentum and weight decay (tenmo/optim.mojo:405-581, 123-158)."""
from __future__ import annotations

from .tensor import NDBuffer, handle, panic


class SGD:
    """``SGD(parameters, lr, momentum=0, weight_decay=0)``; ``step()`` updates every parameter that has a
    gradient in ONE kernel launch (the reference launches once per tensor), ``zero_grad()`` clears the
    gradboxes.  Velocities start at zero, one per parameter (optim.mojo:45-70).  Gradient clipping
    (clip_norm / clip_value) is not on this path and raises."""

    def __init__(self, parameters, lr: float = 0.01, momentum: float = 0.0, weight_decay: float = 0.0,
                 clip_norm: float = 0.0, clip_value: float = 0.0):
        if clip_norm or clip_value:
            panic("SGD: gradient clipping is outside the dense training path implemented here")
        self.parameters = list(parameters)
        self.lr, self.momentum, self.weight_decay = float(lr), float(momentum), float(weight_decay)
        self.velocities = [NDBuffer.zeros(p.shape()) for p in self.parameters] if momentum > 0 else None

    def step(self, grad_scale: float = 1.0):
        idx = [i for i, p in enumerate(self.parameters) if p.gradbox is not None]
        if not idx:
            return
        ps = [self.parameters[i].buffer.data_ptr() for i in idx]
        gs = [self.parameters[i].gradbox.data_ptr() for i in idx]
        vs = [self.velocities[i].data_ptr() for i in idx] if self.velocities else None
        ns = [self.parameters[i].buffer.numels() for i in idx]
        handle().sgd_step(ps, gs, vs, ns, self.lr, self.momentum, self.weight_decay, grad_scale)

    def zero_grad(self):
        for p in self.parameters:
            p.zero_grad()
