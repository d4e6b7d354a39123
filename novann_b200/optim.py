"""Vanilla ``SGD`` with the reference's contract (``novann/optim/sgd.py:6-87``, the path with
momentum 0, weight decay 0 and no clipping): ``p.data -= lr * p.grad`` on the GPU, written
back into the same NumPy arrays so the layers' ``Parameters`` stay the source of truth."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib
from .device import DeviceBuffer


class SGD:
    def __init__(self, parameters, lr: float, momentum: float = 0, weight_decay: float = 0,
                 max_grad_norm=None, device: int = 0) -> None:
        if momentum or weight_decay or max_grad_norm:
            raise NotImplementedError("only the vanilla SGD path (momentum 0, weight decay 0, "
                                      "no clipping) is built")
        self.params = list(parameters)
        self.lr = float(lr)
        self.device = device

    def step(self) -> None:
        for p in self.params:
            if p.grad is None:
                continue
            d = DeviceBuffer.from_numpy(np.ascontiguousarray(p.data, np.float32), self.device)
            g = DeviceBuffer.from_numpy(np.ascontiguousarray(p.grad, np.float32), self.device)
            check(lib().nvq_sgd_step_f32(d.at(0), g.at(0), p.data.size, C.c_float(self.lr),
                                         C.c_float(1.0), self.device, None))
            new = d.to_numpy(np.float32, p.data.shape)
            p.data[...] = new

    def zero_grad(self, set_to_none: bool = False) -> None:
        for p in self.params:
            p.zero_grad(set_to_none=set_to_none)


class AdamW:
    """``AdamW`` with the reference's contract (``novann/optim/adamw.py:6-69``): decoupled weight
    decay, skipped for parameters named ``gamma`` / ``beta``.  Moments live on the device."""

    def __init__(self, parameters, lr: float, betas=(0.9, 0.999), weight_decay: float = 0,
                 epsilon: float = 1e-8, device: int = 0) -> None:
        self.params = list(parameters)
        self.lr, self.wd = float(lr), float(weight_decay)
        self.b1, self.b2, self.eps = float(betas[0]), float(betas[1]), float(epsilon)
        self.device = device
        self.t = 0
        self._m = [DeviceBuffer(max(8, p.data.nbytes), device) for p in self.params]
        self._v = [DeviceBuffer(max(8, p.data.nbytes), device) for p in self.params]
        for b in self._m + self._v:
            b.zero()

    def step(self) -> None:
        self.t += 1
        for i, p in enumerate(self.params):
            if p.grad is None:
                continue
            decay = self.wd > 0 and getattr(p, "name", None) not in ("gamma", "beta")
            # float64 tensors (BatchNorm's gamma / beta) are stepped in float64, as NumPy would
            wide = p.data.dtype == np.float64
            dt, f = (np.float64, C.c_double) if wide else (np.float32, C.c_float)
            fn = lib().nvq_adamw_step_f64 if wide else lib().nvq_adamw_step_f32
            d = DeviceBuffer.from_numpy(np.ascontiguousarray(p.data, dt), self.device)
            g = DeviceBuffer.from_numpy(np.ascontiguousarray(p.grad, dt), self.device)
            check(fn(d.at(0), g.at(0), self._m[i].at(0), self._v[i].at(0), p.data.size,
                     f(self.b1), f(1 - self.b1), f(self.b2), f(1 - self.b2), f(1 - self.b1 ** self.t),
                     f(1 - self.b2 ** self.t), f(self.lr), f(self.eps), f(self.lr * self.wd), int(decay),
                     self.device, None))
            p.data[...] = d.to_numpy(dt, p.data.shape)

    def zero_grad(self, set_to_none: bool = False) -> None:
        for p in self.params:
            p.zero_grad(set_to_none=set_to_none)
