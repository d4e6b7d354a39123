"""The reference's module contract, restated: ``Parameters``, ``Module``, ``Layer``.

Mirrors ``novann/module/module.py:6-85`` and ``novann/module/layer.py:6-59`` so that the
GPU-backed layers in ``novann_b200.layers`` can be used wherever a NovaNN ``Layer`` is:
``forward`` / ``backward`` take and return ``np.ndarray``; parameters are ``Parameters``
objects with public mutable ``data``, ``grad`` and ``name``.
"""
from __future__ import annotations

from abc import ABC, abstractmethod

import numpy as np


class Parameters:
    def __init__(self, data: np.ndarray) -> None:
        self.data = data
        self.grad = np.zeros_like(self.data)
        self.name = None

    def zero_grad(self, set_to_none: bool = True) -> None:
        if set_to_none:
            self.grad = None
        elif self.grad is None:
            self.grad = np.zeros_like(self.data)
        else:
            self.grad.fill(0.0)


class Module:
    def __init__(self) -> None:
        self._training = True

    def train(self) -> None:
        self._training = True

    def eval(self) -> None:
        self._training = False

    def parameters(self):
        return []

    def zero_grad(self) -> None:
        for p in self.parameters():
            p.zero_grad()


class Layer(Module, ABC):
    def __call__(self, x: np.ndarray) -> np.ndarray:
        return self.forward(x)

    @abstractmethod
    def forward(self, x: np.ndarray) -> np.ndarray:
        raise NotImplementedError("Layer subclasses must implement forward method")

    @abstractmethod
    def backward(self, grad: np.ndarray) -> np.ndarray:
        raise NotImplementedError("Layer subclasses must implement backward method")
