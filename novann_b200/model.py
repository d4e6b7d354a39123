"""``Sequential`` with the reference's contract (``novann/model/nn.py:185-223``): layers run
in order, gradients flow in reverse, ``parameters()`` lists weight then bias per layer."""
from __future__ import annotations

import numpy as np

from .module import Layer


class Sequential(Layer):
    def __init__(self, *layers: Layer) -> None:
        super().__init__()
        self._layers = list(layers)

    def train(self) -> None:
        super().train()
        for layer in self._layers:
            layer.train()

    def eval(self) -> None:
        super().eval()
        for layer in self._layers:
            layer.eval()

    def forward(self, x: np.ndarray) -> np.ndarray:
        for layer in self._layers:
            x = layer.forward(x)
        return x

    def backward(self, grad: np.ndarray) -> np.ndarray:
        for layer in reversed(self._layers):
            grad = layer.backward(grad)
        return grad

    def parameters(self):
        params = []
        for layer in self._layers:
            params.extend(layer.parameters())
        return params

    def zero_grad(self) -> None:
        for p in self.parameters():
            p.zero_grad()

    def __len__(self):
        return len(self._layers)

    def __getitem__(self, i):
        return self._layers[i]
