"""``CrossEntropyLoss`` with the reference's contract (``novann/losses/loss_functions.py:8-75``),
computed on the GPU: ``loss, grad = loss_fn(logits, labels)``."""
from __future__ import annotations

import numpy as np

from . import functional as F


class CrossEntropyLoss:
    def __init__(self, device: int = 0) -> None:
        self.device = device
        self.N = 0
        self._loss = None
        self._grad = None

    def forward(self, logits: np.ndarray, targets: np.ndarray) -> np.float32:
        if targets.ndim != 1:
            targets = np.argmax(targets, axis=1)   # one-hot rows -> class indices
        self.N = logits.shape[0]
        self._loss, self._grad = F.softmax_ce_host(logits, targets, self.device)
        return np.float32(self._loss)

    def backward(self) -> np.ndarray:
        if self._grad is None:
            raise RuntimeError("forward must be called before backward")
        return self._grad

    def __call__(self, logits: np.ndarray, targets: np.ndarray):
        return self.forward(logits, targets), self.backward()
