"""novann_b200: B200-native (sm_100a) casts, FP8 / FP4 quantisation and quantised Linear /
Conv2d for NovaNN's NumPy-array API, over the C ABI in ``include/nvq.h``.

Nothing here computes on the CPU: every operation calls ``libnvq.so`` and fails loudly if the
library or a GPU is missing."""
from . import functional, quant  # noqa: F401
from .layers import Conv2d, Linear, QuantConv2d, QuantLinear, ReLU  # noqa: F401
from .losses import CrossEntropyLoss  # noqa: F401
from .model import Sequential  # noqa: F401
from .module import Layer, Module, Parameters  # noqa: F401
from .optim import SGD, AdamW  # noqa: F401

__all__ = ["functional", "quant", "Linear", "QuantLinear", "ReLU", "Conv2d", "QuantConv2d",
           "Sequential", "CrossEntropyLoss", "SGD", "AdamW", "Layer", "Module", "Parameters"]
