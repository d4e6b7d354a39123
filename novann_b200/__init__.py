"""novann_b200: B200-native (sm_100a) casts, FP8 / FP4 quantisation, quantised Linear / Conv2d
and the fp32 layers of NovaNN's CNN for NovaNN's NumPy-array API, over the C ABI in
``include/nvq.h``.

No layer arithmetic runs on the CPU: every operation calls ``libnvq.so`` and fails loudly if
the library or a GPU is missing.  (``Dropout`` draws its keep mask from NumPy's generator on
the host, as the reference does, so that seeded runs drop the same units; ``Flatten`` is a
reshape.)"""
from . import functional, quant  # noqa: F401
from .layers import (BatchNorm1d, BatchNorm2d, Conv2d, Dropout, Flatten, GlobalAvgPool2d,  # noqa: F401
                     Linear, MaxPool2d, QuantConv2d, QuantLinear, ReLU)
from .losses import CrossEntropyLoss  # noqa: F401
from .model import Sequential  # noqa: F401
from .module import Layer, Module, Parameters  # noqa: F401
from .optim import SGD, AdamW  # noqa: F401
from .compat import register_if_imported, register_with_novann  # noqa: F401

register_if_imported()

__all__ = ["functional", "quant", "Linear", "QuantLinear", "ReLU", "Conv2d", "QuantConv2d",
           "BatchNorm1d", "BatchNorm2d", "MaxPool2d", "GlobalAvgPool2d", "Flatten", "Dropout",
           "Sequential", "CrossEntropyLoss", "SGD", "AdamW", "Layer", "Module", "Parameters",
           "register_with_novann"]
