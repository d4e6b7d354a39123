"""Use of the GPU-backed layers inside the reference's own containers.

NovaNN's ``Sequential`` decides which layers it initialises with
``isinstance(layer, (Linear, Conv1d, Conv2d))`` and which layers are activations with
``isinstance(layer, Activation)`` (novann/model/nn.py:36-38,79-83), then calls
``layer.reset_parameters(init_fn)`` (novann/model/nn.py:143).  NovaNN's layer classes derive
from ``abc.ABC`` (novann/module/layer.py:6), so they accept virtual subclasses:
``register_with_novann()`` registers ``novann_b200``'s ``Linear`` / ``QuantLinear`` under NovaNN's
``Linear``, ``Conv2d`` / ``QuantConv2d`` under its ``Conv2d``, ``ReLU`` under its ``ReLU`` (and so
``Activation``), and every layer under its ``Layer``.  After that a
``novann.Sequential(novann_b200.Linear(...), novann.ReLU(), novann_b200.QuantLinear(...))`` is
auto-initialised, trained by ``novann.utils.train.train`` and stepped by NovaNN's optimisers
exactly like a model of NovaNN's own layers.  Nothing of NovaNN is imported unless this
function is called (or ``novann`` was imported before ``novann_b200``).
"""
from __future__ import annotations

import sys

_registered = False


def register_with_novann(novann=None) -> bool:
    """Registers the GPU-backed layers as virtual subclasses of NovaNN's.  ``novann`` is the
    imported reference package (imported here when omitted).  Returns True once registered."""
    global _registered
    if _registered:
        return True
    if novann is None:
        import novann  # noqa: F811  (the reference must be importable for this to make sense)
    from novann import layers as ref_layers
    from novann.layers.activations import Activation as RefActivation
    from novann.module import Layer as RefLayer

    from . import layers as L
    from .model import Sequential

    ref_layers.Linear.register(L.Linear)            # QuantLinear derives from Linear
    ref_layers.Conv2d.register(L.Conv2d)            # QuantConv2d derives from Conv2d
    ref_layers.ReLU.register(L.ReLU)
    RefActivation.register(L.ReLU)
    for name in ("BatchNorm1d", "BatchNorm2d", "MaxPool2d", "GlobalAvgPool2d", "Flatten", "Dropout"):
        getattr(ref_layers, name).register(getattr(L, name))
    for cls in (L.Linear, L.Conv2d, L.ReLU, L.BatchNorm1d, L.BatchNorm2d, L.MaxPool2d,
                L.GlobalAvgPool2d, L.Flatten, L.Dropout, Sequential):
        RefLayer.register(cls)
    _registered = True
    return True


def register_if_imported() -> bool:
    """Registers when the reference package is already loaded in this process."""
    if "novann" in sys.modules and hasattr(sys.modules["novann"], "layers"):
        try:
            return register_with_novann(sys.modules["novann"])
        except Exception:
            return False
    return False
