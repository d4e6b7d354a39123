"""The GPU-backed layers inside the reference's own containers, as far as that goes without a
GPU: registration with NovaNN's classes, auto-initialisation by NovaNN's ``Sequential``
(novann/model/nn.py:79-143), parameter lists, modes.  No compute call is made here."""
import numpy as np
import pytest

import _reference

novann = _reference.import_novann()
pytestmark = pytest.mark.skipif(novann is None, reason="the reference package is not importable here")


def test_layers_are_instances_of_the_reference_classes():
    import novann_b200 as nb
    from novann.layers import Conv2d as RefConv2d, Linear as RefLinear, ReLU as RefReLU
    from novann.layers.activations import Activation
    from novann.module import Layer as RefLayer
    assert nb.register_with_novann(novann)
    lin, ql = nb.Linear(4, 3), nb.QuantLinear(16, 8)
    conv, qc = nb.Conv2d(1, 2, 3), nb.QuantConv2d(64, 8, 3)
    assert all(isinstance(x, RefLinear) for x in (lin, ql))
    assert all(isinstance(x, RefConv2d) for x in (conv, qc))
    assert isinstance(nb.ReLU(), RefReLU) and isinstance(nb.ReLU(), Activation)
    assert nb.ReLU().init_key == "relu"
    assert all(isinstance(x, RefLayer) for x in (lin, ql, conv, qc, nb.ReLU(), nb.Flatten(), nb.BatchNorm2d(3)))
    assert not isinstance(nb.ReLU(), RefLinear)


def test_reference_sequential_initialises_gpu_layers_like_its_own():
    """Same seed, same stack, NovaNN's Sequential on both sides: it must pick the same
    initialiser for a novann_b200 layer as for its own (Kaiming-normal next to ReLU) and consume
    NumPy's generator identically, so the weights are equal bit for bit; quantised layers defer
    their codes to the first forward, so nothing here touches a GPU."""
    import novann_b200 as nb
    from novann.layers import Conv2d as RefConv2d, Flatten as RefFlatten, Linear as RefLinear, ReLU as RefReLU
    nb.register_with_novann(novann)
    np.random.seed(0)
    ours = novann.Sequential(nb.Conv2d(1, 4, 3, padding=1), nb.ReLU(), RefFlatten(), nb.Linear(64, 16),
                             RefReLU(), nb.QuantLinear(16, 8), nb.ReLU(), nb.Linear(8, 4))
    np.random.seed(0)
    ref = novann.Sequential(RefConv2d(1, 4, 3, padding=1), RefReLU(), RefFlatten(), RefLinear(64, 16),
                            RefReLU(), RefLinear(16, 8), RefReLU(), RefLinear(8, 4))
    po, pr = ours.parameters(), ref.parameters()
    assert len(po) == len(pr) == 8
    for a, b in zip(po, pr):
        assert a.name == b.name and a.data.dtype == np.float32
        assert np.array_equal(a.data, b.data)
    assert float(np.std(po[2].data)) > 0.05            # Kaiming scale, not the 0.001 stand-alone default
    assert ours._layers[5]._codes is None              # QuantLinear: codes come with the first forward
    ours.eval()
    assert not ours._layers[0]._training and not ours._layers[5]._training
    ours.train()
    assert ours._layers[3]._training
    ours.zero_grad()
    assert all(p.grad is None for p in ours.parameters())


def test_init_fn_is_respected_by_the_reference_sequential():
    import novann_b200 as nb
    nb.register_with_novann(novann)
    marker = lambda shape: np.full(shape, 0.25, np.float32)  # noqa: E731
    m = novann.Sequential(nb.Linear(4, 3, init=marker), nb.ReLU(), nb.Linear(3, 2))
    assert np.all(m._layers[0].weight.data == 0.25)      # init_fn set -> the container leaves it alone
    assert not np.all(m._layers[2].weight.data == 0.25)
