"""Central-difference gradient checks of the GPU layers, in the style of the reference's own
tests (tests/layers/linear/test_linear.py:31-64 and tests/layers/conv/test_conv2d.py:46-84 use
``numeric_grad_wrt_param`` with a max-abs threshold of 5e-3): perturb sampled entries of a
parameter or of the input, re-run the layer's forward, compare with ``backward``."""
import numpy as np
import pytest

import novann_b200 as nb

pytestmark = pytest.mark.gpu
THRESHOLD = 5e-3          # the reference's bound
EPS = 1e-2                # larger than the reference's 1e-5: the forward here is fp32 end to end


def _numeric(layer, x, proj, array, picks):
    out = []
    for idx in picks:
        old = array[idx]
        array[idx] = old + EPS
        hi = float(np.sum(layer.forward(x).astype(np.float64) * proj))
        array[idx] = old - EPS
        lo = float(np.sum(layer.forward(x).astype(np.float64) * proj))
        array[idx] = old
        out.append((hi - lo) / (2 * EPS))
    return np.array(out)


def _picks(shape, k, rng):
    return [tuple(rng.integers(0, s) for s in shape) for _ in range(k)]


def test_linear_gradients(gpu):
    rng = np.random.default_rng(0)
    layer = nb.Linear(20, 12, device=gpu, init=nb.layers.kaiming_normal)
    x = rng.standard_normal((6, 20)).astype(np.float32)
    proj = rng.standard_normal((6, 12))
    layer.forward(x)
    dx = layer.backward(proj.astype(np.float32))
    for arr, grad in ((layer.weight.data, layer.weight.grad), (layer.bias.data, layer.bias.grad), (x, dx)):
        picks = _picks(arr.shape, 8, rng)
        num = _numeric(layer, x, proj, arr, picks)
        ana = np.array([grad[i] for i in picks])
        assert np.max(np.abs(num - ana)) < THRESHOLD


@pytest.mark.parametrize("stride,padding,mode", [(1, 1, "zeros"), (2, 1, "zeros"), ((2, 1), (0, 2), "zeros")])
def test_conv2d_gradients(gpu, stride, padding, mode):
    rng = np.random.default_rng(1)
    layer = nb.Conv2d(3, 4, 3, stride=stride, padding=padding, padding_mode=mode, device=gpu)
    layer.weight.data = (rng.standard_normal(layer.weight.data.shape) * 0.5).astype(np.float32)
    x = rng.standard_normal((2, 3, 7, 6)).astype(np.float32)
    out = layer.forward(x)
    proj = rng.standard_normal(out.shape)
    dx = layer.backward(proj.astype(np.float32))
    for arr, grad in ((layer.weight.data, layer.weight.grad), (layer.bias.data, layer.bias.grad), (x, dx)):
        picks = _picks(arr.shape, 8, rng)
        num = _numeric(layer, x, proj, arr, picks)
        ana = np.array([grad[i] for i in picks])
        assert np.max(np.abs(num - ana)) < THRESHOLD


def test_relu_mask_and_sequential_shapes(gpu):
    """tests/layers/activations/test_relu.py:23-26 and tests/sequential/test_sequential.py:112-145:
    the mask equals (x > 0); a stack keeps shapes and fills every gradient."""
    rng = np.random.default_rng(2)
    x = rng.standard_normal((5, 9)).astype(np.float32)
    r = nb.ReLU(device=gpu)
    y = r.forward(x)
    assert np.array_equal(r._mask, (x > 0).astype(np.float32)) and np.array_equal(y, x * (x > 0))
    init = nb.layers.kaiming_normal
    model = nb.Sequential(nb.Linear(9, 7, device=gpu, init=init), nb.ReLU(device=gpu),
                          nb.Linear(7, 3, device=gpu, init=init))
    out = model(x)
    assert out.shape == (5, 3) and out.dtype == np.float32
    model.backward(np.ones_like(out))
    assert all(p.grad is not None and p.grad.shape == p.data.shape for p in model.parameters())
    model.zero_grad()
    assert all(p.grad is None for p in model.parameters())
