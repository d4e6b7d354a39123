"""novann_b200 as a drop-in behind the reference's own API, on the GPU.

The reference package (NovaNN) runs here unmodified: its ``Sequential``, its loop body
(novann/utils/train/train.py:60-75), its ``CrossEntropyLoss`` and ``SGD``, its ``train()`` and
``DataLoader``.  Only the layers (and, in the functional tests, ``F.linear`` / ``F.conv2d``)
come from ``novann_b200``.  Every result is compared with the all-reference run on the same
seed.  Tolerances: fp32 GEMMs differ from NumPy's sgemm by summation order (1e-5 of the largest
magnitude, 1e-4 after three chained updates); FP8 layers use the 1e-2 weight-code bound.
"""
import numpy as np
import pytest

import _reference

novann = _reference.import_novann()
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(novann is None, reason="the reference package is not importable here")]


def _close(a, b, rel):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.max(np.abs(a - b)) <= rel * max(1e-30, np.max(np.abs(b)))


def _mlp(kind, gpu):
    """784-256-128-10 MLP built by NovaNN's Sequential; ``kind``: 'ref', 'gpu' (fp32 layers on the
    GPU mixed with the reference's ReLU) or 'quant' (middle layer FP8)."""
    import novann_b200 as nb
    from novann.layers import Linear as RefLinear, ReLU as RefReLU
    nb.register_with_novann(novann)
    np.random.seed(0)
    if kind == "ref":
        return novann.Sequential(RefLinear(784, 256), RefReLU(), RefLinear(256, 128), RefReLU(), RefLinear(128, 10))
    mid = nb.QuantLinear(256, 128, device=gpu) if kind == "quant" else nb.Linear(256, 128, device=gpu)
    return novann.Sequential(nb.Linear(784, 256, device=gpu), RefReLU(), mid, nb.ReLU(device=gpu),
                             nb.Linear(128, 10, device=gpu))


def _loop(model, x, y, steps):
    """The reference's loop body, with the reference's loss and optimiser."""
    from novann.losses import CrossEntropyLoss
    from novann.optim import SGD
    loss_fn, opt = CrossEntropyLoss(), SGD(model.parameters(), lr=0.01)
    out = []
    model.train()
    for s in range(steps):
        opt.zero_grad()
        logits = model(x[s])
        cost, grad = loss_fn(logits, y[s])
        model.backward(grad)
        grads = [p.grad.copy() for p in model.parameters()]
        opt.step()
        out.append((np.array(logits), float(cost), grads))
    return out, [p.data.copy() for p in model.parameters()]


def test_reference_loop_on_gpu_layers_matches_all_reference_run(gpu):
    rng = np.random.default_rng(0)
    x = rng.random((3, 128, 784), dtype=np.float32)
    y = rng.integers(0, 10, (3, 128))
    ref_steps, ref_params = _loop(_mlp("ref", gpu), x, y, 3)
    got_steps, got_params = _loop(_mlp("gpu", gpu), x, y, 3)
    for (lg, cost, grads), (rlg, rcost, rgrads) in zip(got_steps, ref_steps):
        assert lg.dtype == np.float32 and _close(lg, rlg, 1e-4)
        assert abs(cost - rcost) <= 1e-4 * abs(rcost)
        assert all(_close(a, b, 2e-4) for a, b in zip(grads, rgrads))
    assert all(_close(a, b, 1e-5) for a, b in zip(got_params, ref_params))


def test_reference_loop_with_a_quantised_layer(gpu):
    """QuantLinear in the middle of NovaNN's Sequential, trained by NovaNN's SGD: the codes are
    refreshed from the weight the optimiser updated in place, and the run stays within the FP8
    bound of the all-reference run."""
    rng = np.random.default_rng(1)
    x = rng.random((3, 128, 784), dtype=np.float32)
    y = rng.integers(0, 10, (3, 128))
    ref_steps, ref_params = _loop(_mlp("ref", gpu), x, y, 3)
    model = _mlp("quant", gpu)
    got_steps, got_params = _loop(model, x, y, 3)
    for (lg, _, _), (rlg, _, _) in zip(got_steps, ref_steps):
        assert _close(lg, rlg, 4e-2)
    # weights stay within the FP8 bound of the reference's; the three updates themselves (three
    # bits of weight mantissa in the forward pass show up as a few per cent in the gradients)
    # within 0.25 of the largest update of each tensor
    init = [p.data.copy() for p in _mlp("ref", gpu).parameters()]
    for a, b, p0 in zip(got_params, ref_params, init):
        if a.shape[0] != 1:
            assert _close(a, b, 1e-2)
        assert _close(a - p0, b - p0, 0.25)
    # the codes in use are those of the current weight
    from novann_b200 import quant
    q = model._layers[2]
    model.eval()
    codes_before = q._codes.copy()
    model(x[0])
    assert np.array_equal(q._codes, codes_before)          # evaluation mode reuses the codes
    want, _ = quant.quantize_weight(q.weight.data, "e4m3", gpu)
    model.train()
    model(x[0])
    assert np.array_equal(q._codes, want)


def test_reference_train_function_and_accuracy(gpu):
    """novann.utils.train.train + DataLoader + metrics.accuracy over a model of GPU layers."""
    from novann.losses import CrossEntropyLoss
    from novann.metrics import accuracy
    from novann.optim import SGD
    from novann.utils.data import DataLoader
    from novann.utils.train import train
    rng = np.random.default_rng(2)
    centers = rng.standard_normal((10, 784)).astype(np.float32)
    yl = rng.integers(0, 10, 512)
    xl = (centers[yl] + 0.3 * rng.standard_normal((512, 784))).astype(np.float32)
    model = _mlp("gpu", gpu)
    loader = DataLoader(xl, yl, batch_size=128, shuffle=False)
    before = accuracy(model, loader)
    opt = SGD(model.parameters(), lr=0.05)
    train(loader, loader, model, opt, CrossEntropyLoss(), epochs=3, metric=accuracy, verbose=False)
    after = accuracy(model, loader)
    assert after > max(0.9, before)


@pytest.mark.parametrize("bias", [True, False])
def test_functional_linear_has_the_reference_signature(gpu, bias):
    import novann.functional as RF
    from novann.module import Parameters
    from novann_b200 import functional as F
    rng = np.random.default_rng(3)
    x = rng.standard_normal((37, 50)).astype(np.float32)
    w = Parameters(rng.standard_normal((21, 50)).astype(np.float32))
    b = Parameters(rng.standard_normal((1, 21)).astype(np.float32)) if bias else None
    want = RF.linear(x, w, b)
    got = F.linear(x, w, b, device=gpu)
    assert got.dtype == np.float32 and got.shape == want.shape and _close(got, want, 1e-5)
    assert _close(F.linear(x.astype(np.float64), w, bias=b, device=gpu), want, 1e-5)   # float64 in: GPU cast


@pytest.mark.parametrize("mode", ["zeros", "reflect", "replicate", "circular"])
@pytest.mark.parametrize("stride,padding", [(1, 1), (2, 1), ((2, 1), (0, 2))])
def test_functional_conv2d_has_the_reference_signature(gpu, mode, stride, padding):
    import novann.functional as RF
    from novann.module import Parameters
    from novann_b200 import functional as F
    rng = np.random.default_rng(4)
    x = rng.standard_normal((3, 5, 9, 8)).astype(np.float32)
    w = Parameters(rng.standard_normal((6, 5, 3, 3)).astype(np.float32))
    b = Parameters(rng.standard_normal((6, 1)).astype(np.float32))
    want, col, w_col = RF.conv2d(x, w, 3, stride, padding, bias=b, padding_mode=mode, extras=True)
    got, gcol, gw_col = F.conv2d(x, w, 3, stride, padding, bias=b, padding_mode=mode, extras=True, device=gpu)
    assert got.shape == want.shape and _close(got, want, 1e-5)
    assert np.array_equal(gcol, col) and np.array_equal(gw_col, w_col)       # im2col is a gather: bit-identical
    plain = F.conv2d(x, w, (3, 3), stride, padding, bias=b, padding_mode=mode, device=gpu)
    assert np.array_equal(plain, got)
    with pytest.raises(ValueError):
        F.conv2d(x, w, 3, padding="same", device=gpu)
    with pytest.raises(ValueError):
        F.conv2d(x, w, 3, padding_mode="mirror", device=gpu)


def test_float64_from_a_reference_batchnorm_is_narrowed_on_the_gpu(gpu):
    """A reference BatchNorm1d emits float64 (its gamma / beta are float64,
    novann/layers/batchnorm/batchnorm1d.py); the layer after it narrows with
    astype(np.float32).  With a novann_b200 Linear after it that narrowing is nvq_cast on the GPU
    and the result equals the reference Linear's on the same weights."""
    import novann_b200 as nb
    from novann.layers import BatchNorm1d as RefBN, Linear as RefLinear
    rng = np.random.default_rng(5)
    x = rng.standard_normal((64, 40)).astype(np.float32)
    bn = RefBN(40)
    h = bn(x)
    assert h.dtype == np.float64
    ours, ref = nb.Linear(40, 12, device=gpu, init=nb.layers.kaiming_normal), RefLinear(40, 12)
    ref.weight.data[...] = ours.weight.data
    got, want = ours(h), ref(h)
    assert got.dtype == np.float32 and _close(got, want, 1e-5)
    assert np.array_equal(ours._cache_input.view(np.uint32), h.astype(np.float32).view(np.uint32))
    g = rng.standard_normal((64, 12))                      # a float64 gradient narrows the same way
    dx, rdx = ours.backward(g), ref.backward(g)
    assert _close(dx, rdx, 1e-5) and _close(ours.weight.grad, ref.weight.grad, 1e-5)
