"""Generates ``tests/golden/*.npz`` by running the reference (NovaNN) itself.

Run in a container that has the reference checked out:

    PYTHONDONTWRITEBYTECODE=1 NOVANN_REF=/path/to/NovaNN python tests/golden/make_golden.py

The reference is imported read-only; inputs come from ``novann_b200.workloads`` (seeded),
weights are assigned into the reference's layers so that its own RNG plays no part.  The
vectors pin the CPU oracle (``tests/test_golden.py``), which in turn checks the CUDA path.
"""
import logging
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
if "NOVANN_REF" not in os.environ:
    raise SystemExit("set NOVANN_REF to a checkout of the reference (NovaNN)")
sys.path.insert(0, os.environ["NOVANN_REF"])
logging.disable(logging.CRITICAL)

import novann  # noqa: E402  (the reference)
import novann.functional as RF  # noqa: E402
from novann.layers import Conv2d, Linear, ReLU  # noqa: E402
from novann.losses import CrossEntropyLoss  # noqa: E402
from novann.model import Sequential  # noqa: E402
from novann.module import Parameters  # noqa: E402
from novann.optim import SGD  # noqa: E402

from novann_b200 import workloads  # noqa: E402


def mlp_step(batch, dims, seed):
    x, y, params = workloads.mlp_inputs(batch, dims, seed)
    layers = []
    for i, (fi, fo) in enumerate(zip(dims[:-1], dims[1:])):
        layers.append(Linear(fi, fo))
        if i < len(dims) - 2:
            layers.append(ReLU())
    model = Sequential(*layers)
    lin = [l for l in model._layers if isinstance(l, Linear)] if hasattr(model, "_layers") else \
        [l for l in layers if isinstance(l, Linear)]
    for i, l in enumerate(lin):
        l.weight.data = params[2 * i].copy()
        l.bias.data = params[2 * i + 1].copy()
    opt = SGD(model.parameters(), lr=0.01)
    loss_fn = CrossEntropyLoss()
    opt.zero_grad()
    logits = model(x)
    loss, grad = loss_fn(logits, y)
    model.backward(grad)
    grads = [p.grad.copy() for p in model.parameters()]
    opt.step()
    new = [p.data.copy() for p in model.parameters()]
    return x, y, params, logits, np.float32(loss), grad, grads, new


def main():
    out = {}
    # ---- small MLP step: everything stored in full
    x, y, params, logits, loss, lgrad, grads, new = mlp_step(16, (32, 16, 8, 10), seed=1)
    out["mlp_small"] = dict(logits=logits, loss=loss, loss_grad=lgrad,
                            **{f"grad{i}": g for i, g in enumerate(grads)},
                            **{f"new{i}": p for i, p in enumerate(new)})
    # ---- config MLP step (batch 128, 784-256-128-10): logits + loss in full; gradients and
    # updated parameters as 4096 sampled entries each plus float64 sums (keeps the fixture small)
    x, y, params, logits, loss, lgrad, grads, new = mlp_step(128, (784, 256, 128, 10), seed=0)
    rng = np.random.default_rng(99)
    cfg = dict(logits=logits, loss=loss, loss_grad=lgrad)
    for i, (g, p) in enumerate(zip(grads, new)):
        idx = rng.integers(0, g.size, min(4096, g.size))
        cfg[f"idx{i}"] = idx.astype(np.int64)
        cfg[f"grad{i}"] = g.ravel()[idx]
        cfg[f"new{i}"] = p.ravel()[idx]
        cfg[f"gsum{i}"] = np.float64(g.astype(np.float64).sum())
        cfg[f"psum{i}"] = np.float64(p.astype(np.float64).sum())
    out["mlp_config"] = cfg
    # ---- Linear forward / backward
    rs = np.random.default_rng(5)
    lin = Linear(24, 12)
    lin.weight.data = rs.standard_normal((12, 24)).astype(np.float32)
    lin.bias.data = rs.standard_normal((1, 12)).astype(np.float32)
    xi = rs.standard_normal((7, 24)).astype(np.float32)
    yo = lin(xi)
    gi = rs.standard_normal((7, 12)).astype(np.float32)
    dx = lin.backward(gi)
    out["linear"] = dict(x=xi, w=lin.weight.data, b=lin.bias.data, y=yo, g=gi, dx=dx,
                         dw=lin.weight.grad, db=lin.bias.grad)
    # ---- ReLU and CrossEntropyLoss
    r = ReLU()
    xr = rs.standard_normal((9, 11)).astype(np.float32)
    xr[0, :3] = [0.0, -0.0, 1e-30]
    yr = r.forward(xr)
    gr = r.backward(np.ones_like(xr))
    lg = rs.standard_normal((13, 10)).astype(np.float32) * 3
    lb = rs.integers(0, 10, 13)
    ce = CrossEntropyLoss()
    closs, cgrad = ce(lg, lb)
    out["relu_ce"] = dict(x=xr, y=yr, mask_grad=gr, logits=lg, labels=lb.astype(np.int32),
                          loss=np.float32(closs), grad=cgrad)
    # ---- Conv2d forward: strides, paddings and every padding mode
    cases = [
        dict(n=2, c=3, h=9, w=8, co=4, k=(3, 3), s=(1, 1), p=(1, 1), mode="zeros"),
        dict(n=3, c=2, h=10, w=11, co=8, k=(3, 2), s=(2, 1), p=(2, 1), mode="reflect"),
        dict(n=1, c=4, h=7, w=7, co=5, k=(2, 2), s=(2, 2), p=(0, 0), mode="zeros"),
        dict(n=2, c=1, h=6, w=9, co=3, k=(3, 3), s=(1, 2), p=(2, 2), mode="replicate"),
        dict(n=2, c=2, h=5, w=6, co=2, k=(3, 3), s=(1, 1), p=(1, 2), mode="circular"),
        dict(n=4, c=16, h=14, w=14, co=32, k=(3, 3), s=(2, 2), p=(1, 1), mode="zeros"),
    ]
    conv = {}
    for i, cs in enumerate(cases):
        layer = Conv2d(cs["c"], cs["co"], cs["k"], stride=cs["s"], padding=cs["p"], padding_mode=cs["mode"])
        layer.weight.data = rs.standard_normal(layer.weight.data.shape).astype(np.float32)
        layer.bias.data = rs.standard_normal(layer.bias.data.shape).astype(np.float32)
        xc = rs.standard_normal((cs["n"], cs["c"], cs["h"], cs["w"])).astype(np.float32)
        yc = np.ascontiguousarray(layer(xc))
        conv[f"x{i}"], conv[f"w{i}"], conv[f"b{i}"], conv[f"y{i}"] = xc, layer.weight.data, layer.bias.data, yc
        gc = rs.standard_normal(yc.shape).astype(np.float32)
        dxc = np.ascontiguousarray(layer.backward(gc))
        conv[f"g{i}"], conv[f"dx{i}"], conv[f"dw{i}"], conv[f"db{i}"] = gc, dxc, layer.weight.grad, layer.bias.grad
        conv[f"geom{i}"] = np.array([*cs["k"], *cs["s"], *cs["p"],
                                     ["zeros", "reflect", "replicate", "circular"].index(cs["mode"])])
        if i == 1:
            conv["col1"] = np.ascontiguousarray(layer._cache["col"])
    conv["n_cases"] = np.array(len(cases))
    out["conv2d"] = conv
    # ---- SGD on a plain array
    p = Parameters(rs.standard_normal((5, 7)).astype(np.float32))
    p.grad = rs.standard_normal((5, 7)).astype(np.float32)
    before = p.data.copy()
    SGD([p], lr=0.01).step()
    out["sgd"] = dict(before=before, grad=p.grad, after=p.data)
    # ---- AdamW, three steps, one decayed tensor and one named "gamma" (no decay)
    from novann.optim import AdamW
    pa = Parameters(rs.standard_normal((6, 9)).astype(np.float32))
    pg = Parameters(rs.standard_normal((9,)).astype(np.float32))
    pg.name = "gamma"
    ad = dict(p0=pa.data.copy(), q0=pg.data.copy())
    opt = AdamW([pa, pg], lr=1e-3, weight_decay=1e-2)
    for t in range(3):
        pa.grad = rs.standard_normal((6, 9)).astype(np.float32)
        pg.grad = rs.standard_normal((9,)).astype(np.float32)
        ad[f"gp{t}"], ad[f"gq{t}"] = pa.grad.copy(), pg.grad.copy()
        opt.step()
        ad[f"p{t + 1}"], ad[f"q{t + 1}"] = pa.data.copy(), pg.data.copy()
    out["adamw"] = ad
    # ---- NumPy's own narrowing / widening on the edge block (the reference's cast primitive)
    e = workloads.edge_block_f32()
    with np.errstate(all="ignore"):
        h = e.astype(np.float16)
    out["astype"] = dict(f32_bits=e.view(np.uint32), f16_bits=h.view(np.uint16),
                         back_bits=h.astype(np.float32).view(np.uint32))
    for name, d in out.items():
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **d)
        print(name, os.path.getsize(os.path.join(HERE, f"{name}.npz")), "bytes")
    print("reference version:", getattr(novann, "__version__", "?"), "numpy", np.__version__)


if __name__ == "__main__":
    main()
