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
    # ---- BatchNorm2d / BatchNorm1d: training forward + backward + running statistics, then an
    # evaluation forward with the updated statistics
    from novann.layers import BatchNorm1d, BatchNorm2d, Dropout, Flatten, GlobalAvgPool2d, MaxPool2d
    bn = {}
    bn_cases = [("2d", (6, 5, 7, 4)), ("2d", (24, 8, 6, 5)), ("1d", (9, 12)), ("1d", (4, 6, 10)),
                ("2d", (1, 3, 1, 1))]
    for i, (kind, shape) in enumerate(bn_cases):
        layer = (BatchNorm2d if kind == "2d" else BatchNorm1d)(shape[1])
        layer.train()
        layer.gamma.data = rs.standard_normal(layer.gamma.data.shape) * 0.5 + 1.0
        layer.beta.data = rs.standard_normal(layer.beta.data.shape) * 0.3
        layer.running_mean = rs.standard_normal(layer.running_mean.shape) * 0.1
        layer.running_var = rs.random(layer.running_var.shape) + 0.5
        xb = (rs.standard_normal(shape) * 2.0 + 0.7).astype(np.float32)
        gb = rs.standard_normal(shape).astype(np.float32)
        bn[f"x{i}"], bn[f"g{i}"] = xb, gb
        bn[f"gamma{i}"], bn[f"beta{i}"] = layer.gamma.data.ravel().copy(), layer.beta.data.ravel().copy()
        bn[f"rm{i}"], bn[f"rv{i}"] = layer.running_mean.ravel().copy(), layer.running_var.ravel().copy()
        yb = layer.forward(xb)
        dxb = layer.backward(gb)
        bn[f"y{i}"], bn[f"dx{i}"] = yb, dxb
        bn[f"dgamma{i}"], bn[f"dbeta{i}"] = layer.gamma.grad.ravel().copy(), layer.beta.grad.ravel().copy()
        bn[f"rm_new{i}"], bn[f"rv_new{i}"] = layer.running_mean.ravel().copy(), layer.running_var.ravel().copy()
        layer.eval()
        bn[f"y_eval{i}"] = layer.forward(xb)
    bn["n_cases"] = np.array(len(bn_cases))
    out["batchnorm"] = bn
    # ---- MaxPool2d (ties, zero padding taking part in the maximum, every padding mode),
    # GlobalAvgPool2d, Dropout
    pool = {}
    pool_cases = [
        dict(shape=(2, 3, 8, 8), k=(2, 2), s=None, p=(0, 0), mode="zeros"),
        dict(shape=(2, 2, 9, 7), k=(3, 3), s=(2, 2), p=(1, 1), mode="zeros"),
        dict(shape=(1, 2, 7, 9), k=(3, 2), s=(1, 2), p=(1, 1), mode="reflect"),
        dict(shape=(2, 1, 6, 6), k=(3, 3), s=(1, 1), p=(2, 2), mode="replicate"),
        dict(shape=(1, 3, 5, 8), k=(2, 3), s=(2, 1), p=(1, 2), mode="circular"),
        dict(shape=(3, 4, 14, 14), k=(2, 2), s=(2, 2), p=(0, 0), mode="zeros"),
    ]
    for i, cs in enumerate(pool_cases):
        layer = MaxPool2d(cs["k"], cs["s"], cs["p"], cs["mode"])
        xp_ = rs.standard_normal(cs["shape"]).astype(np.float32)
        if i in (0, 1):
            xp_ = np.round(xp_ * 2) / 2          # coarse grid: many ties, many negative windows
        if i == 1:
            xp_ -= 1.0                            # mostly negative: the zero padding wins at the border
        yp = layer.forward(xp_)
        gp_ = rs.standard_normal(yp.shape).astype(np.float32)
        dxp = layer.backward(gp_)
        st = cs["s"] if cs["s"] is not None else cs["k"]
        pool[f"x{i}"], pool[f"y{i}"], pool[f"g{i}"], pool[f"dx{i}"] = xp_, yp, gp_, np.ascontiguousarray(dxp)
        pool[f"geom{i}"] = np.array([*cs["k"], *st, *cs["p"],
                                     ["zeros", "reflect", "replicate", "circular"].index(cs["mode"])])
    pool["n_cases"] = np.array(len(pool_cases))
    gap = GlobalAvgPool2d()
    xg = rs.standard_normal((5, 6, 7, 7)).astype(np.float32)
    pool["gap_x"], pool["gap_y"] = xg, gap.forward(xg)
    gg = rs.standard_normal((5, 6, 1, 1)).astype(np.float32)
    pool["gap_g"], pool["gap_dx"] = gg, gap.backward(gg)
    for i, pdrop in enumerate((0.5, 0.3)):
        dr = Dropout(pdrop)
        dr.train()
        xd = rs.standard_normal((8, 16)).astype(np.float32)
        np.random.seed(77 + i)
        yd = dr.forward(xd)
        pool[f"drop_x{i}"], pool[f"drop_y{i}"], pool[f"drop_mask{i}"] = xd, yd, dr._mask.copy()
        gd = rs.standard_normal((8, 16)).astype(np.float32)
        pool[f"drop_g{i}"], pool[f"drop_dx{i}"] = gd, dr.backward(gd)
        pool[f"drop_p{i}"] = np.float64(pdrop)
    out["pool_dropout"] = pool
    # ---- the CNN of main.py, two AdamW training steps at batch 16 on seeded inputs.  Weights are
    # assigned (the reference's own initialisers play no part); the Dropout masks the reference
    # drew are stored.
    from novann_b200 import workloads as wl
    cnn = {}
    x_all, y_all, cparams = wl.cnn_inputs(16, steps=2, seed=3)
    model = Sequential(
        Conv2d(1, 16, 3, padding=1, bias=False), BatchNorm2d(16), ReLU(),
        Conv2d(16, 32, 3, padding=1, stride=2, bias=False), BatchNorm2d(32), ReLU(),
        MaxPool2d(2, 2),
        Conv2d(32, 64, 3, padding=1, bias=False), BatchNorm2d(64), ReLU(),
        GlobalAvgPool2d(), Flatten(),
        Linear(64, 32, bias=False), BatchNorm1d(32), ReLU(), Dropout(0.5), Linear(32, 10))
    model.train()
    plist = model.parameters()
    assert len(plist) == len(cparams), (len(plist), len(cparams))
    for pr, val in zip(plist, cparams):
        assert pr.data.shape == val.shape, (pr.data.shape, val.shape)
        pr.data = val.copy()
    opt = AdamW(model.parameters(), lr=1e-3, betas=(0.9, 0.999), weight_decay=1e-2, epsilon=1e-8)
    loss_fn = CrossEntropyLoss()
    drop_layer = [l for l in model._layers if isinstance(l, Dropout)][0]
    bns = [l for l in model._layers if isinstance(l, (BatchNorm1d, BatchNorm2d))]
    for t in range(2):
        np.random.seed(500 + t)
        opt.zero_grad()
        logits = model(x_all[t])
        cnn[f"mask{t}"] = drop_layer._mask.astype(np.float32)
        loss, grad = loss_fn(logits, y_all[t])
        model.backward(grad)
        cnn[f"logits{t}"], cnn[f"loss{t}"] = logits, np.float32(loss)
        for i, pr in enumerate(model.parameters()):
            cnn[f"grad{t}_{i}"] = pr.grad.copy()
        opt.step()
        for i, pr in enumerate(model.parameters()):
            cnn[f"param{t}_{i}"] = pr.data.copy()
        for i, b_ in enumerate(bns):
            cnn[f"rm{t}_{i}"], cnn[f"rv{t}_{i}"] = b_.running_mean.ravel().copy(), b_.running_var.ravel().copy()
    model.eval()
    cnn["eval_logits"] = model(x_all[0])
    cnn["n_params"] = np.array(len(plist))
    out["cnn_main"] = cnn
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
