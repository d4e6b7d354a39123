"""Pins the CPU oracle's restatement of the reference's fp32 layers against golden vectors
produced by the reference itself (``tests/golden/make_golden.py``)."""
import os

import numpy as np
import pytest

from novann_b200 import workloads
from oracle import oracle_np as o

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return np.load(os.path.join(G, f"{name}.npz"))


def close(a, b, rel=1e-5):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.max(np.abs(a - b)) <= rel * max(1e-30, np.max(np.abs(b)))


def test_astype_edge_block_is_what_numpy_gives():
    g = load("astype")
    e = workloads.edge_block_f32()
    assert np.array_equal(e.view(np.uint32), g["f32_bits"])          # generator is stable
    assert np.array_equal(o.f32_to_f16_bits(e), g["f16_bits"])
    assert np.array_equal(o.f16_bits_to_f32(g["f16_bits"]).view(np.uint32), g["back_bits"])


def test_linear_forward_backward():
    g = load("linear")
    y = o.linear_fwd_f32(g["x"], g["w"], g["b"])
    assert close(y, g["y"], 1e-6)
    dw, db, dx = o.linear_bwd_f32(g["x"], g["w"], g["g"])
    assert close(dw, g["dw"], 1e-6) and close(db, g["db"], 1e-6) and close(dx, g["dx"], 1e-6)
    assert db.shape == (1, 12)


def test_relu_and_cross_entropy():
    g = load("relu_ce")
    y, m = o.relu_fwd(g["x"])
    assert np.array_equal(y.view(np.uint32), g["y"].view(np.uint32))
    assert np.array_equal(m, g["mask_grad"])
    loss, grad = o.softmax_ce(g["logits"], g["labels"])
    assert close(grad, g["grad"], 1e-6)
    assert abs(float(loss) - float(g["loss"])) <= 1e-6 * abs(float(g["loss"]))


def test_sgd_update_bit_exact():
    g = load("sgd")
    after = (g["before"] - np.float32(0.01) * g["grad"]).astype(np.float32)
    assert np.array_equal(after.view(np.uint32), g["after"].view(np.uint32))


def test_conv2d_forward_all_padding_modes():
    g = load("conv2d")
    modes = ["zeros", "reflect", "replicate", "circular"]
    for i in range(int(g["n_cases"])):
        kh, kw, sh, sw, ph, pw, mi = (int(v) for v in g[f"geom{i}"])
        y = o.conv2d_fwd_f32(g[f"x{i}"], g[f"w{i}"], g[f"b{i}"], (sh, sw), (ph, pw), modes[mi])
        assert y.shape == g[f"y{i}"].shape
        assert close(y, g[f"y{i}"], 1e-5), i
    kh, kw, sh, sw, ph, pw, mi = (int(v) for v in g["geom1"])
    col, _, _ = o.im2col(g["x1"], kh, kw, sh, sw, ph, pw, modes[mi])
    assert np.array_equal(col, g["col1"])                              # same (c,kh,kw) x (n,oh,ow) order


def test_conv2d_backward():
    g = load("conv2d")
    modes = ["zeros", "reflect", "replicate", "circular"]
    for i in range(int(g["n_cases"])):
        kh, kw, sh, sw, ph, pw, mi = (int(v) for v in g[f"geom{i}"])
        col, _, _ = o.im2col(g[f"x{i}"], kh, kw, sh, sw, ph, pw, modes[mi])
        dw, db, dx = o.conv2d_bwd_f32(g[f"g{i}"], col, g[f"w{i}"], g[f"x{i}"].shape, (sh, sw), (ph, pw))
        assert dx.shape == g[f"dx{i}"].shape and db.shape == g[f"db{i}"].shape
        assert close(dw, g[f"dw{i}"], 1e-5) and close(db, g[f"db{i}"], 1e-5) and close(dx, g[f"dx{i}"], 1e-5), i


def test_mlp_step_small_full_vectors():
    g = load("mlp_small")
    x, y, params = workloads.mlp_inputs(16, (32, 16, 8, 10), seed=1)
    r = o.mlp_train_step(params, x, y, 0.01)
    assert close(r["logits"], g["logits"], 1e-6)
    assert abs(float(r["loss"]) - float(g["loss"])) <= 1e-6 * abs(float(g["loss"]))
    for i in range(6):
        assert close(r["grads"][i], g[f"grad{i}"], 1e-5), i
        assert close(r["params"][i], g[f"new{i}"], 1e-6), i
        assert r["grads"][i].shape == g[f"grad{i}"].shape


def test_mlp_step_config_sampled_vectors():
    g = load("mlp_config")
    x, y, params = workloads.mlp_inputs(128, (784, 256, 128, 10), seed=0)
    r = o.mlp_train_step(params, x, y, 0.01)
    assert close(r["logits"], g["logits"], 1e-5)
    assert abs(float(r["loss"]) - float(g["loss"])) <= 1e-5 * abs(float(g["loss"]))
    assert 4.5 < float(g["loss"]) < 5.2          # ~ln(128): the double-softmax value, not textbook CE
    for i in range(6):
        idx = g[f"idx{i}"]
        assert close(r["grads"][i].ravel()[idx], g[f"grad{i}"], 1e-4), i
        assert close(r["params"][i].ravel()[idx], g[f"new{i}"], 1e-6), i
        assert abs(r["grads"][i].astype(np.float64).sum() - float(g[f"gsum{i}"])) <= 1e-4 * (1 + abs(float(g[f"gsum{i}"])))


def test_adamw_three_steps_bit_exact():
    g = load("adamw")
    p, q = g["p0"], g["q0"]
    mp = vp = np.zeros_like(p)
    mq = vq = np.zeros_like(q)
    for t in range(3):
        p, mp, vp = o.adamw_step(p, g[f"gp{t}"], mp, vp, t + 1, 1e-3, wd=1e-2)
        q, mq, vq = o.adamw_step(q, g[f"gq{t}"], mq, vq, t + 1, 1e-3, wd=1e-2, decay=False)
        assert np.array_equal(p.view(np.uint32), g[f"p{t + 1}"].view(np.uint32))
        assert np.array_equal(q.view(np.uint32), g[f"q{t + 1}"].view(np.uint32))


MODES = ["zeros", "reflect", "replicate", "circular"]


def test_batchnorm_forward_backward_running_stats_and_eval():
    g = load("batchnorm")
    for i in range(int(g["n_cases"])):
        x = g[f"x{i}"]
        y, rm, rv, cache = o.batchnorm_fwd(x, g[f"gamma{i}"], g[f"beta{i}"], g[f"rm{i}"], g[f"rv{i}"])
        assert y.dtype == np.float64 and y.shape == x.shape
        assert np.array_equal(y, g[f"y{i}"]), i                    # same NumPy expression: exact
        assert np.array_equal(rm, g[f"rm_new{i}"]) and np.array_equal(rv, g[f"rv_new{i}"])
        dx, dga, dbe = o.batchnorm_bwd(g[f"g{i}"], cache)
        assert np.array_equal(dx, g[f"dx{i}"]), i
        assert np.array_equal(dga, g[f"dgamma{i}"]) and np.array_equal(dbe, g[f"dbeta{i}"])
        ye, _, _, _ = o.batchnorm_fwd(x, g[f"gamma{i}"], g[f"beta{i}"], rm, rv, training=False)
        assert np.array_equal(ye, g[f"y_eval{i}"]), i


def test_maxpool_gap_dropout():
    g = load("pool_dropout")
    for i in range(int(g["n_cases"])):
        kh, kw, sh, sw, ph, pw, mi = (int(v) for v in g[f"geom{i}"])
        y, win, pshape = o.maxpool2d_fwd(g[f"x{i}"], (kh, kw), (sh, sw), (ph, pw), MODES[mi])
        assert np.array_equal(y, g[f"y{i}"]), i
        dx = o.maxpool2d_bwd(g[f"g{i}"], win, pshape, g[f"x{i}"].shape, (kh, kw), (sh, sw), (ph, pw))
        assert np.array_equal(dx.view(np.uint32), g[f"dx{i}"].view(np.uint32)), i
    assert np.array_equal(o.gap2d_fwd(g["gap_x"]), g["gap_y"])
    assert np.array_equal(o.gap2d_bwd(g["gap_g"], g["gap_x"].shape), g["gap_dx"])
    for i in range(2):
        p = float(g[f"drop_p{i}"])
        assert np.array_equal(o.dropout(g[f"drop_x{i}"], g[f"drop_mask{i}"], p), g[f"drop_y{i}"])
        assert np.array_equal(o.dropout(g[f"drop_g{i}"], g[f"drop_mask{i}"], p), g[f"drop_dx{i}"])


def _cnn_state(params):
    bn_c = [p.size for p in params if p.dtype == np.float64][::2]
    return dict(running=[(np.zeros(c), np.ones(c)) for c in bn_c],
                m=[np.zeros_like(p) for p in params], v=[np.zeros_like(p) for p in params])


def test_cnn_main_two_adamw_steps():
    g = load("cnn_main")
    xs, ys, params = workloads.cnn_inputs(16, steps=2, seed=3)
    assert len(params) == int(g["n_params"])
    state = _cnn_state(params)
    opt = dict(lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=1e-2)
    for t in range(2):
        r = o.cnn_train_step(o.cnn_main_spec(), params, state, xs[t], ys[t], [g[f"mask{t}"]], opt, t + 1)
        assert close(r["logits"], g[f"logits{t}"], 1e-5), t
        assert abs(float(r["loss"]) - float(g[f"loss{t}"])) <= 1e-5 * abs(float(g[f"loss{t}"]))
        for i in range(len(params)):
            assert r["grads"][i].shape == g[f"grad{t}_{i}"].shape and r["grads"][i].dtype == g[f"grad{t}_{i}"].dtype
            assert close(r["grads"][i], g[f"grad{t}_{i}"], 2e-4), (t, i)
            assert close(r["params"][i], g[f"param{t}_{i}"], 1e-5), (t, i)
        params, state = r["params"], r["state"]
        for i, (rm, rv) in enumerate(state["running"]):
            assert close(rm, g[f"rm{t}_{i}"], 1e-6) and close(rv, g[f"rv{t}_{i}"], 1e-6)
