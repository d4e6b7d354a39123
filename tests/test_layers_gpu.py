"""The fp32 layers, Conv2d forward, quantised layers and the device-resident MLP step on the
GPU against the reference's golden vectors and the CPU oracle.

Tolerances: fp32 GEMM results differ from NumPy's sgemm by summation order only -> 1e-5 of
the largest magnitude (1e-4 for gradients that sum 128 products of small numbers);
elementwise steps (ReLU, SGD) are bit-exact; quantised layers use the 1e-2 / 5e-2 bounds.
"""
import os

import numpy as np
import pytest

import novann_b200 as nb
from novann_b200 import functional as F, quant, workloads
from novann_b200.train import MLPTrainStep
from oracle import oracle_np as o

from novann_b200.layers import kaiming_normal  # noqa: E402

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return np.load(os.path.join(G, f"{name}.npz"))


def close(a, b, rel=1e-5):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.max(np.abs(a - b)) <= rel * max(1e-30, np.max(np.abs(b)))


def test_linear_layer_matches_reference_vectors(gpu):
    g = load("linear")
    lin = nb.Linear(24, 12, device=gpu)
    lin.weight.data, lin.bias.data = g["w"].copy(), g["b"].copy()
    y = lin(g["x"])
    assert y.shape == (7, 12) and y.dtype == np.float32          # the reference's own assertions
    assert close(y, g["y"], 1e-6)
    dx = lin.backward(g["g"])
    assert dx.shape == (7, 24) and lin.weight.grad.shape == (12, 24) and lin.bias.grad.shape == (1, 12)
    assert close(dx, g["dx"], 1e-6) and close(lin.weight.grad, g["dw"], 1e-6)
    assert close(lin.bias.grad, g["db"], 1e-6)
    assert [p.name for p in lin.parameters()] == ["linear weight", "linear bias"]


def test_linear_accepts_float64_input_like_astype(gpu):
    lin = nb.Linear(8, 4, device=gpu)
    x = np.random.default_rng(0).standard_normal((3, 8))          # float64, as BatchNorm would emit
    y = lin(x)
    assert y.dtype == np.float32
    assert close(y, o.linear_fwd_f32(x.astype(np.float32), lin.weight.data, lin.bias.data), 1e-6)


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (33, 65, 97), (128, 256, 784), (128, 10, 128), (300, 7, 40)])
def test_linear_f32_shapes_against_float64(gpu, m, n, k):
    rng = np.random.default_rng(m * n)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((n, k)).astype(np.float32)
    b = rng.standard_normal((1, n)).astype(np.float32)
    ref = x.astype(np.float64) @ w.T.astype(np.float64) + b
    assert close(F.linear_f32_host(x, w, b, gpu), ref, 2e-6)
    gr = rng.standard_normal((m, n)).astype(np.float32)
    mask = (rng.random((m, k)) > 0.5).astype(np.float32)
    dw, db, dx = F.linear_bwd_f32_host(gr, x, w, True, gpu, mask=mask)
    assert close(dw, gr.T.astype(np.float64) @ x, 2e-6)
    assert close(db, gr.astype(np.float64).sum(0, keepdims=True), 2e-6)
    assert close(dx, (gr.astype(np.float64) @ w) * mask, 2e-6)


def test_relu_bit_exact_including_negative_zero(gpu):
    g = load("relu_ce")
    r = nb.ReLU(device=gpu)
    y = r.forward(g["x"])
    assert np.array_equal(y.view(np.uint32), g["y"].view(np.uint32))
    assert np.array_equal(r.backward(np.ones_like(g["x"])), g["mask_grad"])


def test_cross_entropy_loss_and_grad(gpu):
    g = load("relu_ce")
    loss, grad = nb.CrossEntropyLoss(device=gpu)(g["logits"], g["labels"])
    assert grad.dtype == np.float32 and close(grad, g["grad"], 1e-6)
    assert abs(float(loss) - float(g["loss"])) <= 1e-5 * abs(float(g["loss"]))


def test_sgd_step_bit_exact_and_in_place(gpu):
    g = load("sgd")
    p = nb.Parameters(g["before"].copy())
    p.grad = g["grad"].copy()
    held = p.data
    opt = nb.SGD([p], lr=0.01, device=gpu)
    opt.step()
    assert held is p.data                                          # updated in place, as the reference does
    assert np.array_equal(p.data.view(np.uint32), g["after"].view(np.uint32))
    opt.zero_grad()
    assert not p.grad.any()


def test_conv2d_forward_reference_vectors(gpu):
    g = load("conv2d")
    modes = ["zeros", "reflect", "replicate", "circular"]
    for i in range(int(g["n_cases"])):
        kh, kw, sh, sw, ph, pw, mi = (int(v) for v in g[f"geom{i}"])
        w = g[f"w{i}"]
        layer = nb.Conv2d(w.shape[1], w.shape[0], (kh, kw), stride=(sh, sw), padding=(ph, pw),
                          padding_mode=modes[mi], device=gpu)
        layer.weight.data, layer.bias.data = w.copy(), g[f"b{i}"].copy()
        y = layer(g[f"x{i}"])
        assert y.shape == g[f"y{i}"].shape and y.dtype == np.float32
        assert close(y, g[f"y{i}"], 1e-5), i
        if i == 1:
            assert np.array_equal(layer._cache["col"], g["col1"])   # same im2col ordering, bit for bit


def test_conv2d_backward_reference_vectors(gpu):
    g = load("conv2d")
    modes = ["zeros", "reflect", "replicate", "circular"]
    for i in range(int(g["n_cases"])):
        kh, kw, sh, sw, ph, pw, mi = (int(v) for v in g[f"geom{i}"])
        w = g[f"w{i}"]
        layer = nb.Conv2d(w.shape[1], w.shape[0], (kh, kw), stride=(sh, sw), padding=(ph, pw),
                          padding_mode=modes[mi], device=gpu)
        layer.weight.data, layer.bias.data = w.copy(), g[f"b{i}"].copy()
        layer(g[f"x{i}"])
        dx = layer.backward(g[f"g{i}"])
        assert dx.shape == g[f"x{i}"].shape and dx.dtype == np.float32
        assert layer.weight.grad.shape == w.shape and layer.bias.grad.shape == (w.shape[0], 1)
        assert close(dx, g[f"dx{i}"], 1e-5), i
        assert close(layer.weight.grad, g[f"dw{i}"], 1e-5), i
        assert close(layer.bias.grad, g[f"db{i}"], 1e-5), i


def test_quant_conv2d_backward_uses_master_weight(gpu):
    g = load("conv2d")
    kh, kw, sh, sw, ph, pw, mi = (int(v) for v in g["geom5"])
    w = g["w5"]
    layer = nb.QuantConv2d(w.shape[1], w.shape[0], (kh, kw), stride=(sh, sw), padding=(ph, pw), device=gpu)
    layer.weight.data, layer.bias.data = w.copy(), g["b5"].copy()
    layer.requantize()
    layer(g["x5"])
    dx = layer.backward(g["g5"])
    assert close(dx, g["dx5"], 1e-5) and close(layer.weight.grad, g["dw5"], 1e-5)


def test_conv2d_rejects_bad_padding(gpu):
    with pytest.raises(ValueError):
        nb.Conv2d(1, 1, 3, padding="same")
    layer = nb.Conv2d(1, 1, 3, padding_mode="mirror", device=gpu)
    with pytest.raises(ValueError):
        layer(np.zeros((1, 1, 5, 5), np.float32))


def test_weight_quantisation_per_channel_bit_exact(gpu):
    _, w, _ = workloads.linear_inputs(8, 96, 200, seed=4)
    w[3] = 0
    for fmt in ("e4m3", "e5m2"):
        codes, scales = quant.quantize_weight(w, fmt, gpu)
        wc, ws = o.quantize_weight_per_channel(w, fmt)
        assert np.array_equal(codes, wc)
        assert np.array_equal(scales.view(np.uint32), ws.view(np.uint32))


@pytest.mark.parametrize("fmt,tol", [("e4m3", 1e-2), ("e5m2", 1e-2), ("e2m1_b32", 5e-2)])
def test_quant_linear_layer(gpu, fmt, tol):
    rng = np.random.default_rng(3)
    layer = nb.QuantLinear(256, 192, fmt=fmt, device=gpu, init=kaiming_normal)
    layer.bias.data = rng.standard_normal((1, 192)).astype(np.float32) * 0.01
    x = rng.standard_normal((160, 256)).astype(np.float32)
    y = layer(x)
    assert y.shape == (160, 192) and y.dtype == np.float32
    xb = o.f32_to_bf16_bits(x).reshape(x.shape)
    if fmt == "e2m1_b32":
        wd = o.dequantize_fp4_weight(*o.quantize_fp4_b32(o.f32_to_bf16_bits(layer.weight.data).reshape(192, 256)))
        ref = o.bf16_bits_to_f32(xb).astype(np.float64) @ wd.T.astype(np.float64) + layer.bias.data
    else:
        wq, sc = o.quantize_weight_per_channel(layer.weight.data, fmt)
        ref = o.bf16_bits_to_f32(o.linear_fwd_qweight(xb, wq, sc, layer.bias.data.reshape(-1), fmt)[0])
    assert o.max_abs_rel(y, ref) <= 2.0 ** -6
    # against the unquantised fp32 layer only the quantisation error of the weight remains
    # (3, 2 and 1 mantissa bits): a sanity bound on the codes, not a kernel tolerance
    full = o.linear_fwd_f32(x, layer.weight.data, layer.bias.data)
    assert o.max_abs_rel(y, full) <= {"e4m3": 0.04, "e5m2": 0.08, "e2m1_b32": 0.5}[fmt]
    dx = layer.backward(np.ones((160, 192), np.float32))
    assert dx.shape == (160, 256) and layer.weight.grad.shape == (192, 256)


@pytest.mark.parametrize("m,n,k", [(8, 8, 8), (160, 192, 256), (264, 520, 136), (1024, 512, 2048)])
def test_quant_linear_backward_on_tensor_cores(gpu, m, n, k):
    """dX, dW, db of the quantised Linear as bf16 tensor-core contractions.  Oracle: the same
    bf16-rounded operands contracted in float64; bound 1e-2 (max-abs-rel) as for the forward.
    db is an fp32 sum in row order and matches NumPy's column sum to rounding."""
    rng = np.random.default_rng(m + n)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    g = (rng.standard_normal((m, n)) / m).astype(np.float32)
    wq, sc = o.quantize_weight_per_channel(w, "e4m3")
    dw, db, dx = F.linear_q_bwd_host(g, x, wq, sc, "e4m3", True, gpu)
    r = lambda a: o.bf16_bits_to_f32(o.f32_to_bf16_bits(a)).reshape(a.shape).astype(np.float64)
    wd = r(o.E4M3_TABLE[wq] * sc[:, None])
    assert dx.shape == (m, k) and dw.shape == (n, k) and db.shape == (1, n) and dx.dtype == np.float32
    assert o.max_abs_rel(dx, r(g) @ wd) <= 2.0 ** -10
    assert o.max_abs_rel(dw, r(g).T @ r(x)) <= 2.0 ** -10
    assert close(db, g.astype(np.float64).sum(0, keepdims=True), 1e-5)
    # and against the reference's fp32 rules on the dequantised weight: inside the FP8 bound
    rdw, rdb, rdx = o.linear_bwd_f32(x, (o.E4M3_TABLE[wq] * sc[:, None]).astype(np.float32), g)
    assert o.max_abs_rel(dx, rdx) <= 1e-2 and o.max_abs_rel(dw, rdw) <= 1e-2


def test_quant_linear_layer_tensor_core_backward(gpu):
    rng = np.random.default_rng(1)
    layer = nb.QuantLinear(128, 64, fmt="e4m3", device=gpu, tensor_core_backward=True, init=kaiming_normal)
    x = rng.standard_normal((96, 128)).astype(np.float32)
    layer(x)
    g = rng.standard_normal((96, 64)).astype(np.float32)
    dx = layer.backward(g)
    ref_dw, ref_db, ref_dx = o.linear_bwd_f32(x, layer.weight.data, g)
    assert o.max_abs_rel(dx, ref_dx) <= 4e-2          # FP8 weight error shows in dX
    assert o.max_abs_rel(layer.weight.grad, ref_dw) <= 1e-2
    assert close(layer.bias.grad, ref_db, 1e-5)


@pytest.mark.parametrize("case", [0, 1, 3, 4, 5])
def test_quant_conv2d_layer(gpu, case):
    g = load("conv2d")
    modes = ["zeros", "reflect", "replicate", "circular"]
    kh, kw, sh, sw, ph, pw, mi = (int(v) for v in g[f"geom{case}"])
    w, x = g[f"w{case}"], g[f"x{case}"]
    cout = (w.shape[0] + 7) // 8 * 8                                # tensor-core path wants Cout % 8 == 0
    rng = np.random.default_rng(case)
    w8 = rng.standard_normal((cout, *w.shape[1:])).astype(np.float32)
    w8[:w.shape[0]] = w
    layer = nb.QuantConv2d(w.shape[1], cout, (kh, kw), stride=(sh, sw), padding=(ph, pw),
                           padding_mode=modes[mi], fmt="e4m3", device=gpu)
    layer.weight.data = w8
    layer.bias.data = rng.standard_normal((cout, 1)).astype(np.float32)
    layer.requantize()
    y = layer(x)
    # oracle: same codes, bf16-rounded patches, float64 contraction, bf16-rounded result
    wq, sc = o.quantize_weight_per_channel(w8.reshape(cout, -1), "e4m3")
    wd = (o.E4M3_TABLE[wq] * sc[:, None]).reshape(w8.shape)
    xr = o.bf16_bits_to_f32(o.f32_to_bf16_bits(x)).reshape(x.shape)
    ref = o.conv2d_fwd_f32(xr.astype(np.float64), wd.astype(np.float64), None, (sh, sw), (ph, pw), modes[mi])
    col, oh, ow = o.im2col(xr, kh, kw, sh, sw, ph, pw, modes[mi])
    ref = (wd.reshape(cout, -1).astype(np.float64) @ col.astype(np.float64)) + layer.bias.data
    ref = ref.reshape(cout, x.shape[0], oh, ow).transpose(1, 0, 2, 3)
    assert y.shape == ref.shape
    assert o.max_abs_rel(y, ref) <= 2.0 ** -6
    # the first Cout channels approximate the reference's fp32 convolution within the FP8 bound
    assert o.max_abs_rel(y[:, :w.shape[0]] - layer.bias.data[:w.shape[0]].reshape(1, -1, 1, 1),
                         g[f"y{case}"] - g[f"b{case}"].reshape(1, -1, 1, 1)) <= 6e-2


def _check_step(step_out, g, sampled):
    logits, loss, grads, params = step_out
    assert close(logits, g["logits"], 1e-5)
    assert abs(float(loss) - float(g["loss"])) <= 1e-4 * abs(float(g["loss"]))
    for i in range(6):
        if sampled:
            idx = g[f"idx{i}"]
            assert close(grads[i].ravel()[idx], g[f"grad{i}"], 1e-4), i
            assert close(params[i].ravel()[idx], g[f"new{i}"], 1e-6), i
        else:
            assert grads[i].shape == g[f"grad{i}"].shape
            assert close(grads[i], g[f"grad{i}"], 1e-4), i
            assert close(params[i], g[f"new{i}"], 1e-6), i


def test_mlp_train_step_device_resident_small(gpu):
    x, y, params = workloads.mlp_inputs(16, (32, 16, 8, 10), seed=1)
    st = MLPTrainStep(params, 16, 0.01, gpu)
    st.step(x, y)
    _check_step((st.logits(), st.loss(), st.grads(), st.params()), load("mlp_small"), sampled=False)


def test_mlp_train_step_config_and_three_more_steps(gpu):
    """batch 128, 784-256-128-10, SGD 0.01: the first step against the reference's vectors,
    then three further steps against the oracle run in lock step."""
    dims = (784, 256, 128, 10)
    x, y, params = workloads.mlp_inputs(128, dims, seed=0)
    st = MLPTrainStep(params, 128, 0.01, gpu)
    st.step(x, y)
    _check_step((st.logits(), st.loss(), st.grads(), st.params()), load("mlp_config"), sampled=True)
    cur = o.mlp_train_step(params, x, y, 0.01)["params"]
    for s in range(1, 4):
        xs, ys, _ = workloads.mlp_inputs(128, dims, seed=10 + s)
        r = o.mlp_train_step(cur, xs, ys, 0.01)
        st.step(xs, ys)
        assert close(st.logits(), r["logits"], 1e-4)
        for a, b in zip(st.params(), r["params"]):
            assert close(a, b, 1e-5)
        cur = r["params"]


def test_mlp_train_step_graph_replay_equals_eager(gpu):
    dims = (784, 256, 128, 10)
    x, y, params = workloads.mlp_inputs(128, dims, seed=0)
    eager, graph = MLPTrainStep(params, 128, 0.01, gpu), MLPTrainStep(params, 128, 0.01, gpu)
    graph.step(x, y)                   # first step eagerly (first-call set-up), then capture
    eager.step(x, y)
    graph.capture()
    for s in range(3):
        xs, ys, _ = workloads.mlp_inputs(128, dims, seed=30 + s)
        eager.step(xs, ys)
        graph.step(xs, ys)
    for a, b in zip(eager.params(), graph.params()):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert eager.loss() == graph.loss()
    assert graph.kernels_per_step() == 10


def test_sequential_of_gpu_layers_runs_the_reference_loop(gpu):
    """zero_grad -> forward -> loss -> backward -> step through the Layer API, as in the
    reference's train loop, compared with its vectors."""
    dims = (32, 16, 8, 10)
    x, y, params = workloads.mlp_inputs(16, dims, seed=1)
    layers = []
    for i, (fi, fo) in enumerate(zip(dims[:-1], dims[1:])):
        lin = nb.Linear(fi, fo, device=gpu)
        lin.weight.data, lin.bias.data = params[2 * i].copy(), params[2 * i + 1].copy()
        layers.append(lin)
        if i < len(dims) - 2:
            layers.append(nb.ReLU(device=gpu))
    model = nb.Sequential(*layers)
    opt = nb.SGD(model.parameters(), lr=0.01, device=gpu)
    opt.zero_grad()
    logits = model(x)
    loss, grad = nb.CrossEntropyLoss(device=gpu)(logits, y)
    model.backward(grad)
    grads = [p.grad.copy() for p in model.parameters()]
    opt.step()
    _check_step((logits, loss, grads, [p.data for p in model.parameters()]), load("mlp_small"), sampled=False)
    assert len(model.parameters()) == 6


def test_adamw_bit_exact_against_reference_vectors(gpu):
    g = load("adamw")
    p, q = nb.Parameters(g["p0"].copy()), nb.Parameters(g["q0"].copy())
    q.name = "gamma"
    opt = nb.AdamW([p, q], lr=1e-3, weight_decay=1e-2, device=gpu)
    for t in range(3):
        p.grad, q.grad = g[f"gp{t}"].copy(), g[f"gq{t}"].copy()
        opt.step()
        assert np.array_equal(p.data.view(np.uint32), g[f"p{t + 1}"].view(np.uint32)), t
        assert np.array_equal(q.data.view(np.uint32), g[f"q{t + 1}"].view(np.uint32)), t


def test_quant_mlp_inference_fused_relu(gpu):
    """Device-resident FP8-weight MLP forward with bias + ReLU fused into the GEMM epilogue,
    against the oracle chain (bf16 activations between layers, same codes)."""
    from novann_b200.train import QuantMLPInference
    dims = (512, 384, 256, 16)
    x, _, params = workloads.mlp_inputs(300, dims, seed=3)
    for i in range(len(dims) - 1):
        params[2 * i + 1] = (np.random.default_rng(i).standard_normal((1, dims[i + 1])) * 0.1).astype(np.float32)
    net = QuantMLPInference(params, max_batch=512, device=gpu)
    y = net.forward(x)
    h = o.f32_to_bf16_bits(x).reshape(x.shape)
    for i in range(len(dims) - 1):
        wq, sc = o.quantize_weight_per_channel(params[2 * i], "e4m3")
        _, pre = o.linear_fwd_qweight(h, wq, sc, params[2 * i + 1].ravel(), "e4m3")
        if i < len(dims) - 2:
            pre = pre * (pre > 0)
        h = o.f32_to_bf16_bits(pre).reshape(pre.shape)
    want = o.bf16_bits_to_f32(h)
    assert y.shape == (300, 16)
    assert o.max_abs_rel(y, want) <= 1e-2
    assert np.mean(y == want) > 0.9          # most outputs agree to the last bf16 bit


@pytest.mark.parametrize("case", [
    # n, c, h, w, cout, k, p: stride 1, channels in blocks of 64 -> the implicit-GEMM kernel
    (2, 64, 8, 8, 64, 3, 1),          # one box per image, boxes of 8 x 8
    (3, 64, 14, 14, 72, 3, 1),        # two boxes of 7 rows per image; odd image count: last CTA tile empty
    (2, 128, 12, 10, 264, 3, 1),      # Cout over one 256-column tile; two channel blocks per tap
    (1, 64, 30, 30, 16, 5, 2),        # 5 x 5 taps, boxes of 4 rows, last box of an image partly outside
    (5, 64, 9, 9, 40, 1, 0),          # 1 x 1 convolution, no padding
    (2, 64, 6, 20, 24, 3, 0),         # no padding: output 4 x 18
    (4, 192, 7, 7, 128, 3, 1),        # three channel blocks
    (372, 64, 14, 14, 128, 3, 1),     # five tiles per CTA pair: all four accumulator buffers reused
    (3, 128, 10, 10, 96, 3, 1),       # at most 128 channels out, an even number of k-blocks
    (2, 64, 6, 200, 16, 3, 1),        # output rows of 200 positions: one row per tile (swapped kernel only)
])
def test_implicit_gemm_conv_equals_patch_matrix_conv_and_oracle(gpu, case):
    """The tcgen05 implicit-GEMM convolution (4-D TMA boxes, no patch matrix) against the
    patch-matrix path of the same entry point (bit-identical inputs to the MMAs, so only the fp32
    accumulation order differs) and against the oracle within the FP8 bound."""
    n, c, h, w, cout, k, p = case
    rng = np.random.default_rng(n * 1000 + c + h)
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (rng.standard_normal((cout, c, k, k)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    w_col = wt.reshape(cout, -1)
    assert w_col.shape[1] % 16 == 0
    codes, scales = quant.quantize_weight(w_col, "e4m3", gpu)
    y_imp = F.conv2d_q_host(x, codes, scales, b, (k, k), (1, 1), (p, p), "zeros", "e4m3", gpu)
    y_exp = F.conv2d_q_host(x, codes, scales, b, (k, k), (1, 1), (p, p), "zeros", "e4m3", gpu,
                            path="patch_matrix")
    assert y_imp.shape == y_exp.shape == (n, cout, h + 2 * p - k + 1, w + 2 * p - k + 1)
    # both are bf16-rounded: equal up to one bf16 ulp where the fp32 sums differ in their last bits
    assert o.max_abs_rel(y_imp, y_exp) <= 2.0 ** -8
    assert np.mean(y_imp == y_exp) > 0.9
    # both implicit kernels, whichever the dispatch picks: the CTA-pair kernel and (for at most
    # 128 output channels) the operand-swapped kernel
    for forced in ("cta_pair", "auto"):
        y_f = F.conv2d_q_host(x, codes, scales, b, (k, k), (1, 1), (p, p), "zeros", "e4m3", gpu, path=forced)
        assert o.max_abs_rel(y_f, y_exp) <= 2.0 ** -8, forced
        assert np.mean(y_f == y_exp) > 0.9, forced
    # oracle: bf16 activations x dequantised weight, float64 accumulation
    wd = o.dequantize_fp8(codes, 1.0, "e4m3").reshape(cout, c, k, k) * scales.reshape(-1, 1, 1, 1)
    xb = o.bf16_bits_to_f32(o.f32_to_bf16_bits(x))
    col, oh, ow = o.im2col(xb, k, k, 1, 1, p, p)
    ref = (wd.reshape(cout, -1).astype(np.float64) @ col.astype(np.float64) + b.reshape(-1, 1))
    ref = ref.reshape(cout, n, oh, ow).transpose(1, 0, 2, 3)
    assert o.max_abs_rel(y_imp, ref) <= 1e-2
    F.check_device_errors(gpu)


@pytest.mark.parametrize("case", [
    (2, 64, 16, 16, 64, 3, 1, 2, 2),      # ResNet-style 3 x 3 stride 2: boxes of every second pixel
    (3, 128, 15, 13, 72, 3, 1, 2, 2),     # odd sizes: the last strided pixel sits on the padding
    (2, 64, 12, 20, 40, 3, 0, 2, 2),      # no padding
    (2, 64, 9, 17, 24, 3, 1, 1, 2),       # stride 2 across only
    (2, 64, 17, 9, 24, 5, 2, 2, 1),       # stride 2 down only, 5 x 5 taps
    (37, 64, 28, 28, 128, 3, 1, 2, 2),    # several tiles per CTA pair
])
def test_strided_implicit_gemm_conv(gpu, case):
    """Strides of 2: the 4-D TMA box walks the NHWC tensor with a traversal stride, so the box of
    a filter tap still lands as consecutive operand rows.  Against the patch-matrix path of the
    same call and against the oracle."""
    n, c, h, w, cout, k, p, sh, sw = case
    rng = np.random.default_rng(sum(case))
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (rng.standard_normal((cout, c, k, k)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    codes, scales = quant.quantize_weight(wt.reshape(cout, -1), "e4m3", gpu)
    y_imp = F.conv2d_q_host(x, codes, scales, b, (k, k), (sh, sw), (p, p), "zeros", "e4m3", gpu)
    y_exp = F.conv2d_q_host(x, codes, scales, b, (k, k), (sh, sw), (p, p), "zeros", "e4m3", gpu,
                            path="patch_matrix")
    oh, ow = (h + 2 * p - k) // sh + 1, (w + 2 * p - k) // sw + 1
    assert y_imp.shape == y_exp.shape == (n, cout, oh, ow)
    assert o.max_abs_rel(y_imp, y_exp) <= 2.0 ** -8
    assert np.mean(y_imp == y_exp) > 0.9
    for forced in ("cta_pair", "auto"):
        y_f = F.conv2d_q_host(x, codes, scales, b, (k, k), (sh, sw), (p, p), "zeros", "e4m3", gpu, path=forced)
        assert o.max_abs_rel(y_f, y_exp) <= 2.0 ** -8, forced
        assert np.mean(y_f == y_exp) > 0.9, forced
    wd = o.dequantize_fp8(codes, 1.0, "e4m3").reshape(cout, c, k, k) * scales.reshape(-1, 1, 1, 1)
    xb = o.bf16_bits_to_f32(o.f32_to_bf16_bits(x))
    col, oh2, ow2 = o.im2col(xb, k, k, sh, sw, p, p)
    ref = (wd.reshape(cout, -1).astype(np.float64) @ col.astype(np.float64) + b.reshape(-1, 1))
    ref = ref.reshape(cout, n, oh2, ow2).transpose(1, 0, 2, 3)
    assert o.max_abs_rel(y_imp, ref) <= 1e-2
    F.check_device_errors(gpu)


@pytest.mark.parametrize("case", [
    (2, 64, 10, 10, 32, 3, 1, 1),      # implicit GEMM (stride 1, C % 64 == 0)
    (3, 128, 7, 9, 72, 3, 1, 1),       # implicit, two channel blocks, odd CTA-tile count
    (2, 16, 9, 9, 24, 3, 2, 1),        # patch-matrix path (stride 2, C = 16): kpad = 160
    (2, 3, 8, 8, 8, 5, 1, 2),          # patch-matrix path, K = 75 -> kpad = 96
])
def test_fp4_weight_conv2d(gpu, case):
    """FP4 E2M1 block-32 weights through the quantised convolution (block scales folded into the
    expanded weight): both paths against the oracle within the FP4 bound, and against each other
    where both apply."""
    n, c, h, w, cout, k, s, p = case
    rng = np.random.default_rng(sum(case))
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (rng.standard_normal((cout, c, k, k)) * 0.1).astype(np.float32)
    b = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    ckk = c * k * k
    kpad = (ckk + 31) // 32 * 32
    w_col = np.zeros((cout, kpad), np.float32)
    w_col[:, :ckk] = wt.reshape(cout, -1)
    packed, scales = quant.quantize_weight(w_col, "e2m1_b32", gpu)
    assert packed.shape == (cout, kpad // 2) and scales.shape == (cout, kpad // 32)
    y = F.conv2d_q_host(x, packed, scales, b, (k, k), (s, s), (p, p), "zeros", "e2m1_b32", gpu)
    # oracle: the same codes and scales, bf16 activations, float64 contraction
    wd = o.dequantize_fp4_weight(packed, scales)
    wd = o.bf16_bits_to_f32(o.f32_to_bf16_bits(wd))[:, :ckk]         # the kernels expand to bf16(value * scale)
    xb = o.bf16_bits_to_f32(o.f32_to_bf16_bits(x))
    col, oh, ow = o.im2col(xb, k, k, s, s, p, p)
    ref = (wd.astype(np.float64) @ col.astype(np.float64) + b.reshape(-1, 1)).reshape(cout, n, oh, ow).transpose(1, 0, 2, 3)
    assert y.shape == ref.shape
    assert o.max_abs_rel(y, ref) <= 2.0 ** -7          # same codes: only the bf16 rounding of y is left
    # and against the fp32 convolution with the unquantised weight, within the FP4 bound
    ref32 = o.conv2d_fwd_f32(xb, wt, b.reshape(-1, 1), (s, s), (p, p))
    assert o.max_abs_rel(y, ref32) <= 2.5e-1           # 4-bit weights; the spec's 5e-2 is for the codes' own GEMM
    if s == 1 and c % 64 == 0:
        y2 = F.conv2d_q_host(x, packed, scales, b, (k, k), (s, s), (p, p), "zeros", "e2m1_b32", gpu,
                             path="patch_matrix")
        assert o.max_abs_rel(y, y2) <= 2.0 ** -8
    F.check_device_errors(gpu)


def test_quant_conv2d_layer_fp4(gpu):
    layer = nb.QuantConv2d(64, 16, 3, padding=1, fmt="e2m1_b32", device=gpu)
    x = np.random.default_rng(0).standard_normal((2, 64, 6, 6)).astype(np.float32)
    y = layer(x)
    ref = o.conv2d_fwd_f32(x, layer.weight.data, layer.bias.data, (1, 1), (1, 1))
    assert y.shape == ref.shape and o.max_abs_rel(y, ref) <= 2.5e-1


@pytest.mark.parametrize("case", [
    (2, 64, 16, 16, 64, 3, 1, 1),       # one channel block; quarters past Cout are clipped by the store
    (3, 128, 15, 13, 72, 3, 1, 1),      # odd sizes: ragged tiles take the register-store tail
    (2, 64, 12, 20, 40, 3, 0, 2),       # stride 2, no padding
    (5, 64, 28, 28, 128, 3, 1, 1),      # whole tiles, TMA stores only
    (2, 64, 9, 17, 264, 5, 2, 1),       # three channel blocks, 5 x 5 taps
])
@pytest.mark.parametrize("relu", [False, True])
def test_nhwc_bf16_conv_equals_the_nchw_entry_point(gpu, case, relu):
    """nvq_conv2d_fwd_q_nhwc (bf16 NHWC in and out, the contract between chained quantised
    layers) against nvq_conv2d_fwd_q on the same codes: the same kernel does the contraction, so
    the bf16 results are the same bits once both are laid out alike; ReLU is the reference's
    v * (v > 0)."""
    from novann_b200.device import DeviceBuffer
    n, c, h, w, cout, k, p, s = case
    rng = np.random.default_rng(sum(case))
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wt = (rng.standard_normal((cout, c, k, k)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    codes, scales = quant.quantize_weight(wt.reshape(cout, -1), "e4m3", gpu)
    want = F.conv2d_q_host(x, codes, scales, b, (k, k), (s, s), (p, p), "zeros", "e4m3", gpu)
    if relu:
        want = want * (want > 0)
    oh, ow = want.shape[2], want.shape[3]
    dx32 = DeviceBuffer.from_numpy(x, gpu)
    dx = DeviceBuffer(x.size * 2, gpu)
    F.nchw_f32_to_nhwc_bf16_device(dx, dx32, n, c, h * w)
    assert np.array_equal(dx.to_numpy(np.uint16, (n, h, w, c)),
                          o.f32_to_bf16_bits(x).reshape(n, c, h, w).transpose(0, 2, 3, 1))
    dq, ds, db = (DeviceBuffer.from_numpy(a, gpu) for a in (codes, scales, b))
    ws = DeviceBuffer(cout * c * k * k * 2, gpu)
    guard = 256
    dy = DeviceBuffer(n * oh * ow * cout * 2 + guard, gpu)
    dy.zero()
    F.conv2d_q_nhwc_device(dy, dx, dq, "e4m3", ds, db, ws, n, c, h, w, cout, (k, k), (s, s), (p, p), relu=relu)
    from novann_b200.device import device_sync
    device_sync(gpu)
    F.check_device_errors(gpu)
    y = dy.to_numpy(np.uint16, (n * oh * ow * cout + guard // 2,))
    assert not y[n * oh * ow * cout:].any()                       # nothing written past the end
    got = o.bf16_bits_to_f32(y[:n * oh * ow * cout]).reshape(n, oh, ow, cout).transpose(0, 3, 1, 2)
    assert np.array_equal(got.view(np.uint32), np.ascontiguousarray(want).view(np.uint32))
    back = DeviceBuffer(n * oh * ow * cout * 4, gpu)
    F.nhwc_bf16_to_nchw_f32_device(back, dy, n, cout, oh * ow)
    assert np.array_equal(back.to_numpy(np.float32, want.shape).view(np.uint32), np.ascontiguousarray(want).view(np.uint32))


def test_quant_conv_chain_keeps_activations_bf16_nhwc(gpu):
    """Three chained quantised convolutions with ReLU between them: one layout conversion at each
    end, none between layers; equal, bit for bit, to three separate calls of the NCHW entry
    point with ReLU on the host in between."""
    from novann_b200.train import QuantConvChain
    rng = np.random.default_rng(11)
    x = rng.standard_normal((4, 64, 20, 20)).astype(np.float32)
    specs = []
    for cin, cout, stride, relu in ((64, 128, 1, True), (128, 64, 2, True), (64, 72, 1, False)):
        specs.append(dict(weight=(rng.standard_normal((cout, cin, 3, 3)) * (2.0 / (9 * cin)) ** 0.5).astype(np.float32),
                          bias=(rng.standard_normal(cout) * 0.1).astype(np.float32),
                          stride=(stride, stride), padding=(1, 1), relu=relu))
    chain = QuantConvChain(specs, x.shape, "e4m3", gpu)
    got = chain.forward(x)
    cur = x
    for sp in specs:
        cout = sp["weight"].shape[0]
        codes, scales = quant.quantize_weight(sp["weight"].reshape(cout, -1), "e4m3", gpu)
        cur = F.conv2d_q_host(cur, codes, scales, sp["bias"], (3, 3), sp["stride"], sp["padding"], "zeros", "e4m3", gpu)
        if sp["relu"]:
            cur = cur * (cur > 0)
    assert got.shape == cur.shape == (4, 72, 10, 10)
    assert np.array_equal(got.view(np.uint32), np.ascontiguousarray(cur).view(np.uint32))
    assert np.array_equal(chain.forward(x).view(np.uint32), got.view(np.uint32))     # same bits twice


def test_nhwc_conv_refuses_shapes_outside_its_rule(gpu):
    from novann_b200.device import DeviceBuffer
    d = DeviceBuffer(1 << 16, gpu)
    from novann_b200 import _lib
    st = _lib.lib().nvq_conv2d_fwd_q_nhwc(d.at(0), d.at(0), d.at(0), _lib.E4M3, d.at(0), None, d.at(0), d.nbytes,
                                          1, 48, 8, 8, 16, 3, 3, 1, 1, 1, 1, 0, gpu, None)      # C % 64 != 0
    assert st == _lib.ERR_UNSUPPORTED and b"nvq_conv2d_fwd_q" in _lib.lib().nvq_last_error()
    st = _lib.lib().nvq_conv2d_fwd_q_nhwc(d.at(0), d.at(0), d.at(0), _lib.E4M3, d.at(0), None, d.at(0), d.nbytes,
                                          1, 64, 8, 8, 16, 3, 3, 3, 3, 1, 1, 0, gpu, None)      # stride 3
    assert st == _lib.ERR_UNSUPPORTED
