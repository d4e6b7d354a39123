"""Device-resident training step of a Sequential CNN: the loop body of the reference's main.py
(main.py:74-90: zero_grad, forward, CrossEntropyLoss, backward, AdamW.step) with every tensor
kept in HBM between layers.

The model is given as a list of ``(kind, args)`` pairs; ``main_cnn_spec()`` is the network of
main.py:24-46.  Parameters live in two flat device buckets -- fp32 (convolution and Linear
weights, biases) and float64 (BatchNorm gamma / beta, which the reference keeps as float64) --
so that AdamW is one launch per bucket; activations, ReLU masks, im2col matrices and BatchNorm
statistics are allocated once.  A step is a fixed launch sequence on one stream; forward, loss
and backward can be captured into a CUDA graph and replayed.  Per step the host uploads the
batch, the labels and the Dropout keep masks (drawn on the host from NumPy's generator with
the reference's call, so that a seeded run drops the same units).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib, PAD_MODES
from .device import DeviceBuffer, Stream, _sptr


def main_cnn_spec():
    """The reference's main.py network (main.py:24-46) for 1x28x28 inputs."""
    return [
        ("conv", dict(cin=1, cout=16, k=3, s=1, p=1)), ("bn", dict(c=16)), ("relu", {}),
        ("conv", dict(cin=16, cout=32, k=3, s=2, p=1)), ("bn", dict(c=32)), ("relu", {}),
        ("maxpool", dict(k=2, s=2)),
        ("conv", dict(cin=32, cout=64, k=3, s=1, p=1)), ("bn", dict(c=64)), ("relu", {}),
        ("gap", {}), ("flatten", {}),
        ("linear", dict(fin=64, fout=32, bias=False)), ("bn", dict(c=32)), ("relu", {}),
        ("dropout", dict(p=0.5)),
        ("linear", dict(fin=32, fout=10, bias=True)),
    ]


class _Node:
    """One layer's resolved geometry and buffers."""

    def __init__(self, kind, args, in_shape):
        self.kind, self.a, self.in_shape = kind, args, in_shape
        self.out_shape = None
        self.p32 = []      # (offset in elements, size) into the fp32 bucket
        self.p64 = []      # (offset, size) into the float64 bucket
        self.buf = {}


def _numel(shape):
    return int(np.prod(shape, dtype=np.int64))


class CNNTrainStep:
    """``step(x, labels)`` runs forward, loss, backward and the AdamW update on the device.
    Read results with ``logits()``, ``loss()``, ``grads()``, ``params()``, ``running_stats()``.

    ``params`` is the list ``Sequential.parameters()`` gives for the same model: per layer the
    weight then the bias; for BatchNorm gamma then beta (float64)."""

    def __init__(self, spec, params, batch: int, in_shape, lr: float = 1e-3, betas=(0.9, 0.999),
                 weight_decay: float = 1e-2, epsilon: float = 1e-8, momentum: float = 0.1,
                 bn_eps: float = 1e-5, device: int = 0):
        self.device, self.batch = device, batch
        self.lr, self.b1, self.b2 = float(lr), float(betas[0]), float(betas[1])
        self.wd, self.eps = float(weight_decay), float(epsilon)
        self.momentum, self.bn_eps = float(momentum), float(bn_eps)
        self.t = 0
        self.stream = Stream(device)
        self._graph = None
        self.launches_per_step = 0
        self.training = True
        # ---- resolve shapes and parameter slots
        self.nodes = []
        shape = (batch, *in_shape)
        n32 = n64 = 0
        self._order = []                                    # (bucket, offset, shape) per parameter
        for kind, a in spec:
            nd = _Node(kind, a, shape)
            if kind == "conv":
                n, c, h, w = shape
                if c != a["cin"]:
                    raise ValueError(f"conv expects {a['cin']} channels, got {c}")
                oh = (h + 2 * a["p"] - a["k"]) // a["s"] + 1
                ow = (w + 2 * a["p"] - a["k"]) // a["s"] + 1
                nd.out_shape = (n, a["cout"], oh, ow)
                size = a["cout"] * c * a["k"] * a["k"]
                nd.p32.append((n32, size))
                self._order.append((32, n32, (a["cout"], c, a["k"], a["k"])))
                n32 += size
            elif kind == "bn":
                if shape[1] != a["c"]:
                    raise ValueError(f"BatchNorm expects {a['c']} features, got {shape[1]}")
                nd.out_shape = shape
                pshape = (1, a["c"], 1, 1) if len(shape) == 4 else ((1, a["c"], 1) if len(shape) == 3 else (1, a["c"]))
                for _ in range(2):
                    nd.p64.append((n64, a["c"]))
                    self._order.append((64, n64, pshape))
                    n64 += a["c"]
            elif kind in ("relu", "dropout"):
                nd.out_shape = shape
            elif kind == "maxpool":
                n, c, h, w = shape
                nd.out_shape = (n, c, (h - a["k"]) // a["s"] + 1, (w - a["k"]) // a["s"] + 1)
            elif kind == "gap":
                nd.out_shape = (shape[0], shape[1], 1, 1)
            elif kind == "flatten":
                nd.out_shape = (shape[0], _numel(shape[1:]))
            elif kind == "linear":
                if len(shape) != 2 or shape[1] != a["fin"]:
                    raise ValueError(f"linear expects (N, {a['fin']}) input, got {shape}")
                nd.out_shape = (shape[0], a["fout"])
                nd.p32.append((n32, a["fout"] * a["fin"]))
                self._order.append((32, n32, (a["fout"], a["fin"])))
                n32 += a["fout"] * a["fin"]
                if a["bias"]:
                    nd.p32.append((n32, a["fout"]))
                    self._order.append((32, n32, (1, a["fout"])))
                    n32 += a["fout"]
            else:
                raise ValueError(f"unknown layer kind '{kind}'")
            shape = nd.out_shape
            self.nodes.append(nd)
        if len(params) != len(self._order):
            raise ValueError(f"model has {len(self._order)} parameters, {len(params)} given")
        self.n32, self.n64 = n32, n64
        flat32, flat64 = np.zeros(max(1, n32), np.float32), np.zeros(max(1, n64), np.float64)
        for (bucket, off, shp), p in zip(self._order, params):
            if tuple(p.shape) != tuple(shp):
                raise ValueError(f"parameter shape {p.shape} does not match {shp}")
            (flat32 if bucket == 32 else flat64)[off:off + p.size] = np.asarray(p).ravel()
        # ---- device buffers
        D = lambda nbytes: DeviceBuffer(max(8, nbytes), device)   # noqa: E731
        self.d_p32, self.d_p64 = DeviceBuffer.from_numpy(flat32, device), DeviceBuffer.from_numpy(flat64, device)
        self.d_g32, self.d_g64 = D(flat32.nbytes), D(flat64.nbytes)
        self.d_m32, self.d_v32, self.d_m64, self.d_v64 = D(flat32.nbytes), D(flat32.nbytes), D(flat64.nbytes), D(flat64.nbytes)
        for b in (self.d_g32, self.d_g64, self.d_m32, self.d_v32, self.d_m64, self.d_v64):
            b.zero()
        self.d_x = D(4 * _numel((batch, *in_shape)))
        self.d_labels = D(4 * batch)
        self.d_loss = D(4)
        max_c = max([nd.a["c"] for nd in self.nodes if nd.kind == "bn"] + [1])
        self.d_bn_scratch = D(lib().nvq_batchnorm_scratch_bytes(max_c))
        self._drop_nodes = []
        max_grad = 0
        for nd in self.nodes:
            out_b = 4 * _numel(nd.out_shape)
            max_grad = max(max_grad, 4 * _numel(nd.in_shape), out_b)
            if nd.kind != "flatten":
                nd.buf["out"] = D(out_b)
            if nd.kind == "conv":
                n, c, h, w = nd.in_shape
                _, co, oh, ow = nd.out_shape
                ckk, L = c * nd.a["k"] ** 2, n * oh * ow
                nd.buf["col"], nd.buf["dcol"], nd.buf["gr"] = D(4 * ckk * L), D(4 * ckk * L), D(4 * co * L)
            elif nd.kind == "bn":
                c = nd.a["c"]
                nd.buf["stats"] = D(8 * c)
                rs = np.concatenate([np.zeros(c), np.ones(c)])
                nd.buf["running"] = DeviceBuffer.from_numpy(rs, device)    # mean then var, float64
            elif nd.kind == "relu":
                nd.buf["mask"] = D(out_b)
            elif nd.kind == "dropout":
                nd.buf["mask"] = D(out_b)
                self._drop_nodes.append(nd)
        last = self.nodes[-1].out_shape
        if len(last) != 2:
            raise ValueError("the model must end in (N, classes) logits")
        self.n_classes = last[1]
        self.d_yhat = D(4 * batch * self.n_classes)
        # two gradient buffers, used alternately down the backward pass
        self.d_grad = [D(max_grad), D(max_grad)]

    # ---- host -> device
    def upload(self, x: np.ndarray, labels: np.ndarray, drop_masks=None) -> None:
        x = np.ascontiguousarray(x, np.float32)
        if x.shape != (self.batch, *self.nodes[0].in_shape[1:]):
            raise ValueError(f"input shape {x.shape} does not match {self.nodes[0].in_shape}")
        self.d_x.upload(x, stream=self.stream)
        self.d_labels.upload(np.ascontiguousarray(labels, np.int32), stream=self.stream)
        if self.training and self._drop_nodes:
            if drop_masks is None:
                # the reference's own draw (dropout.py:52), one per Dropout layer in forward order
                drop_masks = [(np.random.rand(*nd.out_shape) < 1.0 - nd.a["p"]) for nd in self._drop_nodes]
            for nd, mk in zip(self._drop_nodes, drop_masks):
                nd.buf["mask"].upload(np.ascontiguousarray(mk, np.float32), stream=self.stream)

    # ---- the launch sequences
    def _p32(self, nd, i):
        return self.d_p32.at(4 * nd.p32[i][0])

    def _g32(self, nd, i):
        return self.d_g32.at(4 * nd.p32[i][0])

    def launch_forward(self) -> None:
        L, dev, st = lib(), self.device, _sptr(self.stream)
        cur = self.d_x
        for nd in self.nodes:
            k, a = nd.kind, nd.a
            out = nd.buf.get("out")
            if k == "conv":
                n, c, h, w = nd.in_shape
                check(L.nvq_conv2d_fwd_f32(out.at(0), cur.at(0), self._p32(nd, 0), None, nd.buf["col"].at(0),
                                           n, c, h, w, a["cout"], a["k"], a["k"], a["s"], a["s"], a["p"], a["p"],
                                           PAD_MODES["zeros"], dev, st))
            elif k == "bn":
                n, c = nd.in_shape[0], nd.in_shape[1]
                s = _numel(nd.in_shape[2:])
                check(L.nvq_batchnorm_fwd_f32(out.at(0), cur.at(0), self.d_p64.at(8 * nd.p64[0][0]),
                                              self.d_p64.at(8 * nd.p64[1][0]), nd.buf["running"].at(0),
                                              nd.buf["running"].at(8 * c), nd.buf["stats"].at(0),
                                              self.d_bn_scratch.at(0), n, c, s, self.momentum, self.bn_eps,
                                              int(self.training), dev, st))
            elif k == "relu":
                check(L.nvq_relu_fwd_f32(out.at(0), nd.buf["mask"].at(0), cur.at(0), _numel(nd.out_shape), dev, st))
            elif k == "maxpool":
                n, c, h, w = nd.in_shape
                check(L.nvq_maxpool2d_fwd_f32(out.at(0), cur.at(0), n, c, h, w, a["k"], a["k"], a["s"], a["s"],
                                              0, 0, PAD_MODES["zeros"], dev, st))
            elif k == "gap":
                n, c, h, w = nd.in_shape
                check(L.nvq_gap2d_fwd_f32(out.at(0), cur.at(0), n * c, h * w, dev, st))
            elif k == "flatten":
                out = cur
            elif k == "linear":
                check(L.nvq_linear_fwd_f32(out.at(0), cur.at(0), self._p32(nd, 0),
                                           self._p32(nd, 1) if a["bias"] else None, nd.in_shape[0], a["fout"],
                                           a["fin"], 0, None, dev, st))
            elif k == "dropout":
                if self.training:
                    check(L.nvq_dropout_f32(out.at(0), cur.at(0), nd.buf["mask"].at(0), _numel(nd.out_shape),
                                            C.c_float(1.0 - a["p"]), dev, st))
                else:
                    out = cur
            nd.buf["in"] = cur
            cur = out
        self._logits = cur

    def launch_backward(self) -> None:
        L, dev, st = lib(), self.device, _sptr(self.stream)
        check(L.nvq_softmax_ce_f32(self.d_grad[0].at(0), self.d_loss.at(0), self._logits.at(0),
                                   self.d_labels.at(0), self.d_yhat.at(0), self.batch, self.n_classes, dev, st))
        g, flip = self.d_grad[0], 0
        first_param_node = next(i for i, nd in enumerate(self.nodes) if nd.p32 or nd.p64)
        for idx in reversed(range(len(self.nodes))):
            nd = self.nodes[idx]
            k, a = nd.kind, nd.a
            need_dx = idx > first_param_node
            nxt = self.d_grad[flip ^ 1]
            if k == "conv":
                n, c, h, w = nd.in_shape
                check(L.nvq_conv2d_bwd_f32(self._g32(nd, 0), None, nxt.at(0) if need_dx else None, g.at(0),
                                           nd.buf["col"].at(0), self._p32(nd, 0), nd.buf["gr"].at(0),
                                           nd.buf["dcol"].at(0), n, c, h, w, a["cout"], a["k"], a["k"],
                                           a["s"], a["s"], a["p"], a["p"], dev, st))
            elif k == "bn":
                n, c = nd.in_shape[0], nd.in_shape[1]
                s = _numel(nd.in_shape[2:])
                check(L.nvq_batchnorm_bwd_f32(nxt.at(0) if need_dx else None,
                                              self.d_g64.at(8 * nd.p64[0][0]), self.d_g64.at(8 * nd.p64[1][0]),
                                              g.at(0), nd.buf["in"].at(0), nd.buf["stats"].at(0),
                                              self.d_p64.at(8 * nd.p64[0][0]), self.d_bn_scratch.at(0),
                                              n, c, s, self.bn_eps, dev, st))
            elif k == "relu":
                check(L.nvq_mul_f32(nxt.at(0), g.at(0), nd.buf["mask"].at(0), _numel(nd.out_shape), dev, st))
            elif k == "maxpool":
                n, c, h, w = nd.in_shape
                check(L.nvq_maxpool2d_bwd_f32(nxt.at(0), g.at(0), nd.buf["in"].at(0), n, c, h, w, a["k"], a["k"],
                                              a["s"], a["s"], 0, 0, PAD_MODES["zeros"], dev, st))
            elif k == "gap":
                n, c, h, w = nd.in_shape
                check(L.nvq_gap2d_bwd_f32(nxt.at(0), g.at(0), n * c, h * w, dev, st))
            elif k == "flatten":
                continue                                   # same buffer, other shape
            elif k == "linear":
                check(L.nvq_linear_bwd_f32(self._g32(nd, 0), self._g32(nd, 1) if a["bias"] else None,
                                           nxt.at(0) if need_dx else None, g.at(0), nd.buf["in"].at(0),
                                           self._p32(nd, 0), None, nd.in_shape[0], a["fout"], a["fin"], dev, st))
            elif k == "dropout":
                check(L.nvq_dropout_f32(nxt.at(0), g.at(0), nd.buf["mask"].at(0), _numel(nd.out_shape),
                                        C.c_float(1.0 - a["p"]), dev, st))
            if not need_dx:
                break
            g, flip = nxt, flip ^ 1

    def launch_update(self) -> None:
        """AdamW over the two buckets (one launch each).  Its bias corrections change with the
        step number, so these two launches stay outside the captured graph."""
        L, dev, st = lib(), self.device, _sptr(self.stream)
        t = self.t
        f, d = C.c_float, C.c_double
        bc1, bc2 = 1 - self.b1 ** t, 1 - self.b2 ** t
        if self.n32:
            check(L.nvq_adamw_step_f32(self.d_p32.at(0), self.d_g32.at(0), self.d_m32.at(0), self.d_v32.at(0),
                                       self.n32, f(self.b1), f(1 - self.b1), f(self.b2), f(1 - self.b2),
                                       f(bc1), f(bc2), f(self.lr), f(self.eps), f(self.lr * self.wd),
                                       int(self.wd > 0), dev, st))
        if self.n64:
            check(L.nvq_adamw_step_f64(self.d_p64.at(0), self.d_g64.at(0), self.d_m64.at(0), self.d_v64.at(0),
                                       self.n64, d(self.b1), d(1 - self.b1), d(self.b2), d(1 - self.b2),
                                       d(bc1), d(bc2), d(self.lr), d(self.eps), d(self.lr * self.wd), 0, dev, st))

    # ---- public
    def step(self, x: np.ndarray, labels: np.ndarray, drop_masks=None) -> None:
        if not self.training:
            raise RuntimeError("step() needs training mode; call train() first")
        self.t += 1
        self.upload(x, labels, drop_masks)
        if self._graph is not None:
            check(lib().nvq_graph_launch(self.device, C.c_void_p(self._graph), _sptr(self.stream)))
            self.launch_update()
        else:
            before = lib().nvq_launch_count()
            self.launch_forward()
            self.launch_backward()
            self.launch_update()
            self.launches_per_step = int(lib().nvq_launch_count() - before)   # this library's kernels
        self.stream.sync()

    def capture(self) -> None:
        """Record forward + loss + backward into a CUDA graph (after one eager step, so that
        first-call set-up is done); later steps replay it and then launch AdamW."""
        if self._graph is not None:
            return
        check(lib().nvq_graph_begin_capture(self.device, _sptr(self.stream)))
        try:
            self.launch_forward()
            self.launch_backward()
        finally:
            h = C.c_void_p()
            check(lib().nvq_graph_end_capture(self.device, _sptr(self.stream), C.byref(h)))
        self._graph = h.value

    def replay(self) -> None:
        """Enqueue one more training step on the batch already in HBM (no upload, no sync):
        the captured graph if there is one, else the eager sequence; then AdamW."""
        self.t += 1
        if self._graph is not None:
            check(lib().nvq_graph_launch(self.device, C.c_void_p(self._graph), _sptr(self.stream)))
        else:
            self.launch_forward()
            self.launch_backward()
        self.launch_update()

    def forward(self, x: np.ndarray) -> np.ndarray:
        """Forward pass only (uses running statistics and no Dropout after ``eval()``)."""
        self.upload(x, np.zeros(self.batch, np.int32))
        self.launch_forward()
        self.stream.sync()
        return self.logits()

    def train(self) -> None:
        self.training = True

    def eval(self) -> None:
        self.training = False

    # ---- results
    def logits(self) -> np.ndarray:
        return self._logits.to_numpy(np.float32, (self.batch, self.n_classes))

    def loss(self) -> np.float32:
        return self.d_loss.to_numpy(np.float32, (1,))[0]

    def _unflatten(self, b32: np.ndarray, b64: np.ndarray):
        out = []
        for bucket, off, shp in self._order:
            src = b32 if bucket == 32 else b64
            out.append(src[off:off + _numel(shp)].reshape(shp).copy())
        return out

    def params(self):
        return self._unflatten(self.d_p32.to_numpy(np.float32, (max(1, self.n32),)),
                               self.d_p64.to_numpy(np.float64, (max(1, self.n64),)))

    def grads(self):
        return self._unflatten(self.d_g32.to_numpy(np.float32, (max(1, self.n32),)),
                               self.d_g64.to_numpy(np.float64, (max(1, self.n64),)))

    def running_stats(self):
        """[(running_mean, running_var)] per BatchNorm layer, float64."""
        out = []
        for nd in self.nodes:
            if nd.kind == "bn":
                c = nd.a["c"]
                r = nd.buf["running"].to_numpy(np.float64, (2 * c,))
                out.append((r[:c].copy(), r[c:].copy()))
        return out
