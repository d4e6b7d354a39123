"""GPU-backed layers with the reference's ``Layer`` contract (NumPy in, NumPy out).

* ``Linear`` / ``ReLU`` / ``Conv2d``: fp32, the reference's own arithmetic on the GPU
  (``novann/layers/linear/linear.py``, ``novann/layers/activations/relu.py``,
  ``novann/layers/convolutional/conv2d.py`` forward).
* ``QuantLinear`` / ``QuantConv2d``: the weight is kept as FP8 (per output channel) or FP4
  (block 32) codes and the forward contraction runs on the tcgen05 tensor cores with bf16
  activations.  ``parameters()`` still exposes the fp32 master weight; ``requantize()``
  refreshes the codes after the optimiser changed it.

Every call uploads its inputs and downloads its result (that is the reference's API); the
device-resident fast path for whole training steps is ``novann_b200.train``.
"""
from __future__ import annotations

import numpy as np

from . import functional as F
from .device import DeviceBuffer
from .module import Layer, Parameters


def kaiming_normal(shape) -> np.ndarray:
    """N(0, 2 / fan_in) from the global legacy NumPy RNG, the law the reference's Sequential
    gives a Linear followed by ReLU (novann/core/init.py:155-179)."""
    fan_in = int(np.prod(shape[1:]))
    return np.random.normal(0.0, np.sqrt(2.0 / fan_in), shape).astype(np.float32)


def small_normal(shape) -> np.ndarray:
    """0.001 * N(0, 1): the law a stand-alone reference ``Linear`` starts from
    (novann/core/init.py:209-219), drawn with the same call on the global legacy NumPy
    generator, so a seeded model gets the reference's weights."""
    return np.random.randn(*shape).astype(np.float32) * 0.001


def kaiming_uniform_relu(shape) -> np.ndarray:
    """U(-l, l), l = sqrt(2) * sqrt(3 / fan_in): the law a stand-alone reference ``Conv2d``
    starts from (novann/layers/convolutional/conv2d.py:62, novann/core/init.py:182-206)."""
    fan_in = int(np.prod(shape[1:]))
    limit = np.sqrt(2.0) * np.sqrt(3.0 / fan_in)
    return np.random.uniform(-limit, limit, shape).astype(np.float32)


def _pair(x):
    if isinstance(x, int):
        return (x, x)
    if isinstance(x, str):
        if x == "valid":
            return (0, 0)
        if x == "same":
            raise ValueError("The 'same' value is not currently supported")
        raise ValueError(f"Unsupported value '{x}'")
    return tuple(x)


def _dev(a: np.ndarray, device: int) -> DeviceBuffer:
    return DeviceBuffer.from_numpy(np.ascontiguousarray(a), device)


def _as_f32(x: np.ndarray, device: int) -> np.ndarray:
    """The reference's layer-entry ``x.astype(np.float32, copy=False)``
    (novann/layers/linear/linear.py:81): float32 passes through untouched; float64 (what a
    reference BatchNorm emits) and float16 are narrowed / widened on the GPU by ``nvq_cast``.
    Other dtypes are refused: nothing is converted on the CPU."""
    x = np.asarray(x)
    if x.dtype == np.float32:
        return np.ascontiguousarray(x)
    if x.dtype in (np.float64, np.float16):
        from . import quant
        return quant.cast(x, np.float32, device=device)
    raise TypeError(f"layer input must be float32, float64 or float16, got {x.dtype}")


class Linear(Layer):
    """y = x W^T + b in fp32 on the GPU; same attributes and gradient rules as the reference."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, init=None,
                 device: int = 0) -> None:
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.use_bias = bias
        self.init_fn = init
        self.device = device
        self.weight = None
        self.bias = None
        self._cache_input = None
        self.reset_parameters()

    def reset_parameters(self, initializer=None) -> None:
        init = initializer or self.init_fn or small_normal
        w = init((self.out_features, self.in_features))
        self.weight = Parameters(np.asarray(w, dtype=np.float32))
        self.weight.name = "linear weight"
        if self.use_bias:
            self.bias = Parameters(np.zeros((1, self.out_features), dtype=np.float32))
            self.bias.name = "linear bias"
        else:
            self.bias = None

    def forward(self, x: np.ndarray) -> np.ndarray:
        x = _as_f32(x, self.device)
        self._cache_input = x
        return F.linear_f32_host(x, self.weight.data, None if self.bias is None else self.bias.data,
                                 self.device)

    def backward(self, grad: np.ndarray) -> np.ndarray:
        grad = _as_f32(grad, self.device)
        dw, db, dx = F.linear_bwd_f32_host(grad, self._cache_input, self.weight.data,
                                           self.bias is not None, self.device)
        self.weight.grad = dw
        if self.bias is not None:
            self.bias.grad = db
        return dx

    def parameters(self):
        return [self.weight] + ([self.bias] if self.bias is not None else [])

    def __repr__(self):
        return f"Linear(in_features={self.in_features}, out_features={self.out_features}, bias={self.use_bias})"


class ReLU(Layer):
    """``novann/layers/activations/relu.py``.  ``name`` / ``affect_init`` / ``init_key`` are what
    the reference's ``Sequential`` reads from an activation to choose the initialiser of the
    weighted layers around it (novann/layers/activations/activations.py:19-38)."""

    def __init__(self, device: int = 0) -> None:
        super().__init__()
        self._mask = None
        self.device = device
        self.name = "relu"
        self.affect_init = True

    def get_init_key(self):
        return self.name if self.affect_init else None

    @property
    def init_key(self):
        return self.get_init_key()

    def forward(self, x: np.ndarray) -> np.ndarray:
        out, self._mask = F.relu_host(_as_f32(x, self.device), self.device)
        return out

    def backward(self, grad: np.ndarray) -> np.ndarray:
        return F.mul_host(grad, self._mask, self.device)

    def __repr__(self):
        return "ReLU()"


class QuantLinear(Linear):
    """Linear whose forward contraction uses FP8 / FP4 weight codes on the tensor cores.

    Forward: ``bf16(x) @ dequant(Wq)^T * s + b`` -> bf16 -> returned as float32.  Backward
    follows the reference's rules (straight-through to the fp32 master weight): in fp32 on
    the CUDA cores by default, or with ``tensor_core_backward=True`` (FP8 formats, batch and
    feature sizes multiples of 8) as bf16 contractions on the tensor cores against the codes."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, init=None,
                 fmt: str = "e4m3", device: int = 0, tensor_core_backward: bool = False) -> None:
        self.fmt = fmt
        self.tensor_core_backward = tensor_core_backward
        self._codes = self._scales = self._resident = None
        super().__init__(in_features, out_features, bias, init, device)

    def reset_parameters(self, initializer=None) -> None:
        super().reset_parameters(initializer)
        self._codes = self._scales = None      # quantised on the next forward
        self._resident = None

    def requantize(self) -> None:
        """Recompute the weight codes from ``weight.data``."""
        from . import quant
        self._codes, self._scales = quant.quantize_weight(self.weight.data, self.fmt, self.device)
        self._resident = None                  # the device-resident copy follows the codes

    def forward(self, x: np.ndarray) -> np.ndarray:
        from . import quant
        x = _as_f32(x, self.device)
        self._cache_input = x
        # Optimisers update weight.data in place (novann/optim/sgd.py:62-82) and say nothing, so
        # in training mode the codes are refreshed on every forward; in evaluation mode the
        # codes of the last refresh are reused.
        if self._training or self._codes is None:
            self.requantize()
        xb = quant.cast(x, "bf16", device=self.device)
        b = None if self.bias is None else self.bias.data.reshape(-1)
        if self._training:
            yb = F.linear_q_host(xb, self._codes, self._scales, b, self.fmt, self.device)
        else:
            # evaluation: codes, scales and bias stay on the device and the expanded weight is
            # made once per requantize() instead of once per forward
            if self._resident is None:
                self._resident = F.LinearWeightCache(self._codes, self._scales, b, self.fmt, self.device)
            yb = self._resident.forward_host(xb)
        return quant.cast(yb, "f32", src_dtype="bf16", device=self.device)

    def backward(self, grad: np.ndarray) -> np.ndarray:
        if not (self.tensor_core_backward and self.fmt in ("e4m3", "e5m2")):
            return super().backward(grad)
        grad = _as_f32(grad, self.device)
        dw, db, dx = F.linear_q_bwd_host(grad, self._cache_input, self._codes, self._scales, self.fmt,
                                         self.bias is not None, self.device)
        self.weight.grad = dw
        if self.bias is not None:
            self.bias.grad = db
        return dx


class Conv2d(Layer):
    """2-D convolution in fp32 on the GPU: im2col + GEMM forward, GEMMs + col2im gather backward
    (the reference's layouts and gradient rules)."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0,
                 bias: bool = True, padding_mode: str = "zeros", init=None, device: int = 0):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.KH, self.KW = _pair(kernel_size)
        self.sh, self.sw = _pair(stride if stride is not None else kernel_size)
        self.ph, self.pw = _pair(padding)
        self.pm = padding_mode
        self.init_fn = init
        self.use_bias = bias
        self.device = device
        self.weight = self.bias = None
        self._cache = {}
        self.reset_parameters()

    def reset_parameters(self, initializer=None):
        init = initializer or self.init_fn or kaiming_uniform_relu
        w = init((self.out_channels, self.in_channels, self.KH, self.KW))
        self.weight = Parameters(np.asarray(w, dtype=np.float32))
        self.weight.name = "conv2d weight"
        if self.use_bias:
            self.bias = Parameters(np.zeros((self.out_channels, 1), dtype=np.float32))
            self.bias.name = "conv2d bias"
        else:
            self.bias = None

    def forward(self, x: np.ndarray) -> np.ndarray:
        x = _as_f32(x, self.device)
        out, col = F.conv2d_f32_host(x, self.weight.data, None if self.bias is None else self.bias.data,
                                     (self.sh, self.sw), (self.ph, self.pw), self.pm, self.device,
                                     return_col=True)
        self._cache = {"x_shape": x.shape, "col": col,
                       "w_col": self.weight.data.reshape(self.out_channels, -1)}
        return out

    def backward(self, grad: np.ndarray) -> np.ndarray:
        grad = _as_f32(grad, self.device)
        dw, db, dx = F.conv2d_bwd_f32_host(grad, self._cache["col"], self.weight.data,
                                           self._cache["x_shape"], (self.sh, self.sw),
                                           (self.ph, self.pw), self.bias is not None, self.device)
        self.weight.grad = dw
        if self.bias is not None:
            self.bias.grad = db
        return dx

    def parameters(self):
        return [self.weight] + ([self.bias] if self.bias is not None else [])

    def __repr__(self):
        return (f"Conv2d(in_channels={self.in_channels}, out_channels={self.out_channels}, "
                f"kernel_size={(self.KH, self.KW)}, stride={(self.sh, self.sw)}, "
                f"padding={(self.ph, self.pw)}, bias={self.use_bias})")


class QuantConv2d(Conv2d):
    """Conv2d whose im2col contraction runs on the tensor cores with FP8 weight codes."""

    def __init__(self, *args, fmt: str = "e4m3", **kwargs):
        self.fmt = fmt
        self._codes = self._scales = None
        super().__init__(*args, **kwargs)

    def reset_parameters(self, initializer=None):
        super().reset_parameters(initializer)
        self._codes = self._scales = None      # quantised on the next forward

    def requantize(self) -> None:
        from . import quant
        w_col = self.weight.data.reshape(self.out_channels, -1)
        q = 32 if self.fmt == "e2m1_b32" else 16
        kpad = (w_col.shape[1] + q - 1) // q * q
        padded = np.zeros((self.out_channels, kpad), np.float32)
        padded[:, :w_col.shape[1]] = w_col
        self._codes, self._scales = quant.quantize_weight(padded, self.fmt, self.device)

    def forward(self, x: np.ndarray) -> np.ndarray:
        x = _as_f32(x, self.device)
        if self._training or self._codes is None:     # see QuantLinear.forward
            self.requantize()
        # backward uses the fp32 master weight (straight-through), so it needs the fp32 patches
        self._cache = {"x_shape": x.shape, "col": F.im2col_f32_host(
            x, (self.KH, self.KW), (self.sh, self.sw), (self.ph, self.pw), self.pm, self.device)}
        b = None if self.bias is None else self.bias.data.reshape(-1)
        return F.conv2d_q_host(x, self._codes, self._scales, b, (self.KH, self.KW), (self.sh, self.sw),
                               (self.ph, self.pw), self.pm, self.fmt, self.device)


class _BatchNorm(Layer):
    """Shared body of ``BatchNorm1d`` / ``BatchNorm2d``.  As in the reference, gamma, beta and the
    running statistics are float64 arrays.  The reference's forward therefore returns float64,
    which every consumer narrows with ``astype(np.float32)``; here the narrowed fp32 value is
    returned directly (and likewise for the input gradient)."""

    _param_shape = None     # set by subclasses: shape of gamma / beta for a given C

    def __init__(self, num_features: int, momentum: float = 0.1, eps: float = 1e-5, device: int = 0):
        super().__init__()
        self.num_features = int(num_features)
        self.momentum, self.eps = float(momentum), float(eps)
        self.device = device
        shp = self._shape()
        self.gamma = Parameters(np.ones(shp))
        self.beta = Parameters(np.zeros(shp))
        self.gamma.name, self.beta.name = "gamma", "beta"
        self.running_mean = np.zeros(shp)
        self.running_var = np.ones(shp)
        self._x = self._stats = None

    def _check(self, x):
        raise NotImplementedError

    def forward(self, x: np.ndarray) -> np.ndarray:
        x = _as_f32(x, self.device)
        self._check(x)
        y, rm, rv, stats = F.batchnorm_fwd_host(x, self.gamma.data, self.beta.data, self.running_mean,
                                                self.running_var, self.momentum, self.eps,
                                                self._training, self.device)
        if self._training:
            self._x, self._stats = x, stats
            self.running_mean = rm.reshape(self.running_mean.shape)
            self.running_var = rv.reshape(self.running_var.shape)
        return y

    def backward(self, grad: np.ndarray) -> np.ndarray:
        if self._x is None or self._stats is None:
            raise ValueError("Backward called before forward pass or cache cleared")
        dx, dg, db = F.batchnorm_bwd_host(grad, self._x, self._stats, self.gamma.data, self.eps, self.device)
        self.gamma.grad = dg.reshape(self.gamma.data.shape)
        self.beta.grad = db.reshape(self.beta.data.shape)
        return dx

    def parameters(self):
        return [self.gamma, self.beta]

    def __repr__(self):
        return f"{type(self).__name__}(num_features={self.num_features}, momentum={self.momentum}, eps={self.eps})"


class BatchNorm2d(_BatchNorm):
    """``novann/layers/batchnorm/batchnorm2d.py``: per-channel statistics over (N, H, W);
    parameters shaped (1, C, 1, 1)."""

    def _shape(self):
        return (1, self.num_features, 1, 1)

    def _check(self, x):
        if x.ndim != 4 or x.shape[1] != self.num_features:
            raise ValueError(f"BatchNorm2d expects (N, {self.num_features}, H, W) input, got {x.shape}")


class BatchNorm1d(_BatchNorm):
    """``novann/layers/batchnorm/batchnorm1d.py``: statistics over the batch for (N, C) input, over
    batch and length for (N, C, L) input (gamma / beta are then reshaped to (1, C, 1), as the
    reference does)."""

    def _shape(self):
        return (1, self.num_features)

    def _check(self, x):
        if x.ndim not in (2, 3):
            raise ValueError(f"BatchNorm1d expects 2D or 3D input, got {x.ndim}D")
        if x.shape[1] != self.num_features:
            raise ValueError(f"BatchNorm1d expects {self.num_features} features, got {x.shape[1]}")
        if x.ndim == 3:
            self.gamma.data = self.gamma.data.reshape(1, self.num_features, 1)
            self.beta.data = self.beta.data.reshape(1, self.num_features, 1)


class MaxPool2d(Layer):
    """``novann/layers/pooling/maxpool/maxpool2d.py``: windows over the padded input; ties share
    the gradient evenly."""

    def __init__(self, kernel_size, stride=None, padding=0, padding_mode: str = "zeros", device: int = 0):
        super().__init__()
        self.KH, self.KW = _pair(kernel_size)
        self.sh, self.sw = _pair(stride if stride is not None else kernel_size)
        self.ph, self.pw = _pair(padding)
        self.pm = padding_mode
        self.device = device
        self._x = None

    def forward(self, x: np.ndarray) -> np.ndarray:
        x = _as_f32(x, self.device)
        self._x = x
        return F.max_pool2d_host(x, (self.KH, self.KW), (self.sh, self.sw), (self.ph, self.pw), self.pm,
                                 self.device)

    def backward(self, grad_output: np.ndarray) -> np.ndarray:
        grad_output = _as_f32(grad_output, self.device)
        dx = F.max_pool2d_bwd_host(grad_output, self._x, (self.KH, self.KW), (self.sh, self.sw),
                                   (self.ph, self.pw), self.pm, self.device)
        self._x = None
        return dx

    def __repr__(self):
        return f"MaxPool2d(kernel_size={(self.KH, self.KW)}, stride={(self.sh, self.sw)}, padding={(self.ph, self.pw)})"


class GlobalAvgPool2d(Layer):
    """``novann/layers/pooling/gap/gap2d.py``: (N, C, H, W) -> (N, C, 1, 1)."""

    def __init__(self, device: int = 0):
        super().__init__()
        self.device = device
        self._x_shape = None

    def forward(self, x: np.ndarray) -> np.ndarray:
        x = _as_f32(x, self.device)
        self._x_shape = x.shape
        return F.avg_pool2d_host(x, self.device)

    def backward(self, grad_output: np.ndarray) -> np.ndarray:
        return F.avg_pool2d_bwd_host(_as_f32(grad_output, self.device), self._x_shape, self.device)

    def __repr__(self):
        return "GlobalAvgPool2d()"


class Flatten(Layer):
    """``novann/layers/flatten/flatten.py``: a reshape; nothing to compute."""

    def __init__(self):
        super().__init__()
        self._origin_shape = None

    def forward(self, x: np.ndarray) -> np.ndarray:
        self._origin_shape = x.shape
        return x.reshape(x.shape[0], -1)

    def backward(self, grad: np.ndarray) -> np.ndarray:
        return grad.reshape(*self._origin_shape)

    def __repr__(self):
        return "Flatten()"


class Dropout(Layer):
    """``novann/layers/regularization/dropout.py``: the keep mask is drawn on the host from
    NumPy's global generator with the reference's own call (so a seeded run drops the same
    units); the masking and scaling run on the GPU."""

    def __init__(self, p: float, device: int = 0) -> None:
        super().__init__()
        if not (0.0 < p < 1.0):
            raise ValueError("Dropout probability must be in the interval [0.0, 1.0).")
        self.p = p
        self.device = device
        self._mask = None

    def train(self) -> None:
        super().train()
        self._mask = None

    def eval(self) -> None:
        super().eval()
        self._mask = None

    def forward(self, x: np.ndarray) -> np.ndarray:
        if not self._training or self.p == 0.0:
            return x
        keep = 1.0 - self.p
        self._mask = (np.random.rand(*x.shape) < keep).astype(np.float32)
        return F.dropout_host(x, self._mask, keep, self.device)

    def backward(self, grad: np.ndarray) -> np.ndarray:
        if not self._training:
            return grad
        out = F.dropout_host(grad, self._mask, 1.0 - self.p, self.device)
        self._mask = None
        return out

    def __repr__(self):
        return f"Dropout(p={self.p})"
