"""Device-resident training step of an MLP: the reference's loop body
(``novann/utils/train/train.py:60-75``: zero_grad, forward, CrossEntropyLoss, backward,
SGD.step) for ``Sequential(Linear, ReLU, ..., Linear)`` with every tensor kept in HBM.

Weights, activations, masks and gradients live in one device arena; a step is a fixed
sequence of kernel launches on one stream (fused Linear+bias+ReLU forward, softmax-CE,
Linear backward with the bias gradient as a by-product of the weight-gradient GEMM and the ReLU
mask folded into dX, SGD over the flat parameter bucket).
With more than one rank the flat gradient bucket is summed over ranks with one NCCL
all-reduce and scaled by 1/world inside the SGD kernel, which equals the gradient of the
global batch because the reference divides its loss gradient by the local batch size.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib
from .device import DeviceBuffer, Event, Stream, _sptr


def shard_rows(n_rows: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous row range [lo, hi) of ``rank`` when ``n_rows`` rows are split evenly."""
    if n_rows % world:
        raise ValueError(f"{n_rows} rows do not split evenly over {world} ranks")
    per = n_rows // world
    return rank * per, (rank + 1) * per


def flatten_params(params) -> np.ndarray:
    """[W0, b0, W1, b1, ...] -> one flat fp32 bucket (layer order, weight then bias)."""
    return np.concatenate([np.ascontiguousarray(p, np.float32).ravel() for p in params])


def unflatten_params(flat: np.ndarray, dims) -> list[np.ndarray]:
    out, off = [], 0
    for fi, fo in zip(dims[:-1], dims[1:]):
        out.append(flat[off:off + fo * fi].reshape(fo, fi).copy())
        off += fo * fi
        out.append(flat[off:off + fo].reshape(1, fo).copy())
        off += fo
    return out


class Communicator:
    """NCCL communicator of the library (one process per GPU)."""

    def __init__(self, unique_id: bytes, rank: int, world: int, device: int):
        self.rank, self.world, self.device = rank, world, device
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        h = C.c_void_p()
        check(lib().nvq_comm_init(buf, rank, world, device, C.byref(h)))
        self.handle = h.value

    @staticmethod
    def make_unique_id() -> bytes:
        buf = (C.c_uint8 * 128)()
        check(lib().nvq_comm_unique_id(buf))
        return bytes(buf)

    def allreduce_sum(self, buf: DeviceBuffer, n: int, stream=None, offset: int = 0) -> None:
        check(lib().nvq_allreduce_sum_f32(C.c_void_p(self.handle), buf.at(offset), n, self.device,
                                          _sptr(stream)))

    def wait(self, stream, timeout_ms: int = 30000) -> None:
        """Host-side watchdog around the collective: returns when ``stream`` has drained; raises
        ``NvqError`` (``ERR_TIMEOUT`` / ``ERR_NCCL``) when the all-reduce is still pending after
        ``timeout_ms`` or NCCL reported an asynchronous error.  The wait polls; it never blocks
        inside the driver, so a peer that never joined cannot hold this thread.  After a
        failure call ``abort()``."""
        check(lib().nvq_comm_wait(C.c_void_p(self.handle), self.device, _sptr(stream), int(timeout_ms)))

    def abort(self) -> None:
        """``ncclCommAbort``: tear the communicator down without waiting for what is in flight."""
        if self.handle:
            lib().nvq_comm_abort(C.c_void_p(self.handle))
            self.handle = None

    def close(self) -> None:
        if self.handle:
            lib().nvq_comm_destroy(C.c_void_p(self.handle))
            self.handle = None


class _DeviceView:
    """Device memory owned by someone else, with ``DeviceBuffer``'s addressing."""

    def __init__(self, ptr: int, nbytes: int, device: int):
        self.ptr, self.nbytes, self.device = ptr, nbytes, device

    def at(self, offset: int) -> C.c_void_p:
        return C.c_void_p(self.ptr + offset)

    def to_numpy(self, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype)
        check(lib().nvq_memcpy_d2h(out.ctypes.data_as(C.c_void_p), C.c_void_p(self.ptr), out.nbytes,
                                   self.device, None))
        check(lib().nvq_device_sync(self.device))
        return out


class PeerGroup:
    """Gradient all-reduce fused with the SGD update over NVLink peer memory (``nvq_peer_*``):
    one kernel per step and rank instead of an NCCL all-reduce plus the SGD kernel.

    ``allgather(payload) -> [payload of rank 0, 1, ...]`` is the launcher's side channel for the
    64-byte IPC handles (``launch.allgather_bytes`` over a shared directory, or a
    ``torch.distributed`` gather).  ``absent`` lists ranks that are never connected - their
    announcement never comes, so the step gives up after ``timeout_ms`` with an error flag;
    tests use it to make the bounded wait run out on one GPU."""

    def __init__(self, rank: int, world: int, n_floats: int, device: int, allgather=None,
                 timeout_ms: int = 2000, absent=()):
        self.rank, self.world, self.device, self.n = rank, world, device, int(n_floats)
        self._allgather = allgather
        h = C.c_void_p()
        check(lib().nvq_peer_create(C.byref(h), rank, world, self.n, int(timeout_ms), device))
        self.handle = h.value
        hb = C.c_size_t()
        check(lib().nvq_peer_handle_bytes(C.byref(hb)))
        mine = (C.c_uint8 * hb.value)()
        check(lib().nvq_peer_export(C.c_void_p(self.handle), mine))
        if world > 1:
            if allgather is not None:
                blobs = allgather(bytes(mine))
            else:
                blobs = [bytes(mine) if r == rank else bytes(hb.value) for r in range(world)]
            blobs = [bytes(hb.value) if r in absent else b for r, b in enumerate(blobs)]
            allh = (C.c_uint8 * (hb.value * world)).from_buffer_copy(b"".join(blobs))
            check(lib().nvq_peer_connect(C.c_void_p(self.handle), allh))
        self.calls = 0
        self.grad_views = []
        for parity in (0, 1):
            p = C.c_void_p()
            check(lib().nvq_peer_grad_buffer(C.c_void_p(self.handle), parity, C.byref(p)))
            self.grad_views.append(_DeviceView(p.value, self.n * 4, device))

    def grads(self) -> _DeviceView:
        """Where the backward pass of the NEXT step writes this rank's gradients."""
        return self.grad_views[self.calls & 1]

    def allreduce_sgd(self, d_params: DeviceBuffer, lr: float, stream=None, parity: int | None = None) -> None:
        """Enqueue the fused all-reduce / update of the next step.  With ``parity`` given the
        launch is only recorded (CUDA graph capture of the step that reads that buffer) and
        ``advance()`` is called by whoever replays it."""
        check(lib().nvq_peer_allreduce_sgd(C.c_void_p(self.handle),
                                           self.calls & 1 if parity is None else parity,
                                           d_params.at(0), C.c_float(lr), _sptr(stream)))
        if parity is None:
            self.calls += 1

    def advance(self) -> None:
        self.calls += 1

    def close(self) -> None:
        """Host rendezvous (a peer may still be reading this rank's buffers until its own last
        step has completed and it has synchronised), then unmap and free."""
        if self.handle:
            if self._allgather is not None and self.world > 1:
                self._allgather(b"closing")
            lib().nvq_peer_destroy(C.c_void_p(self.handle))
            self.handle = None


class MLPTrainStep:
    """``step(x, labels)`` runs one training step on the device and returns nothing; read
    results with ``logits()``, ``loss()``, ``grads()``, ``params()``.  Data parallel: ``comm=``
    (NCCL all-reduce, then the SGD kernel) or ``peer=`` (``PeerGroup``: all-reduce and update in
    one kernel over NVLink peer memory)."""

    def __init__(self, params, batch: int, lr: float, device: int = 0, comm: Communicator | None = None,
                 gate=None, collective_timeout_ms: int = 30000, peer: PeerGroup | None = None):
        self.dims = [params[0].shape[1]] + [params[2 * i].shape[0] for i in range(len(params) // 2)]
        self.nl = len(self.dims) - 1
        self.batch, self.lr, self.device, self.comm = batch, float(lr), device, comm
        self.gate = gate            # launch.StepGate: host rendezvous before each collective step
        self.collective_timeout_ms = collective_timeout_ms
        self._step_no = 0
        self.stream = Stream(device)
        self.side = Stream(device)          # weight-gradient GEMMs, beside the dX chain
        self.side2 = Stream(device)         # the loss value, beside both
        flat = flatten_params(params)
        self.n_params = flat.size
        self.d_params = DeviceBuffer.from_numpy(flat, device)
        self.peer = peer
        if peer is not None and comm is not None:
            raise ValueError("comm= and peer= are alternatives")
        if peer is not None and peer.n != flat.size:
            raise ValueError("the peer group was made for another parameter count")
        self.d_grads = DeviceBuffer(flat.nbytes, device) if peer is None else peer.grads()
        self.w_off, self.b_off, off = [], [], 0
        for fi, fo in zip(self.dims[:-1], self.dims[1:]):
            self.w_off.append(off * 4)
            off += fo * fi
            self.b_off.append(off * 4)
            off += fo
        f4 = 4 * batch
        self.d_x = DeviceBuffer(f4 * self.dims[0], device)
        self.d_labels = DeviceBuffer(4 * batch, device)
        self.d_act = [self.d_x] + [DeviceBuffer(f4 * d, device) for d in self.dims[1:]]
        self.d_mask = [DeviceBuffer(f4 * d, device) for d in self.dims[1:-1]]
        self.d_g = [DeviceBuffer(f4 * d, device) for d in self.dims]     # gradient w.r.t. each activation
        self.d_yhat = DeviceBuffer(f4 * self.dims[-1], device)
        self.d_loss = DeviceBuffer(4, device)
        self.ev_fork = [Event(device) for _ in range(self.nl)]
        self.ev_join = Event(device)
        self.ev_loss = Event(device)
        self.ev_loss_done = Event(device)
        self._graph = None
        self._graph_is_partial = False
        self._peer_graphs = [None, None]    # forward / loss / backward into gradient buffer 0 / 1

    def upload(self, x: np.ndarray, labels: np.ndarray) -> None:
        self.d_x.upload(np.ascontiguousarray(x, np.float32), stream=self.stream)
        self.d_labels.upload(np.ascontiguousarray(labels, np.int32), stream=self.stream)

    def launch(self) -> None:
        """Enqueue one step on ``self.stream`` (inputs already uploaded)."""
        self.launch_compute()
        self.launch_update()

    def launch_compute(self, grads=None) -> None:
        """Forward, loss and backward: the gradients of this rank's rows land in ``d_grads``
        (with a peer group: in the buffer the next fused update reads, or in ``grads``)."""
        L, dev, st, B = lib(), self.device, _sptr(self.stream), self.batch
        if grads is not None:
            self.d_grads = grads
        elif self.peer is not None:
            self.d_grads = self.peer.grads()
        for i in range(self.nl):
            last = i == self.nl - 1
            check(L.nvq_linear_fwd_f32(self.d_act[i + 1].at(0), self.d_act[i].at(0),
                                       self.d_params.at(self.w_off[i]), self.d_params.at(self.b_off[i]),
                                       B, self.dims[i + 1], self.dims[i], 0 if last else 1,
                                       None if last else self.d_mask[i].at(0), dev, st))
        # the gradient of the loss on the step's stream; the loss VALUE (the reference's double
        # softmax), which nothing downstream reads, beside the backward pass on the side stream
        check(L.nvq_softmax_ce_f32(self.d_g[self.nl].at(0), None, self.d_act[self.nl].at(0),
                                   self.d_labels.at(0), self.d_yhat.at(0), B, self.dims[-1], dev, st))
        self.ev_loss.record(self.stream)
        self.ev_loss.block(self.side2)
        check(L.nvq_ce_loss_f32(self.d_loss.at(0), self.d_yhat.at(0), self.d_labels.at(0), B, self.dims[-1],
                                dev, _sptr(self.side2)))
        self.ev_loss_done.record(self.side2)
        # Backward: the chain loss -> dX(nl-1) -> ... -> dX(1) runs on the step's stream; every
        # weight gradient (with its bias gradient) depends on one link of that chain only and runs
        # on a side stream, joined before the update - in a CUDA graph these are parallel branches.
        side = _sptr(self.side)
        for i in reversed(range(self.nl)):
            self.ev_fork[i].record(self.stream)          # d_g[i + 1] is complete
            self.ev_fork[i].block(self.side)
            check(L.nvq_linear_bwd_f32(self.d_grads.at(self.w_off[i]), self.d_grads.at(self.b_off[i]),
                                       None, self.d_g[i + 1].at(0), self.d_act[i].at(0), None, None,
                                       B, self.dims[i + 1], self.dims[i], dev, side))
            if i > 0:
                check(L.nvq_linear_bwd_f32(None, None, self.d_g[i].at(0), self.d_g[i + 1].at(0),
                                           None, self.d_params.at(self.w_off[i]), self.d_mask[i - 1].at(0),
                                           B, self.dims[i + 1], self.dims[i], dev, st))
        self.ev_join.record(self.side)
        self.ev_join.block(self.stream)
        self.ev_loss_done.block(self.stream)

    def launch_update(self) -> None:
        """The gradient all-reduce (data parallel) and the SGD update."""
        L, dev, st = lib(), self.device, _sptr(self.stream)
        if self.peer is not None:
            self.peer.allreduce_sgd(self.d_params, self.lr, stream=self.stream)
            return
        scale = 1.0
        if self.comm is not None and self.comm.world > 1:
            self.comm.allreduce_sum(self.d_grads, self.n_params, stream=self.stream)
            scale = 1.0 / self.comm.world
        check(L.nvq_sgd_step_f32(self.d_params.at(0), self.d_grads.at(0), self.n_params,
                                 C.c_float(self.lr), C.c_float(scale), dev, st))

    def capture(self) -> None:
        """Record the step's launch sequence into a CUDA graph (after one eager step has run,
        so that first-call set-up is done).  ``replay()`` then issues the whole step as one
        graph launch; the buffers it reads and writes are the same ones ``upload`` fills.
        With a communicator of more than one rank the graph holds forward, loss and backward
        only: the NCCL all-reduce is never captured (it is enqueued after the graph, followed by
        the SGD kernel), so a step costs three host calls instead of eleven."""
        if self._graph is not None:
            return
        if self.peer is not None:
            # the gradients alternate between the peer group's two buffers: one graph per buffer
            for parity in (0, 1):
                check(lib().nvq_graph_begin_capture(self.device, _sptr(self.stream)))
                try:
                    self.launch_compute(grads=self.peer.grad_views[parity])
                    self.peer.allreduce_sgd(self.d_params, self.lr, stream=self.stream, parity=parity)
                finally:
                    h = C.c_void_p()
                    check(lib().nvq_graph_end_capture(self.device, _sptr(self.stream), C.byref(h)))
                self._peer_graphs[parity] = h.value
            self._graph = self._peer_graphs[0]
            self._graph_is_partial = False     # the fused all-reduce / update is the library's own kernel
            self.launches_per_step = self.kernels_per_step()
            return
        self._graph_is_partial = self.comm is not None and self.comm.world > 1
        check(lib().nvq_graph_begin_capture(self.device, _sptr(self.stream)))
        try:
            if self._graph_is_partial:
                self.launch_compute()
            else:
                self.launch()
        finally:
            h = C.c_void_p()
            check(lib().nvq_graph_end_capture(self.device, _sptr(self.stream), C.byref(h)))
        self._graph = h.value
        self.launches_per_step = self.kernels_per_step()

    def replay(self) -> None:
        graph = self._graph
        if self.peer is not None:
            graph = self._peer_graphs[self.peer.calls & 1]
            self.d_grads = self.peer.grads()
        check(lib().nvq_graph_launch(self.device, C.c_void_p(graph), _sptr(self.stream)))
        if self.peer is not None:
            self.peer.advance()
        if self._graph_is_partial:
            self.launch_update()

    def kernels_per_step(self) -> int:
        """Kernel launches of this library in one step: nl forward, 1 loss, per layer one GEMM for
        dW with db as its by-product (+ one for dX except for the first layer), 1 SGD."""
        return self.nl + 1 + (2 * self.nl - 1) + 1

    def step(self, x: np.ndarray, labels: np.ndarray) -> None:
        if self.gate is not None:
            self.gate.enter(self._step_no + 1)  # raises PeerLost before anything is launched
        self._step_no += 1
        self.upload(x, labels)
        if self._graph is not None:
            self.replay()
        else:
            self.launch()
        self.sync()

    def sync(self) -> None:
        """Waits for the step on the host; with a communicator the wait is the NCCL watchdog
        (bounded, polls the communicator's asynchronous error state)."""
        if self.comm is not None and self.comm.world > 1:
            self.comm.wait(self.stream, self.collective_timeout_ms)
        else:
            self.stream.sync()
        if self.peer is not None:
            # a rank that never announced the step: the kernel gave up, the parameters are untouched
            from .functional import check_device_errors
            check_device_errors(self.device)

    # ---- results
    def logits(self) -> np.ndarray:
        return self.d_act[self.nl].to_numpy(np.float32, (self.batch, self.dims[-1]))

    def loss(self) -> np.float32:
        return self.d_loss.to_numpy(np.float32, (1,))[0]

    def grads(self) -> list[np.ndarray]:
        return unflatten_params(self.d_grads.to_numpy(np.float32, (self.n_params,)), self.dims)

    def params(self) -> list[np.ndarray]:
        return unflatten_params(self.d_params.to_numpy(np.float32, (self.n_params,)), self.dims)


class QuantMLPInference:
    """Forward pass of ``Sequential(Linear, ReLU, ..., Linear)`` with FP8 weights, resident on the
    device: weights are quantised per output channel and expanded once at construction; a call
    uploads the fp32 batch, casts it to bf16, runs one tensor-core kernel per layer with bias and
    ReLU fused into the epilogue (activations stay bf16 in HBM between layers), casts the logits
    back to fp32 and downloads them."""

    def __init__(self, params, max_batch: int, fmt: str = "e4m3", device: int = 0):
        from . import functional as F, quant
        self.F, self.quant = F, quant
        self.device, self.fmt, self.max_batch = device, fmt, max_batch
        self.dims = [params[0].shape[1]] + [params[2 * i].shape[0] for i in range(len(params) // 2)]
        self.stream = Stream(device)
        self.wd, self.scales, self.bias = [], [], []
        for i in range(len(params) // 2):
            w = np.ascontiguousarray(params[2 * i], np.float32)
            n, k = w.shape
            codes, sc = quant.quantize_weight(w, fmt, device)
            dq = DeviceBuffer.from_numpy(codes, device)
            wd = DeviceBuffer(n * k * 2, device)
            F.linear_expand_weight_device(wd, dq, fmt, None, n, k)
            self.wd.append(wd)
            self.scales.append(DeviceBuffer.from_numpy(sc, device))
            self.bias.append(DeviceBuffer.from_numpy(np.ascontiguousarray(params[2 * i + 1], np.float32).ravel(), device))
        self.d_x32 = DeviceBuffer(max_batch * self.dims[0] * 4, device)
        self.d_act = [DeviceBuffer(max_batch * d * 2, device) for d in self.dims]
        self.d_out32 = DeviceBuffer(max_batch * self.dims[-1] * 4, device)

    def forward(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        m = x.shape[0]
        if m > self.max_batch:
            raise ValueError("batch larger than max_batch")
        st = self.stream
        self.d_x32.upload(x, stream=st)
        self.quant.cast_device(self.d_act[0], "bf16", self.d_x32, "f32", m * self.dims[0], stream=st)
        nl = len(self.wd)
        for i in range(nl):
            self.F.linear_expanded_device(self.d_act[i + 1], self.d_act[i], self.wd[i], self.scales[i],
                                          self.bias[i], m, self.dims[i + 1], self.dims[i], stream=st,
                                          relu=i < nl - 1)
        self.quant.cast_device(self.d_out32, "f32", self.d_act[nl], "bf16", m * self.dims[-1], stream=st)
        out = np.empty((m, self.dims[-1]), np.float32)
        self.d_out32.download(out, stream=st)
        st.sync()
        self.F.check_device_errors(self.device)
        return out


class QuantConvChain:
    """A stack of quantised 3x3-style convolutions (optionally each followed by ReLU) whose
    activations stay in HBM as bf16 NHWC from the first layer to the last: one layout conversion
    at each end of the chain, none between layers (``nvq_conv2d_fwd_q_nhwc``).  The weights are
    quantised once at construction; ``forward`` takes and returns fp32 NCHW host arrays like
    ``F.conv2d`` (novann/functional.py:275-385), ``forward_device`` works on resident buffers.

    ``layers``: list of dicts with ``weight`` (Cout, C, KH, KW) fp32, ``bias`` (Cout,) or None,
    ``stride``, ``padding`` (pairs) and ``relu`` (bool).  Shape rules of the entry point apply
    (strides 1 or 2, C % 64 == 0, Cout % 8 == 0, zero padding)."""

    def __init__(self, layers, input_shape, fmt: str = "e4m3", device: int = 0):
        from . import functional as F, quant
        self.F, self.device, self.fmt = F, device, fmt
        self.stream = Stream(device)
        n, c, h, w = input_shape
        self.shapes = [(n, c, h, w)]
        self.layers = []
        for spec in layers:
            wt = np.ascontiguousarray(spec["weight"], np.float32)
            cout, cin, kh, kw = wt.shape
            if cin != c:
                raise ValueError(f"layer expects {cin} input channels, got {c}")
            sh, sw = spec.get("stride", (1, 1))
            ph, pw = spec.get("padding", (0, 0))
            w_col = wt.reshape(cout, -1)
            q = 32 if fmt == "e2m1_b32" else 16
            kpad = (w_col.shape[1] + q - 1) // q * q
            padded = np.zeros((cout, kpad), np.float32)
            padded[:, :w_col.shape[1]] = w_col
            codes, scales = quant.quantize_weight(padded, fmt, device)
            oh, ow = F.conv2d_out_size(h, w, kh, kw, sh, sw, ph, pw)
            b = spec.get("bias")
            self.layers.append(dict(
                codes=DeviceBuffer.from_numpy(codes, device), scales=DeviceBuffer.from_numpy(scales, device),
                bias=None if b is None else DeviceBuffer.from_numpy(np.ascontiguousarray(b, np.float32).ravel(), device),
                ws=DeviceBuffer(cout * cin * kh * kw * 2, device), geom=(n, c, h, w, cout, (kh, kw), (sh, sw), (ph, pw)),
                relu=bool(spec.get("relu", False))))
            c, h, w = cout, oh, ow
            self.shapes.append((n, c, h, w))
        self.act = [DeviceBuffer(int(np.prod(s)) * 2, device) for s in self.shapes]
        self.d_in32 = DeviceBuffer(int(np.prod(self.shapes[0])) * 4, device)
        self.d_out32 = DeviceBuffer(int(np.prod(self.shapes[-1])) * 4, device)

    def forward_device(self) -> None:
        """act[0] (bf16 NHWC) -> act[-1] (bf16 NHWC), one kernel pair per layer on ``self.stream``."""
        for i, L in enumerate(self.layers):
            n, c, h, w, cout, k, s, p = L["geom"]
            self.F.conv2d_q_nhwc_device(self.act[i + 1], self.act[i], L["codes"], self.fmt, L["scales"], L["bias"],
                                        L["ws"], n, c, h, w, cout, k, s, p, relu=L["relu"], stream=self.stream)

    def forward(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        if x.shape != self.shapes[0]:
            raise ValueError(f"expected input {self.shapes[0]}, got {x.shape}")
        n, c, h, w = self.shapes[0]
        self.d_in32.upload(x, stream=self.stream)
        self.F.nchw_f32_to_nhwc_bf16_device(self.act[0], self.d_in32, n, c, h * w, stream=self.stream)
        self.forward_device()
        n, c, h, w = self.shapes[-1]
        self.F.nhwc_bf16_to_nchw_f32_device(self.d_out32, self.act[-1], n, c, h * w, stream=self.stream)
        out = np.empty(self.shapes[-1], np.float32)
        self.d_out32.download(out, stream=self.stream)
        self.stream.sync()
        self.F.check_device_errors(self.device)
        return out
