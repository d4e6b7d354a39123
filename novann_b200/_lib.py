"""ctypes binding of ``libnvq.so`` (the C ABI declared in ``include/nvq.h``).

There is no fallback of any kind: if the library is missing, or a call fails, an
exception is raised.  ``lib()`` loads lazily so that the package can be imported on
a machine without a GPU (the library itself loads there too; only calls fail).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("NVQ_LIB", os.path.join(_HERE, "libnvq.so"))

# dtype ids of nvq_dtype
F32, F16, BF16, E4M3, E5M2, E2M1_B32, F64 = 0, 1, 2, 3, 4, 5, 6
DTYPE_IDS = {"f32": F32, "f16": F16, "bf16": BF16, "e4m3": E4M3, "e5m2": E5M2, "e2m1_b32": E2M1_B32,
             "f64": F64}
DTYPE_SIZE = {F32: 4, F16: 2, BF16: 2, E4M3: 1, E5M2: 1, F64: 8}
# path selectors of nvq_linear_fwd_opts / nvq_conv2d_fwd_q_opts
LINEAR_AUTO, LINEAR_BF16_ACTIVATIONS, LINEAR_EXPAND_IN_KERNEL, LINEAR_SINGLE_CTA, LINEAR_CTA_PAIR = 0, 1, 2, 4, 8
LINEAR_CLUSTER_REDUCE = 16
LINEAR_CODES_FINITE = 32
CONV_AUTO, CONV_PATCH_MATRIX, CONV_CTA_PAIR = 0, 1, 2
PAD_MODES = {"zeros": 0, "reflect": 1, "replicate": 2, "circular": 3}

OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_TIMEOUT, ERR_NCCL = 0, -1, -2, -3, -4, -5

vp, sz, i32, f32c, u64 = C.c_void_p, C.c_size_t, C.c_int, C.c_float, C.c_uint64
f64c = C.c_double
pvp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes).  Every symbol declared in include/nvq.h is listed here;
# tests/test_abi.py checks the two against each other and against the built library.
SIGNATURES = {
    "nvq_last_error": (C.c_char_p, []),
    "nvq_version": (C.c_char_p, []),
    "nvq_device_count": (i32, [C.POINTER(i32)]),
    "nvq_device_info": (i32, [i32, C.POINTER(i32), C.POINTER(sz), C.POINTER(i32), C.POINTER(i32)]),
    "nvq_shutdown": (i32, []),
    "nvq_malloc": (i32, [i32, sz, pvp]),
    "nvq_free": (i32, [i32, vp]),
    "nvq_host_alloc": (i32, [sz, pvp]),
    "nvq_host_free": (i32, [vp]),
    "nvq_memcpy_h2d": (i32, [vp, vp, sz, i32, vp]),
    "nvq_memcpy_d2h": (i32, [vp, vp, sz, i32, vp]),
    "nvq_memcpy_d2d": (i32, [vp, vp, sz, i32, vp]),
    "nvq_memset": (i32, [vp, i32, sz, i32, vp]),
    "nvq_stream_create": (i32, [i32, pvp]),
    "nvq_stream_destroy": (i32, [i32, vp]),
    "nvq_stream_sync": (i32, [i32, vp]),
    "nvq_device_sync": (i32, [i32]),
    "nvq_event_create": (i32, [i32, pvp]),
    "nvq_event_destroy": (i32, [i32, vp]),
    "nvq_event_record": (i32, [i32, vp, vp]),
    "nvq_stream_wait_event": (i32, [i32, vp, vp]),
    "nvq_event_sync": (i32, [i32, vp]),
    "nvq_event_elapsed_ms": (i32, [vp, vp, C.POINTER(f32c)]),
    "nvq_graph_begin_capture": (i32, [i32, vp]),
    "nvq_graph_end_capture": (i32, [i32, vp, pvp]),
    "nvq_graph_launch": (i32, [i32, vp, vp]),
    "nvq_graph_destroy": (i32, [i32, vp]),
    "nvq_launch_count": (u64, []),
    "nvq_cast": (i32, [vp, i32, vp, i32, sz, i32, vp]),
    "nvq_cast_host": (i32, [vp, i32, vp, i32, sz, i32]),
    "nvq_amax_f32": (i32, [vp, sz, vp, i32, vp]),
    "nvq_quantize_fp8": (i32, [vp, vp, sz, i32, f32c, i32, vp]),
    "nvq_dequantize_fp8": (i32, [vp, vp, sz, i32, f32c, i32, vp]),
    "nvq_quantize_fp8_tensor": (i32, [vp, vp, vp, sz, i32, vp, i32, vp]),
    "nvq_quantize_fp8_rows": (i32, [vp, vp, vp, sz, sz, i32, i32, vp]),
    "nvq_quantize_fp4_b32": (i32, [vp, vp, vp, sz, sz, i32, vp]),
    "nvq_dequantize_fp4_b32": (i32, [vp, vp, vp, sz, sz, i32, vp]),
    "nvq_linear_workspace_bytes": (i32, [sz, sz, i32, C.POINTER(sz)]),
    "nvq_linear_fwd": (i32, [vp, vp, vp, i32, vp, vp, sz, sz, sz, vp, sz, i32, vp]),
    "nvq_linear_fwd_opts": (i32, [vp, vp, vp, i32, vp, vp, sz, sz, sz, vp, sz, C.c_uint32, i32, vp]),
    "nvq_linear_expand_weight": (i32, [vp, vp, i32, vp, sz, sz, i32, vp]),
    "nvq_linear_fwd_expanded": (i32, [vp, vp, vp, vp, vp, sz, sz, sz, i32, i32, vp]),
    "nvq_peer_handle_bytes": (i32, [C.POINTER(sz)]),
    "nvq_peer_create": (i32, [pvp, i32, i32, sz, C.c_uint32, i32]),
    "nvq_peer_export": (i32, [vp, vp]),
    "nvq_peer_connect": (i32, [vp, vp]),
    "nvq_peer_grad_buffer": (i32, [vp, i32, pvp]),
    "nvq_peer_allreduce_sgd": (i32, [vp, i32, vp, f32c, vp]),
    "nvq_peer_destroy": (i32, [vp]),
    "nvq_linear_cache_create": (i32, [pvp, sz, sz, i32, i32]),
    "nvq_linear_cache_fwd": (i32, [vp, vp, vp, vp, vp, vp, sz, u64, i32, C.POINTER(i32), vp]),
    "nvq_linear_cache_destroy": (i32, [vp]),
    "nvq_linear_w8a8_workspace_bytes": (i32, [sz, sz, C.POINTER(sz)]),
    "nvq_linear_fwd_w8a8": (i32, [vp, vp, vp, vp, vp, sz, sz, sz, vp, sz, i32, vp]),
    "nvq_linear_bwd_q_workspace_bytes": (i32, [sz, sz, sz, C.POINTER(sz)]),
    "nvq_linear_bwd_q": (i32, [vp, vp, vp, vp, vp, vp, i32, vp, sz, sz, sz, vp, sz, i32, vp]),
    "nvq_device_error_flag": (i32, [i32, C.POINTER(i32)]),
    "nvq_selftest_bounded_wait": (i32, [i32, vp]),
    "nvq_linear_fwd_f32": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp, i32, vp]),
    "nvq_linear_bwd_f32": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp]),
    "nvq_relu_fwd_f32": (i32, [vp, vp, vp, sz, i32, vp]),
    "nvq_mul_f32": (i32, [vp, vp, vp, sz, i32, vp]),
    "nvq_softmax_ce_f32": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, vp]),
    "nvq_ce_loss_f32": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "nvq_sgd_step_f32": (i32, [vp, vp, sz, f32c, f32c, i32, vp]),
    "nvq_adamw_step_f32": (i32, [vp, vp, vp, vp, sz] + [f32c] * 9 + [i32, i32, vp]),
    "nvq_conv2d_out_size": (i32, [i32] * 8 + [C.POINTER(i32), C.POINTER(i32)]),
    "nvq_im2col_f32": (i32, [vp, vp] + [i32] * 10 + [i32, i32, vp]),
    "nvq_conv2d_fwd_f32": (i32, [vp, vp, vp, vp, vp] + [i32] * 11 + [i32, i32, vp]),
    "nvq_conv2d_bwd_f32": (i32, [vp] * 8 + [i32] * 11 + [i32, vp]),
    "nvq_conv2d_q_sizes": (i32, [i32] * 11 + [C.POINTER(sz), C.POINTER(sz)]),
    "nvq_batchnorm_scratch_bytes": (sz, [i32]),
    "nvq_batchnorm_fwd_f32": (i32, [vp] * 8 + [i32, i32, i32, f64c, f64c, i32, i32, vp]),
    "nvq_batchnorm_bwd_f32": (i32, [vp] * 8 + [i32, i32, i32, f64c, i32, vp]),
    "nvq_maxpool2d_fwd_f32": (i32, [vp, vp] + [i32] * 10 + [i32, i32, vp]),
    "nvq_maxpool2d_bwd_f32": (i32, [vp, vp, vp] + [i32] * 10 + [i32, i32, vp]),
    "nvq_gap2d_fwd_f32": (i32, [vp, vp, sz, i32, i32, vp]),
    "nvq_gap2d_bwd_f32": (i32, [vp, vp, sz, i32, i32, vp]),
    "nvq_dropout_f32": (i32, [vp, vp, vp, sz, f32c, i32, vp]),
    "nvq_adamw_step_f64": (i32, [vp, vp, vp, vp, sz] + [f64c] * 9 + [i32, i32, vp]),
    "nvq_conv2d_fwd_q": (i32, [vp, vp, vp, i32, vp, vp, vp, vp, vp, sz] + [i32] * 11 + [i32, i32, vp]),
    "nvq_conv2d_fwd_q_opts": (i32, [vp, vp, vp, i32, vp, vp, vp, vp, vp, sz] + [i32] * 11 +
                              [i32, C.c_uint32, i32, vp]),
    "nvq_conv2d_fwd_q_nhwc": (i32, [vp, vp, vp, i32, vp, vp, vp, sz] + [i32] * 11 + [i32, i32, vp]),
    "nvq_nchw_f32_to_nhwc_bf16": (i32, [vp, vp, i32, i32, i32, i32, vp]),
    "nvq_nhwc_bf16_to_nchw_f32": (i32, [vp, vp, i32, i32, i32, i32, vp]),
    "nvq_comm_unique_id": (i32, [vp]),
    "nvq_comm_init": (i32, [vp, i32, i32, i32, pvp]),
    "nvq_comm_destroy": (i32, [vp]),
    "nvq_allreduce_sum_f32": (i32, [vp, vp, sz, i32, vp]),
    "nvq_comm_wait": (i32, [vp, i32, vp, C.c_uint32]),
    "nvq_comm_abort": (i32, [vp]),
    "nvq_linear_fwd_static": (i32, [vp, vp, vp, i32, vp, vp, sz, sz, sz, vp, i32, vp]),
}


class NvqError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"nvq status {status}: {message}")
        self.status = status


_lib = None


def _point_at_bundled_nccl() -> None:
    """Name the NCCL build that ships with PyTorch (when present) as the one the library
    should dlopen, so that a process which also imports torch holds a single libnccl."""
    if "NVQ_NCCL_LIB" in os.environ:
        return
    try:
        import importlib.util
        spec = importlib.util.find_spec("nvidia.nccl")
        for root in (spec.submodule_search_locations if spec else []):
            cand = os.path.join(root, "lib", "libnccl.so.2")
            if os.path.exists(cand):
                os.environ["NVQ_NCCL_LIB"] = cand
                return
    except Exception:
        pass


def lib() -> C.CDLL:
    """The loaded library.  Raises if it has not been built (no CPU fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} not found: build it with `python -m novann_b200.build` "
                "(there is no CPU fallback)")
        _point_at_bundled_nccl()
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status: int) -> None:
    if status != OK:
        msg = lib().nvq_last_error()
        raise NvqError(status, msg.decode() if msg else "")
