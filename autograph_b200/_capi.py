"""ctypes declarations of the C ABI in include/autograph_b200.h."""
from __future__ import annotations

import ctypes
from ctypes import (POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint64,
                    c_void_p)
from pathlib import Path

AG_F32, AG_BF16, AG_U8, AG_U16, AG_U32 = 0, 1, 2, 3, 4
AG_OK = 0
AG_ERR_INVALID, AG_ERR_SHAPE, AG_ERR_DTYPE, AG_ERR_CUDA = -1, -2, -3, -4
AG_ERR_OOM, AG_ERR_DEVICE_TIMEOUT, AG_ERR_UNSUPPORTED, AG_ERR_LIMIT = -5, -6, -7, -8
AG_LAYER_CONV2, AG_LAYER_RELU, AG_LAYER_MAXPOOL2, AG_LAYER_FLATTEN, AG_LAYER_DENSE = 0, 1, 2, 3, 4

_STATUS_NAMES = {
    -1: "AG_ERR_INVALID", -2: "AG_ERR_SHAPE", -3: "AG_ERR_DTYPE", -4: "AG_ERR_CUDA",
    -5: "AG_ERR_OOM", -6: "AG_ERR_DEVICE_TIMEOUT", -7: "AG_ERR_UNSUPPORTED", -8: "AG_ERR_LIMIT",
}


class AgError(RuntimeError):
    """An ag_status < 0 with the library's message (≙ the reference's anyhow::Error)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{_STATUS_NAMES.get(status, status)}: {message}")
        self.status = status
        self.message = message


class ConvOptions(ctypes.Structure):
    _fields_ = [("filter", c_int32 * 2), ("padding", c_int32 * 2), ("stride", c_int32 * 2),
                ("dilation", c_int32 * 2)]


class ConvStage(ctypes.Structure):
    _fields_ = [("w", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("oc", c_int64),
                ("options", ConvOptions), ("relu", c_int32), ("pool", c_int32 * 2)]


class LayerSpec(ctypes.Structure):
    _fields_ = [("kind", c_int32), ("a", c_int32), ("b", c_int32), ("c", c_int32), ("d", c_int32),
                ("bias", c_int32)]


def lib_path() -> Path:
    import os
    # AG_LIB: a side build of the same library (e.g. one with phase timestamps compiled in)
    if os.environ.get("AG_LIB"):
        return Path(os.environ["AG_LIB"]).resolve()
    return Path(__file__).resolve().parent / "libautograph_b200.so"


_P = c_void_p
_SIGNATURES = {
    "ag_last_error": (c_char_p, []),
    "ag_version": (c_char_p, []),
    "ag_kernel_launch_count": (c_int, [POINTER(c_uint64)]),
    "ag_device_count": (c_int, [POINTER(c_int)]),
    "ag_device_create": (c_int, [c_int, POINTER(_P)]),
    "ag_device_create_on_stream": (c_int, [c_int, _P, POINTER(_P)]),
    "ag_device_destroy": (c_int, [_P]),
    "ag_device_wait": (c_int, [_P]),
    "ag_debug_expiring_wait": (c_int, [_P, c_uint64]),
    "ag_device_stream": (_P, [_P]),
    "ag_device_ordinal": (c_int, [_P]),
    "ag_alloc": (c_int, [_P, c_size_t, POINTER(_P)]),
    "ag_free": (c_int, [_P, _P]),
    "ag_host_alloc": (c_int, [c_size_t, POINTER(_P)]),
    "ag_host_free": (c_int, [_P]),
    "ag_upload": (c_int, [_P, _P, _P, c_size_t]),
    "ag_download": (c_int, [_P, _P, _P, c_size_t]),
    "ag_copy": (c_int, [_P, _P, _P, c_size_t]),
    "ag_fill_zero": (c_int, [_P, _P, c_size_t]),
    "ag_gemm": (c_int, [_P, c_int, c_int64, c_int64, c_int64, c_float, _P, c_int64, c_int64,
                        c_int64, _P, c_int64, c_int64, c_int64, c_float, _P, c_int64, c_int64,
                        c_int64]),
    "ag_gemm_static_scratch": (c_int, [c_int, _P, c_int, c_int64, c_int64, c_int64, c_float, _P,
                                       c_int64, c_int64, c_int64, _P, c_int64, c_int64, c_int64,
                                       c_float, _P, c_int64, c_int64, c_int64]),
    "ag_dense_forward": (c_int, [_P, c_int, _P, c_int64, c_int64, _P, c_int64, _P, c_int, _P]),
    "ag_dense_chain_forward": (c_int, [_P, c_int, _P, c_int64, c_int32, POINTER(c_int64),
                                       POINTER(_P), POINTER(_P), POINTER(c_int32), _P]),
    "ag_dense_chain_forward_keep": (c_int, [_P, c_int, _P, c_int64, c_int32, POINTER(c_int64),
                                            POINTER(_P), POINTER(_P), POINTER(c_int32),
                                            POINTER(_P), POINTER(_P)]),
    "ag_dense_chain_backward": (c_int, [_P, c_int, c_int64, c_int32, POINTER(c_int64), POINTER(_P),
                                        POINTER(_P), POINTER(_P), _P, POINTER(_P), _P, POINTER(_P),
                                        POINTER(_P)]),
    "ag_conv_dense_chain_forward": (c_int, [_P, c_int, _P, c_int64, c_int64, c_int64, c_int64,
                                            c_int32, POINTER(ConvStage), c_int32, POINTER(c_int64),
                                            POINTER(_P), POINTER(_P), POINTER(c_int32), _P]),
    "ag_conv_dense_chain_forward_u8": (c_int, [_P, c_int, _P, ctypes.c_float, c_int64, c_int64,
                                               c_int64, c_int64, c_int32, POINTER(ConvStage),
                                               c_int32, POINTER(c_int64), POINTER(_P), POINTER(_P),
                                               POINTER(c_int32), _P]),
    "ag_scaled_cast_u8": (c_int, [_P, c_int, ctypes.c_float, _P, _P, c_int64]),
    "ag_model_infer_u8": (c_int, [_P, _P, c_int64, c_int64, c_int64, c_int64, ctypes.c_float, _P]),
    "ag_model_infer_enqueue": (c_int, [_P, _P, c_int64, c_int64, c_int64, c_int64, _P,
                                       ctypes.POINTER(ctypes.c_int32)]),
    "ag_model_infer_wait": (c_int, [_P, ctypes.c_int32]),
    "ag_conv2_relu_max_pool2_forward": (c_int, [_P, c_int, _P, c_int64, c_int64, c_int64, c_int64,
                                                _P, c_int64, _P, POINTER(ConvOptions), c_int,
                                                c_int32, c_int32, _P]),
    "ag_conv2_relu_max_pool2_forward_keep": (c_int, [_P, c_int, _P, c_int64, c_int64, c_int64,
                                                     c_int64, _P, c_int64, _P, POINTER(ConvOptions),
                                                     _P, _P]),
    "ag_conv2_forward": (c_int, [_P, c_int, _P, c_int64, c_int64, c_int64, c_int64, _P, c_int64,
                                 _P, POINTER(ConvOptions), c_int, _P]),
    "ag_conv2_backward_input": (c_int, [_P, c_int, _P, c_int64, c_int64, _P, c_int64, c_int64,
                                        c_int64, POINTER(ConvOptions), _P]),
    "ag_conv2_backward_weight": (c_int, [_P, c_int, _P, c_int64, c_int64, c_int64, c_int64, _P,
                                         c_int64, POINTER(ConvOptions), c_float, _P]),
    "ag_conv2_output_shape": (c_int, [c_int64, c_int64, POINTER(ConvOptions), POINTER(c_int64),
                                      POINTER(c_int64)]),
    "ag_im2col_conv2": (c_int, [_P, c_int, _P, c_int64, c_int64, c_int64, c_int64,
                                POINTER(ConvOptions), _P]),
    "ag_col2im_conv2": (c_int, [_P, c_int, _P, c_int64, c_int64, c_int64, c_int64,
                                POINTER(ConvOptions), _P]),
    "ag_max_pool2": (c_int, [_P, c_int, _P, c_int64, c_int64, c_int64, c_int64, c_int32, c_int32,
                             c_int32, c_int32, _P]),
    "ag_max_pool2_backward_from_input": (c_int, [_P, c_int, _P, c_int64, c_int64, c_int64, c_int64,
                                                 c_int32, c_int32, c_int32, c_int32, _P, _P]),
    "ag_relu_max_pool2_forward": (c_int, [_P, c_int, _P, c_int64, c_int64, c_int64, c_int64, _P]),
    "ag_relu_max_pool2_backward": (c_int, [_P, c_int, _P, c_int64, c_int64, c_int64, c_int64, _P,
                                           _P]),
    "ag_max_pool2_backward": (c_int, [_P, c_int, _P, c_int64, c_int64, c_int64, c_int64, c_int32,
                                      c_int32, c_int32, c_int32, _P]),
    "ag_relu": (c_int, [_P, c_int, _P, _P, c_int64]),
    "ag_relu_backward": (c_int, [_P, c_int, _P, _P, _P, c_int64]),
    "ag_scaled_add": (c_int, [_P, c_int, c_float, _P, _P, c_int64]),
    "ag_bias_add": (c_int, [_P, c_int, _P, _P, c_int64, c_int64, c_int64]),
    "ag_bias_grad": (c_int, [_P, c_int, _P, c_int64, c_int64, c_int64, c_float, _P]),
    "ag_cross_entropy_loss": (c_int, [_P, c_int, c_int, _P, _P, c_int64, c_int64,
                                      POINTER(c_float)]),
    "ag_cross_entropy_loss_device": (c_int, [_P, c_int, c_int, _P, _P, c_int64, c_int64, _P]),
    "ag_cross_entropy_loss_device_grad": (c_int, [_P, c_int, c_int, _P, _P, c_int64, c_int64, _P,
                                                  c_float, _P]),
    "ag_cross_entropy_loss_backward": (c_int, [_P, c_int, c_int, _P, _P, c_int64, c_int64, c_float,
                                               _P]),
    "ag_accuracy": (c_int, [_P, c_int, c_int, _P, _P, c_int64, c_int64, POINTER(c_uint64)]),
    "ag_sgd_update": (c_int, [_P, c_int, _P, _P, c_int64, c_float]),
    "ag_sgd_update_momentum": (c_int, [_P, c_int, _P, _P, _P, c_int64, c_float, c_float]),
    "ag_model_create": (c_int, [_P, c_int, POINTER(LayerSpec), c_int32, c_uint64, POINTER(_P)]),
    "ag_model_create_lenet5": (c_int, [_P, c_int, c_uint64, POINTER(_P)]),
    "ag_model_destroy": (c_int, [_P]),
    "ag_model_parameter_count": (c_int, [_P, POINTER(c_int32)]),
    "ag_model_parameter_len": (c_int, [_P, c_int32, POINTER(c_int64)]),
    "ag_model_set_parameter": (c_int, [_P, c_int32, _P]),
    "ag_model_get_parameter": (c_int, [_P, c_int32, _P]),
    "ag_model_get_gradient": (c_int, [_P, c_int32, _P]),
    "ag_model_set_sgd": (c_int, [_P, c_float]),
    "ag_model_get_velocity": (c_int, [_P, c_int32, _P]),
    "ag_model_set_velocity": (c_int, [_P, c_int32, _P]),
    "ag_model_set_grad_scale": (c_int, [_P, c_float]),
    "ag_model_infer": (c_int, [_P, _P, c_int64, c_int64, c_int64, c_int64, _P]),
    "ag_model_forward_device": (c_int, [_P, _P, c_int64, c_int64, c_int64, c_int64, _P]),
    "ag_model_train_step": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, c_int64, c_float,
                                    POINTER(c_float)]),
    "ag_model_train_forward_backward": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, c_int64,
                                                POINTER(c_float), POINTER(_P), POINTER(c_int64)]),
    "ag_model_apply_update": (c_int, [_P, c_float]),
    "ag_model_last_loss": (c_int, [_P, POINTER(c_float)]),
    "ag_comm_create": (c_int, [POINTER(_P), c_int, POINTER(_P)]),
    "ag_comm_unique_id": (c_int, [_P, c_size_t]),
    "ag_comm_create_rank": (c_int, [_P, c_int, c_int, _P, c_size_t, POINTER(_P)]),
    "ag_comm_destroy": (c_int, [_P]),
    "ag_comm_world": (c_int, [_P, POINTER(c_int), POINTER(c_int)]),
    "ag_comm_set_timeout": (c_int, [_P, ctypes.c_double]),
    "ag_allreduce_sum": (c_int, [_P, c_int, c_int, _P, c_int64]),
    "ag_allreduce_sum_all": (c_int, [_P, c_int, POINTER(_P), c_int64]),
    "ag_comm_wait": (c_int, [_P, c_int]),
    "ag_model_allreduce_update": (c_int, [_P, _P, c_int, c_float]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """Loads the C-ABI library; raises when it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not path.exists():
            raise ImportError(
                f"{path} is missing: build it with `python -m autograph_b200.build` "
                "(nvcc, sm_100a). There is no CPU fallback.")
        handle = ctypes.CDLL(str(path))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def signatures():
    return dict(_SIGNATURES)


def check(status: int) -> None:
    if status != AG_OK:
        raise AgError(status, lib().ag_last_error().decode("utf-8", "replace"))
