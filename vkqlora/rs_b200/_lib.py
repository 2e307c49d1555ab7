"""ctypes declarations for libqlora_cuda.so (the C ABI in include/qlora_cuda.h).

There is no fallback: if the shared library is missing or cannot be loaded this module raises
ImportError and nothing in the package works.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# QLORA_CUDA_LIBRARY names another build of the library (A/B measurements of two builds in one process tree)
LIB_PATH = os.environ.get("QLORA_CUDA_LIBRARY") or os.path.join(_HERE, "libqlora_cuda.so")

OK, ERR_SHAPE_MISMATCH, ERR_INVALID_CONFIG, ERR_GPU = 0, 1, 2, 3
DTYPE_F32, DTYPE_BF16, DTYPE_F16 = 0, 1, 2
PRECISION_AUTO, PRECISION_FP32_EXACT, PRECISION_BF16, PRECISION_TF32 = 0, 1, 2, 3
SIZE_MAX = (1 << (8 * C.sizeof(C.c_size_t))) - 1

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} not found: build it with `python vkqlora/rs_b200/build.py` "
        "(there is no CPU or pure-Python fallback)")
lib = C.CDLL(LIB_PATH)

_vp, _sz, _i = C.c_void_p, C.c_size_t, C.c_int
_pp = C.POINTER(C.c_void_p)


class QTensorInfo(C.Structure):
    _fields_ = [("rows", _sz), ("cols", _sz), ("block_size", _sz), ("num_elements", _sz), ("num_blocks", _sz),
                ("codes_len", _sz), ("absmax2_len", _sz), ("storage_bytes", _sz), ("double_quant", _i)]


class AdamConfig(C.Structure):
    _fields_ = [("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
                ("block_size", _sz), ("max_resident_pages", _sz)]


class AdamStats(C.Structure):
    _fields_ = [("pages_streamed", _sz), ("state_bytes", _sz)]


# name -> (restype, argtypes); every symbol declared in include/qlora_cuda.h is listed here.
SIGNATURES = {
    "qlc_last_error_message": (C.c_char_p, []),
    "qlc_ctx_create": (_i, [_i, _pp]),
    "qlc_ctx_destroy": (_i, [_vp]),
    "qlc_ctx_set_precision": (_i, [_vp, _i]),
    "qlc_ctx_set_reserved_sms": (_i, [_vp, _i]),
    "qlc_ctx_synchronize": (_i, [_vp]),
    "qlc_ctx_stream": (_vp, [_vp]),
    "qlc_ctx_copy_to_host": (_i, [_vp, _vp, _vp, _sz]),
    "qlc_ctx_copy_to_device": (_i, [_vp, _vp, _vp, _sz]),
    "qlc_ctx_launch_count": (C.c_uint64, [_vp]),
    "qlc_ctx_profile_enable": (_i, [_vp, _i]),
    "qlc_ctx_profile_read": (_i, [_vp, _i, C.POINTER(C.c_double), C.POINTER(C.c_uint64)]),
    "qlc_quantize_nf4": (_i, [_vp, _vp, _sz, _sz, _sz, _sz, _i, _pp]),
    "qlc_quantize_nf4_typed": (_i, [_vp, _vp, _i, _sz, _sz, _sz, _i, _pp]),
    "qlc_quantize_nf4_dev": (_i, [_vp, _vp, _sz, _sz, _sz, _i, _pp]),
    "qlc_qtensor_requantize_dev": (_i, [_vp, _vp, _vp]),
    "qlc_qtensor_from_raw_parts": (_i, [_vp, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _pp]),
    "qlc_qtensor_from_double_quant_parts": (_i, [_vp, _sz, _sz, _sz, _vp, _sz, _vp, _sz, _vp, _sz, _pp]),
    "qlc_qtensor_destroy": (_i, [_vp]),
    "qlc_qtensor_get_info": (_i, [_vp, C.POINTER(QTensorInfo)]),
    "qlc_qtensor_codes": (_i, [_vp, _vp, _sz]),
    "qlc_qtensor_absmax_codes": (_i, [_vp, _vp, _sz]),
    "qlc_qtensor_absmax2": (_i, [_vp, _vp, _sz]),
    "qlc_qtensor_block_scales": (_i, [_vp, _vp, _sz]),
    "qlc_qtensor_device_ptrs": (_i, [_vp, _pp, _pp, _pp, _pp]),
    "qlc_dequantize": (_i, [_vp, _vp, _vp, _sz]),
    "qlc_dequantize_dev": (_i, [_vp, _vp, _vp, _i]),
    "qlc_matmul": (_i, [_vp, _vp, _sz, _vp, _sz, _sz, _sz, _sz, _vp]),
    "qlc_matmul_trans_b": (_i, [_vp, _vp, _sz, _vp, _sz, _sz, _sz, _sz, _vp]),
    "qlc_matmul_trans_a": (_i, [_vp, _vp, _sz, _vp, _sz, _sz, _sz, _sz, _vp]),
    "qlc_layer_create": (_i, [_vp, _vp, _vp, _sz, _vp, _sz, _sz, C.c_float, _pp]),
    "qlc_layer_create_from_fp32": (_i, [_vp, _vp, _sz, _sz, _sz, _sz, _i, _vp, _sz, _vp, _sz, _sz, C.c_float, _pp]),
    "qlc_layer_destroy": (_i, [_vp]),
    "qlc_layer_set_weights": (_i, [_vp, _vp, _sz, _vp, _sz]),
    "qlc_layer_set_weights_dev": (_i, [_vp, _vp, _vp]),
    "qlc_layer_adapter_dev": (_i, [_vp, _pp, _pp]),
    "qlc_layer_adapter_updated": (_i, [_vp]),
    "qlc_train_step_dev": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _sz, _vp]),
    "qlc_layer_dims": (_i, [_vp, C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_sz), C.POINTER(C.c_float)]),
    "qlc_layer_weight": (_vp, [_vp]),
    "qlc_layer_grad_bucket": (_i, [_vp, _pp, C.POINTER(_sz)]),
    "qlc_qlora_forward": (_i, [_vp, _vp, _vp, _sz, _sz, _vp]),
    "qlc_qlora_backward": (_i, [_vp, _vp, _vp, _sz, _vp, _sz, _sz, _vp, _vp, _vp]),
    "qlc_qlora_forward_host": (_i, [_vp, _vp, _vp, _i, _sz, _vp]),
    "qlc_qlora_backward_host": (_i, [_vp, _vp, _vp, _vp, _i, _sz, _vp, _vp, _vp]),
    "qlc_qlora_forward_backward_host": (_i, [_vp, _vp, _vp, _vp, _i, _sz, _vp, _vp, _vp, _vp]),
    "qlc_qlora_forward_backward_host_async": (_i, [_vp, _vp, _vp, _vp, _i, _sz, _vp, _vp, _vp, _vp, C.POINTER(C.c_uint64)]),
    "qlc_ctx_wait": (_i, [_vp, C.c_uint64]),
    "qlc_qlora_forward_dev": (_i, [_vp, _vp, _vp, _i, _sz, _vp]),
    "qlc_qlora_forward_dev_noalloc": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "qlc_qlora_backward_dev": (_i, [_vp, _vp, _vp, _vp, _i, _sz, _vp, _vp, _vp]),
    "qlc_adam_config_default": (None, [C.POINTER(AdamConfig)]),
    "qlc_adam_create": (_i, [_vp, C.POINTER(AdamConfig), _pp]),
    "qlc_adam_destroy": (_i, [_vp]),
    "qlc_adam_step": (_i, [_vp, _sz, _pp, C.POINTER(_sz), _pp, C.POINTER(_sz), C.POINTER(AdamStats)]),
    "qlc_adam_step_dev": (_i, [_vp, _sz, _pp, _pp, C.POINTER(_sz), C.POINTER(AdamStats)]),
    "qlc_adam_set_fast_math": (_i, [_vp, _i]),
    "qlc_adam_state_bytes": (_sz, [_vp]),
    "qlc_adam_get_state": (_i, [_vp, _sz, C.POINTER(_sz), C.POINTER(C.c_uint64), _vp, _vp, _vp, _vp]),
    "qlc_adam_set_state": (_i, [_vp, _sz, _sz, C.c_uint64, _vp, _vp, _vp, _vp]),
    "qlc_adam_paging_info": (_i, [_vp, C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_sz)]),
    "qlc_llama_create": (_i, [_vp, _vp, _vp, _vp, _pp]),
    "qlc_llama_destroy": (_i, [_vp]),
    "qlc_llama_set_layer": (_i, [_vp, _sz, _vp, _vp, _vp, _sz, _i]),
    "qlc_llama_set_layer_mixed": (_i, [_vp, _sz, _vp, _vp, _vp, _vp, _sz, _i]),
    "qlc_llama_attach_adapter": (_i, [_vp, _sz, _i, _vp, _vp, _sz, C.c_float]),
    "qlc_llama_projection": (_vp, [_vp, _sz, _i]),
    "qlc_llama_forward": (_i, [_vp, _vp, _sz, _sz, _vp]),
    "qlc_llama_backward": (_i, [_vp, _vp, _vp, _sz, _sz]),
    "qlc_llama_loss_backward": (_i, [_vp, _vp, _vp, _sz, _sz, C.POINTER(C.c_float)]),
    "qlc_llama_train_step": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, C.POINTER(C.c_float)]),
    "qlc_llama_train_step_dp": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, C.POINTER(C.c_float)]),
    "qlc_llama_adapter_grads": (_i, [_vp, _sz, _i, _vp, _vp]),
    "qlc_llama_adapter_weights": (_i, [_vp, _sz, _i, _vp, _vp]),
    "qlc_comm_unique_id": (_i, [_vp, _sz]),
    "qlc_comm_init": (_i, [_vp, _i, _i, _vp, _sz, _pp]),
    "qlc_comm_allreduce_sum_f32": (_i, [_vp, _vp, _sz]),
    "qlc_allreduce_lora_grads": (_i, [_vp, _vp]),
    "qlc_comm_allreduce_sum_f32_many": (_i, [_vp, _vp, _vp, _sz]),
    "qlc_comm_nranks": (_i, [_vp]),
    "qlc_comm_context": (_vp, [_vp]),
    "qlc_comm_destroy": (_i, [_vp]),
    "qlc_selftest_nf4_codes_of_targets": (_i, [_vp, C.c_uint32, _sz, _vp, _sz]),
    "qlc_selftest_nf4_fast_path": (_i, [_vp, C.c_float, C.c_uint32, C.c_uint64, C.POINTER(C.c_uint64),
                                        C.POINTER(C.c_uint64), C.POINTER(C.c_uint32)]),
    "qlc_selftest_adam_math": (_i, [_vp, _i, C.c_uint32, C.c_uint64, C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "qlc_selftest_wait_timeout": (_i, [_vp, C.c_uint64]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here means header and library disagree
    _fn.restype = _res
    _fn.argtypes = _args


class QloraError(ValueError):
    """Mirror of qlora_core::QloraError (qlora-core/src/error.rs:7-26).

    Derives from ValueError because the reference's Python module maps every QloraError to
    ValueError (qlora-python/src/lib.rs:20-22)."""

    def __init__(self, kind: int, message: str):
        super().__init__(message)
        self.kind = kind


class ShapeMismatch(QloraError):
    pass


class InvalidConfig(QloraError):
    pass


class GpuError(QloraError):
    pass


_KINDS = {ERR_SHAPE_MISMATCH: ShapeMismatch, ERR_INVALID_CONFIG: InvalidConfig, ERR_GPU: GpuError}


def check(status: int) -> None:
    if status != OK:
        msg = lib.qlc_last_error_message().decode("utf-8", "replace")
        raise _KINDS.get(status, GpuError)(status, msg)
