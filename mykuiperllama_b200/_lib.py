"""ctypes bindings of the two native libraries.

The kernels are reached only through the C ABI declared in ``include/kuiper_b200.h``
(``libkuiper_b200.so``) and the engine through ``include/kuiper_llama.h``
(``libkuiper_llama.so``).  There is no Python or CPU fallback: if a library is missing
the import of the symbol raises.
"""
from __future__ import annotations

import ctypes as C
import os

from . import _build

_kernels = None
_host = None


class KuiperError(RuntimeError):
    """Non-zero status from the C ABI (numbering of the reference's base::StatusCode)."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"kuiper status {code}: {msg}")
        self.code = code


_i32, _i64, _f32, _sz, _vp = C.c_int32, C.c_int64, C.c_float, C.c_size_t, C.c_void_p

# name -> (restype, argtypes); the list every test checks against include/kuiper_b200.h
KERNEL_API = {
    "kuiper_version": (C.c_char_p, []),
    "kuiper_last_error": (C.c_char_p, []),
    "kuiper_set_tuning": (_i32, [C.c_char_p, _i32]),
    "kuiper_add_f32": (_i32, [_vp, _vp, _vp, _i64, _vp]),
    "kuiper_awq_unpack_u8": (_i32, [_vp, _vp, _i32, _i32, _vp]),
    "kuiper_awq_dequant_f32": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "kuiper_awq_dequant_bf16": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "kuiper_awq_gemv_workspace_bytes": (_sz, [_i32, _i32, _i32]),
    "kuiper_workspace_init": (_i32, [_vp, _sz, _vp]),
    "kuiper_awq_gemv_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "kuiper_awq_gemv_accum_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "kuiper_rmsnorm_awq_gemv_accum_f32": (_i32, [_vp, _vp, _f32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "kuiper_swiglu_awq_gemv_accum_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "kuiper_awq_gemv_ticket_bytes": (_sz, []),
    "kuiper_awq_gemv_accum_balanced_f32": (_i32, [_vp, _vp, _f32, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp]),
    "kuiper_awq_gemv_group_table_bytes": (_sz, [_i32]),
    "kuiper_awq_gemv_group_plan": (_i32, [_vp, _i32, _i32, _vp, _vp]),
    "kuiper_awq_gemv_group_f32": (_i32, [_vp, _i32, _i64, _i32, _vp, _vp]),
    "kuiper_awq_gemv_status": (_i32, []),
    "kuiper_awq_gemv_noalloc_scratch_bytes": (_sz, []),
    "kuiper_awq_gemv_f32_noalloc": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "kuiper_awq_gemm_workspace_bytes": (_sz, [_i32, _i32]),
    "kuiper_awq_gemm_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "kuiper_awq_gemm_f16in_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp]),
    "kuiper_awq_gemm_status": (_i32, []),
    "kuiper_allreduce_buffer_bytes": (_sz, [_i32, _i64]),
    "kuiper_allreduce_state_bytes": (_sz, []),
    "kuiper_allreduce_sum_f32": (_i32, [_vp, _vp, _vp, _i32, _i64, _i32, _i32, _vp, _i64, _vp, _vp]),
    "kuiper_argmax_allgather": (_i32, [_vp, _vp, _i32, _i32, _i32, _i32, _vp, _i64, _vp, _vp]),
    "kuiper_allreduce_status": (_i32, [_vp, _i32]),
    "kuiper_bf16_gemv_f32": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "kuiper_rmsnorm_f32": (_i32, [_vp, _vp, _vp, _i32, _i32, _f32, _vp]),
    "kuiper_rmsnorm_f16": (_i32, [_vp, _vp, _vp, _i32, _i32, _f32, _vp]),
    "kuiper_qknorm_rope_kvwrite": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _i32, _i32,
                                          _vp, _vp, _vp, _i32, _vp, _i64, _vp]),
    "kuiper_flash_decode_workspace_bytes": (_sz, [_i32, _i32, _i32, _i32]),
    "kuiper_flash_decode_status": (_i32, []),
    "kuiper_flash_decode": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "kuiper_flash_prefill": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "kuiper_rope_flash_decode": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _f32,
                                        _i32, _i32, _i32, _i32, _vp, _i64, _vp, _sz, _vp]),
    "kuiper_swiglu_f32": (_i32, [_vp, _vp, _i32, _i32, _i32, _vp]),
    "kuiper_swiglu_f16": (_i32, [_vp, _vp, _i32, _i32, _i32, _vp]),
    "kuiper_embedding_bf16": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "kuiper_argmax_f32": (_i32, [_vp, _vp, _i32, _i32, _vp]),
    "kuiper_decode_advance": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _vp]),
}


def _bind(lib: C.CDLL, api: dict) -> None:
    for name, (res, args) in api.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing: fail loudly
        fn.restype = res
        fn.argtypes = args


def kernels() -> C.CDLL:
    """The kernel library; built on first use if the .so is absent or stale."""
    global _kernels
    if _kernels is None:
        path = _build.KERNEL_LIB
        if not os.path.exists(path):
            _build.build_kernels()
        lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
        _bind(lib, KERNEL_API)
        if _build.TRACE:  # measurement build only
            _bind(lib, {"kuiper_flash_trace_read": (_i32, [_vp, _i32]), "kuiper_gemv_trace_read": (_i32, [_vp, _i32])})
        _kernels = lib
    return _kernels


def check(code: int) -> None:
    if code != 0:
        raise KuiperError(code, kernels().kuiper_last_error().decode())


class ModelConfigC(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "hidden", "n_q_heads", "n_kv_heads", "head_dim", "inter", "vocab",
                                         "group", "max_seq", "max_batch", "max_rows")] + \
               [("eps", C.c_float), ("rope_theta", C.c_double), ("act_mode", C.c_int32), ("tp_rank", C.c_int32),
                ("tp_size", C.c_int32)]


LAYER_FIELDS = ("input_norm", "post_norm", "q_norm", "k_norm", "qkv_qw", "qkv_qz", "qkv_s", "o_qw", "o_qz", "o_s",
                "gu_qw", "gu_qz", "gu_s", "down_qw", "down_qz", "down_s")


class LayerWeightsC(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in LAYER_FIELDS]


HOST_API = {
    "kuiper_llama_last_error": (C.c_char_p, []),
    "kuiper_model_create": (_vp, [C.POINTER(ModelConfigC)]),
    "kuiper_model_destroy": (None, [_vp]),
    "kuiper_model_load_layer": (_i32, [_vp, _i32, C.POINTER(LayerWeightsC), _i32]),
    "kuiper_model_load_globals": (_i32, [_vp, _vp, _vp, _vp, _i32]),
    "kuiper_model_load_checkpoint": (_i32, [_vp, C.c_char_p]),
    "kuiper_checkpoint_inspect": (_i32, [C.c_char_p, C.c_char_p, _sz]),
    "kuiper_tp_unique_id": (_i32, [_vp]),
    "kuiper_model_init_tp": (_i32, [_vp, _vp]),
    "kuiper_model_tp_one_shot": (_i32, [_vp]),
    "kuiper_model_tp_status": (_i32, [_vp]),
    "kuiper_model_predict": (_i32, [_vp, _vp, _vp, _vp, _i32, _vp, _vp]),
    "kuiper_model_prefill": (_i32, [_vp, _vp, _i32, _i32, _vp]),
    "kuiper_model_decode_begin": (_i32, [_vp, _vp, _vp, _vp, _i32]),
    "kuiper_model_decode_step": (_i32, [_vp, _i32]),
    "kuiper_model_decode_read": (_i32, [_vp, _vp, _i32]),
    "kuiper_model_decode_predict": (_i32, [_vp, _vp, _i32, _vp]),
    "kuiper_model_kernels_per_step": (_i32, [_vp]),
    "kuiper_model_stream": (_vp, [_vp]),
    "kuiper_model_synchronize": (_i32, [_vp]),
    "kuiper_selftest": (_i32, [_i32, C.c_char_p, _sz]),
}


def host() -> C.CDLL:
    """The C++ engine library (loads the kernel library first)."""
    global _host
    if _host is None:
        kernels()
        path = _build.HOST_LIB
        if not os.path.exists(path):
            _build.build_host()
        lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
        _bind(lib, HOST_API)
        _host = lib
    return _host


def check_host(code: int) -> None:
    if code != 0:
        raise KuiperError(code, host().kuiper_llama_last_error().decode())
