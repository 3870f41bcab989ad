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
    "kuiper_bf16_gemv_f32": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "kuiper_rmsnorm_f32": (_i32, [_vp, _vp, _vp, _i32, _i32, _f32, _vp]),
    "kuiper_qknorm_rope_kvwrite": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _i32, _i32,
                                          _vp, _vp, _vp, _vp]),
    "kuiper_flash_decode_workspace_bytes": (_sz, [_i32, _i32, _i32, _i32]),
    "kuiper_flash_decode": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "kuiper_swiglu_f32": (_i32, [_vp, _vp, _i32, _i32, _vp]),
    "kuiper_embedding_bf16": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "kuiper_argmax_f32": (_i32, [_vp, _vp, _i32, _i32, _vp]),
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
        _kernels = lib
    return _kernels


def check(code: int) -> None:
    if code != 0:
        raise KuiperError(code, kernels().kuiper_last_error().decode())
