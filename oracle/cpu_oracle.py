"""ctypes/numpy front end of the CPU oracle (``oracle/liboracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke`` and by
the CPU-baseline / reference legs of ``bench.py`` as the checker.  The product (the
CUDA kernels and the C++ engine) never imports it.

PARITY UNPINNED: the reference repository has no implementation, golden vector or
known-answer test for the INT4/attention/norm path (its op headers
``kuiper/include/op/matmul.h:1-11`` ... are empty), so these functions restate the
workload specification; see ``oracle/oracle.h``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

ROUND_NONE, ROUND_FP16, ROUND_BF16, ROUND_I16_BLOCK32, ROUND_ENGINE = 0, 1, 2, 3, 4
AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


def build(force: bool = False) -> str:
    """Compile ``oracle.c`` with the committed Makefile (gcc, OpenMP)."""
    src_m = max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("oracle.c", "oracle.h", "Makefile"))
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < src_m:
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_model_create.restype = C.c_void_p
        _lib.orc_model_kcache.restype = C.c_void_p
        _lib.orc_model_vcache.restype = C.c_void_p
        _lib.orc_f32_to_f16.restype = C.c_uint16
        _lib.orc_f32_to_f16.argtypes = [C.c_float]
    return _lib


def set_num_threads(n: int) -> int:
    """OpenMP threads of the oracle's loops (n <= 0 only queries); returns the number in effect."""
    return int(lib().orc_set_num_threads(int(n)))


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"], "oracle wants C-contiguous arrays"
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# --------------------------------------------------------------------------- conversions
def f32_to_bf16(a) -> np.ndarray:
    a = _f32(a)
    out = np.empty(a.shape, np.uint16)
    lib().orc_f32_to_bf16_n(_p(a), _p(out), C.c_int64(a.size))
    return out


def f32_to_f16(a) -> np.ndarray:
    a = _f32(a)
    out = np.empty(a.shape, np.uint16)
    lib().orc_f32_to_f16_n(_p(a), _p(out), C.c_int64(a.size))
    return out


def bf16_to_f32(a) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, np.float32)
    lib().orc_bf16_to_f32_n(_p(a), _p(out), C.c_int64(a.size))
    return out


# --------------------------------------------------------------------------- element ops
def add(a, b) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    out = np.empty_like(a)
    lib().orc_add(_p(a), _p(b), _p(out), C.c_int64(a.size))
    return out


def swiglu(gate, up) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    lib().orc_swiglu(_p(gate), _p(up), _p(out), C.c_int64(gate.size))
    return out


def rmsnorm(x, w_bf16, eps=1e-6) -> np.ndarray:
    x = _f32(x)
    M, H = x.shape
    out = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(np.ascontiguousarray(w_bf16, np.uint16)), _p(out), M, H, C.c_float(eps))
    return out


def embedding(tokens, table_bf16) -> np.ndarray:
    tokens = np.ascontiguousarray(tokens, np.int32)
    V, H = table_bf16.shape
    out = np.empty((tokens.size, H), np.float32)
    lib().orc_embedding(_p(tokens), _p(table_bf16), _p(out), tokens.size, H)
    return out


def argmax(logits) -> np.ndarray:
    logits = _f32(logits)
    M, V = logits.shape
    out = np.empty(M, np.int32)
    lib().orc_argmax(_p(logits), M, V, _p(out))
    return out


# --------------------------------------------------------------------------- AWQ
def awq_pack(q) -> np.ndarray:
    q = np.ascontiguousarray(q, np.uint8)
    K, N = q.shape
    out = np.empty((K, N // 8), np.int32)
    lib().orc_awq_pack(_p(q), K, N, _p(out))
    return out


def awq_unpack(words) -> np.ndarray:
    words = np.ascontiguousarray(words, np.int32)
    K, NW = words.shape
    out = np.empty((K, NW * 8), np.uint8)
    lib().orc_awq_unpack(_p(words), K, NW * 8, _p(out))
    return out


def awq_dequant(qweight, qzeros, scales_f16, group=128) -> np.ndarray:
    K, NW = qweight.shape
    N = NW * 8
    out = np.empty((K, N), np.float32)
    lib().orc_awq_dequant(_p(qweight), _p(qzeros), _p(scales_f16), K, N, group, _p(out))
    return out


def awq_quantize(W, group=128):
    W = _f32(W)
    K, N = W.shape
    qw = np.empty((K, N // 8), np.int32)
    qz = np.empty((K // group, N // 8), np.int32)
    s = np.empty((K // group, N), np.uint16)
    lib().orc_awq_quantize(_p(W), K, N, group, _p(qw), _p(qz), _p(s))
    return qw, qz, s


def gemv_f32(x, W, acc_double=True, act_round=ROUND_NONE) -> np.ndarray:
    x, W = _f32(x), _f32(W)
    M, K = x.shape
    N = W.shape[1]
    y = np.empty((M, N), np.float32)
    lib().orc_gemv_f32(_p(x), _p(W), _p(y), M, K, N, int(acc_double), act_round)
    return y


def awq_gemv(x, qweight, qzeros, scales_f16, group=128, acc_double=True, act_round=ROUND_NONE) -> np.ndarray:
    x = _f32(x)
    M, K = x.shape
    N = qweight.shape[1] * 8
    y = np.empty((M, N), np.float32)
    lib().orc_awq_gemv(_p(x), _p(qweight), _p(qzeros), _p(scales_f16), _p(y), M, K, N, group,
                       int(acc_double), act_round)
    return y


def bf16_gemv(x, W_bf16, acc_double=True) -> np.ndarray:
    x = _f32(x)
    M, K = x.shape
    N = W_bf16.shape[0]
    y = np.empty((M, N), np.float32)
    lib().orc_bf16_gemv(_p(x), _p(W_bf16), _p(y), M, K, N, int(acc_double))
    return y


# --------------------------------------------------------------------------- rotary / attention
def rope_tables(max_pos, D, theta):
    c = np.empty((max_pos, D // 2), np.float32)
    s = np.empty((max_pos, D // 2), np.float32)
    lib().orc_rope_tables(max_pos, D, C.c_double(theta), _p(c), _p(s))
    return c, s


def qknorm_rope_kvwrite(qkv, q_norm_w, k_norm_w, cos_t, sin_t, pos, slot, Nq, Nkv, D, eps, kcache, vcache):
    """kcache/vcache: uint16 [n_slots, Nkv, max_seq, D], updated in place.  Returns q [M,Nq,D]."""
    qkv = _f32(qkv)
    M = qkv.shape[0]
    pos = np.ascontiguousarray(pos, np.int32)
    slot = np.ascontiguousarray(slot, np.int32)
    max_seq = kcache.shape[2]
    q = np.empty((M, Nq, D), np.float32)
    lib().orc_qknorm_rope_kvwrite(_p(qkv), _p(q_norm_w), _p(k_norm_w), _p(cos_t), _p(sin_t), _p(pos), _p(slot),
                                  M, Nq, Nkv, D, C.c_float(eps), max_seq, _p(q), _p(kcache), _p(vcache))
    return q


def attention(q, kcache, vcache, seq_len, slot) -> np.ndarray:
    q = _f32(q)
    M, Nq, D = q.shape
    _, Nkv, max_seq, _ = kcache.shape
    seq_len = np.ascontiguousarray(seq_len, np.int32)
    slot = np.ascontiguousarray(slot, np.int32)
    out = np.empty_like(q)
    lib().orc_attention(_p(q), _p(kcache), _p(vcache), _p(seq_len), _p(slot), M, Nq, Nkv, D, max_seq, _p(out))
    return out


# --------------------------------------------------------------------------- whole decoder
class _Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("n_layers", "hidden", "n_q_heads", "n_kv_heads", "head_dim", "inter", "vocab", "group",
                 "max_seq", "max_batch")] + [("eps", C.c_float), ("rope_theta", C.c_double), ("act_round", C.c_int32)]


class _Layer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in
                ("input_norm", "post_norm", "q_norm", "k_norm",
                 "qkv_qw", "qkv_qz", "qkv_s", "o_qw", "o_qz", "o_s",
                 "gu_qw", "gu_qz", "gu_s", "down_qw", "down_qz", "down_s")]


LAYER_FIELDS = tuple(n for n, _ in _Layer._fields_)


@dataclass
class ModelConfig:
    n_layers: int
    hidden: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    inter: int
    vocab: int
    group: int = 128
    max_seq: int = 256
    max_batch: int = 1
    eps: float = 1e-6
    rope_theta: float = 1e6
    act_round: int = ROUND_NONE


class OracleModel:
    """Qwen3-shaped decoder on the CPU.  ``weights`` is a dict with ``embed``, ``final_norm``,
    ``lm_head`` (uint16 bf16 arrays) and ``layers`` (list of dicts keyed by LAYER_FIELDS)."""

    def __init__(self, cfg: ModelConfig, weights: dict):
        self.cfg = cfg
        self._keep = weights  # keep the numpy arrays alive
        c = _Config(cfg.n_layers, cfg.hidden, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.inter, cfg.vocab,
                    cfg.group, cfg.max_seq, cfg.max_batch, cfg.eps, cfg.rope_theta, cfg.act_round)
        arr = (_Layer * cfg.n_layers)()
        for i, lw in enumerate(weights["layers"]):
            for name in LAYER_FIELDS:
                a = lw[name]
                assert a.flags["C_CONTIGUOUS"]
                setattr(arr[i], name, a.ctypes.data)
        self._h = C.c_void_p(lib().orc_model_create(C.byref(c), _p(weights["embed"]), _p(weights["final_norm"]),
                                                    _p(weights["lm_head"]), arr))

    def forward(self, tokens, pos, slot=None, acc_double=True, want_logits=True, logit_rows=None):
        """One pass over the rows; logits / greedy ids for the last ``logit_rows`` rows (default all)."""
        tokens = np.ascontiguousarray(tokens, np.int32)
        pos = np.ascontiguousarray(pos, np.int32)
        M = tokens.size
        R = M if logit_rows is None else logit_rows
        slot = np.zeros(M, np.int32) if slot is None else np.ascontiguousarray(slot, np.int32)
        logits = np.empty((R, self.cfg.vocab), np.float32) if want_logits else None
        nxt = np.empty(R, np.int32)
        lib().orc_model_forward(self._h, _p(tokens), _p(pos), _p(slot), M, int(acc_double), R,
                                _p(logits) if want_logits else None, _p(nxt))
        return logits, nxt

    def caches(self):
        c = self.cfg
        shape = (c.n_layers, c.max_batch, c.n_kv_heads, c.max_seq, c.head_dim)
        n = int(np.prod(shape))
        k = np.ctypeslib.as_array(C.cast(lib().orc_model_kcache(self._h), C.POINTER(C.c_uint16)), (n,)).reshape(shape)
        v = np.ctypeslib.as_array(C.cast(lib().orc_model_vcache(self._h), C.POINTER(C.c_uint16)), (n,)).reshape(shape)
        return k, v

    def close(self):
        if self._h:
            lib().orc_model_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
