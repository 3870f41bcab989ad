"""Python handle on the C++ engine (``model::Qwen3Model`` behind ``include/kuiper_llama.h``).

Used by the tests and the benchmark; all work happens in the native libraries.  Weights
are numpy arrays (host) or torch CUDA tensors (device); the engine copies and, under
tensor parallelism, shards them into its own device memory.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from ._lib import LAYER_FIELDS, LayerWeightsC, ModelConfigC, check_host, host


@dataclass
class EngineConfig:
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
    max_rows: int = 8
    eps: float = 1e-6
    rope_theta: float = 1e6
    act_mode: int = 1
    tp_rank: int = 0
    tp_size: int = 1


def _addr(a):
    """(address, on_device) of a numpy array or a torch tensor."""
    if isinstance(a, np.ndarray):
        assert a.flags["C_CONTIGUOUS"]
        return a.ctypes.data, False
    assert a.is_contiguous()
    return a.data_ptr(), a.is_cuda


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


class Qwen3Engine:
    def __init__(self, cfg: EngineConfig):
        self.cfg = cfg
        c = ModelConfigC(cfg.n_layers, cfg.hidden, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.inter, cfg.vocab,
                         cfg.group, cfg.max_seq, cfg.max_batch, cfg.max_rows, cfg.eps, cfg.rope_theta, cfg.act_mode,
                         cfg.tp_rank, cfg.tp_size)
        self._h = host().kuiper_model_create(C.byref(c))
        if not self._h:
            raise RuntimeError("kuiper_model_create failed: " + host().kuiper_llama_last_error().decode())

    # ---- weights
    def load_layer(self, idx: int, lw: dict) -> None:
        s = LayerWeightsC()
        dev = None
        for name in LAYER_FIELDS:
            addr, on_dev = _addr(lw[name])
            assert dev is None or dev == on_dev, "a layer's weights must all live on the same side"
            dev = on_dev
            setattr(s, name, addr)
        check_host(host().kuiper_model_load_layer(self._h, idx, C.byref(s), int(dev)))

    def load_globals(self, embed, final_norm, lm_head) -> None:
        (e, d1), (f, d2), (l, d3) = _addr(embed), _addr(final_norm), _addr(lm_head)
        assert d1 == d2 == d3
        check_host(host().kuiper_model_load_globals(self._h, e, f, l, int(d1)))

    def load(self, weights: dict) -> None:
        self.load_globals(weights["embed"], weights["final_norm"], weights["lm_head"])
        for i, lw in enumerate(weights["layers"]):
            self.load_layer(i, lw)

    def load_checkpoint(self, path: str) -> None:
        """Loads every weight from an AWQ checkpoint in the safetensors container (Hugging Face Qwen3 tensor names)."""
        check_host(host().kuiper_model_load_checkpoint(self._h, str(path).encode()))

    # ---- tensor parallel
    @staticmethod
    def tp_unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        check_host(host().kuiper_tp_unique_id(buf))
        return buf.raw

    def init_tp(self, unique_id: bytes) -> None:
        check_host(host().kuiper_model_init_tp(self._h, C.c_char_p(unique_id)))

    def tp_one_shot(self) -> bool:
        """True if decode rows are all-reduced by the one-shot exchange over peer memory (else NCCL)."""
        return bool(host().kuiper_model_tp_one_shot(self._h))

    def tp_status(self) -> None:
        """Raises if a bounded wait of the one-shot all-reduce ever ran out."""
        check_host(host().kuiper_model_tp_status(self._h))

    # ---- passes
    def predict(self, tokens, pos, slot=None, want_logits=False):
        tokens, pos = _i32(tokens), _i32(pos)
        M = tokens.size
        slot = np.zeros(M, np.int32) if slot is None else _i32(slot)
        nxt = np.empty(M, np.int32)
        logits = np.empty((M, self.cfg.vocab), np.float32) if want_logits else None
        check_host(host().kuiper_model_predict(self._h, tokens.ctypes.data, pos.ctypes.data, slot.ctypes.data, M,
                                               nxt.ctypes.data, logits.ctypes.data if want_logits else None))
        return (logits, nxt) if want_logits else nxt

    def prefill(self, tokens, slot=0) -> int:
        tokens = _i32(tokens)
        nxt = C.c_int32(0)
        check_host(host().kuiper_model_prefill(self._h, tokens.ctypes.data, tokens.size, slot, C.byref(nxt)))
        return int(nxt.value)

    def decode_begin(self, tokens, pos, slot=None) -> None:
        tokens, pos = _i32(tokens), _i32(pos)
        slot = np.arange(tokens.size, dtype=np.int32) if slot is None else _i32(slot)
        check_host(host().kuiper_model_decode_begin(self._h, tokens.ctypes.data, pos.ctypes.data, slot.ctypes.data,
                                                    tokens.size))

    def decode_step(self, n=1) -> None:
        check_host(host().kuiper_model_decode_step(self._h, n))

    def decode_read(self, B) -> np.ndarray:
        out = np.empty(B, np.int32)
        check_host(host().kuiper_model_decode_read(self._h, out.ctypes.data, B))
        return out

    def decode_predict(self, tokens) -> np.ndarray:
        tokens = _i32(tokens)
        out = np.empty(tokens.size, np.int32)
        check_host(host().kuiper_model_decode_predict(self._h, tokens.ctypes.data, tokens.size, out.ctypes.data))
        return out

    @property
    def kernels_per_step(self) -> int:
        return host().kuiper_model_kernels_per_step(self._h)

    @property
    def stream(self) -> int:
        return host().kuiper_model_stream(self._h) or 0

    def synchronize(self) -> None:
        check_host(host().kuiper_model_synchronize(self._h))

    def close(self) -> None:
        if self._h:
            host().kuiper_model_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
