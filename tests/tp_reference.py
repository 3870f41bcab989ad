"""numpy restatement of the engine's tensor-parallel shard plan (Qwen3Model::load_layer): column split of the fused
QKV (whole heads per rank) and gate|up projections, row split (at group boundaries) of O and down."""
import numpy as np


def _cols(qw, qz, s, col0, cols):
    return qw[:, col0 // 8:(col0 + cols) // 8], qz[:, col0 // 8:(col0 + cols) // 8], s[:, col0:col0 + cols]


def shard_layer(w, cfg, rank, world, group=128):
    D = cfg.head_dim
    Hq, Hkv, I = cfg.n_q_heads // world, cfg.n_kv_heads // world, cfg.inter // world
    out = {}
    parts = [_cols(w["qkv_qw"], w["qkv_qz"], w["qkv_s"], rank * Hq * D, Hq * D),
             _cols(w["qkv_qw"], w["qkv_qz"], w["qkv_s"], cfg.n_q_heads * D + rank * Hkv * D, Hkv * D),
             _cols(w["qkv_qw"], w["qkv_qz"], w["qkv_s"], (cfg.n_q_heads + cfg.n_kv_heads) * D + rank * Hkv * D, Hkv * D)]
    out["qkv_qw"], out["qkv_qz"], out["qkv_s"] = (np.ascontiguousarray(np.concatenate([p[i] for p in parts], 1)) for i in range(3))
    parts = [_cols(w["gu_qw"], w["gu_qz"], w["gu_s"], rank * I, I),
             _cols(w["gu_qw"], w["gu_qz"], w["gu_s"], cfg.inter + rank * I, I)]
    out["gu_qw"], out["gu_qz"], out["gu_s"] = (np.ascontiguousarray(np.concatenate([p[i] for p in parts], 1)) for i in range(3))
    for name, width in (("o", Hq * D), ("down", I)):
        r0 = rank * width
        out[name + "_qw"] = np.ascontiguousarray(w[name + "_qw"][r0:r0 + width])
        out[name + "_qz"] = np.ascontiguousarray(w[name + "_qz"][r0 // group:(r0 + width) // group])
        out[name + "_s"] = np.ascontiguousarray(w[name + "_s"][r0 // group:(r0 + width) // group])
    return out
