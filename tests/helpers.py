"""Seeded synthetic inputs shared by the parity tests (shapes and distributions of the workload spec)."""
import numpy as np


def awq_random(rng, K, N, group=128):
    """Uniform nibbles, uniform zeros, fp16 scales in [0.002, 0.02]: the single-GEMV workload."""
    q = rng.integers(0, 16, (K, N), dtype=np.uint8)
    z = rng.integers(0, 16, (K // group, N), dtype=np.uint8)
    s = rng.uniform(0.002, 0.02, (K // group, N)).astype(np.float16)
    return q, z, s


def rel_err(y, ref):
    """max |y - ref| / max |ref|: the error measure every matmul / attention tolerance refers to."""
    y = np.asarray(y, np.float64)
    ref = np.asarray(ref, np.float64)
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30))


def make_model_weights(oracle, cfg, seed=0, norm_jitter=0.02):
    """Random-init Qwen3-shaped weights: N(0, 0.02) fp32 quantised to INT4-AWQ g128; bf16 embed / lm_head / norms."""
    rng = np.random.default_rng(seed)
    H, D, I = cfg.hidden, cfg.head_dim, cfg.inter
    QKV = (cfg.n_q_heads + 2 * cfg.n_kv_heads) * D

    def quant(K, N):
        W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
        return oracle.awq_quantize(W, cfg.group)

    def norm(n):
        return oracle.f32_to_bf16((1.0 + norm_jitter * rng.standard_normal(n)).astype(np.float32))

    weights = {
        "embed": oracle.f32_to_bf16((rng.standard_normal((cfg.vocab, H)) * 0.02).astype(np.float32)),
        "final_norm": norm(H),
        "lm_head": oracle.f32_to_bf16((rng.standard_normal((cfg.vocab, H)) * 0.02).astype(np.float32)),
        "layers": [],
    }
    for _ in range(cfg.n_layers):
        lw = {"input_norm": norm(H), "post_norm": norm(H), "q_norm": norm(D), "k_norm": norm(D)}
        for name, (K, N) in {"qkv": (H, QKV), "o": (cfg.n_q_heads * D, H), "gu": (H, 2 * I), "down": (I, H)}.items():
            qw, qz, s = quant(K, N)
            lw[f"{name}_qw"], lw[f"{name}_qz"], lw[f"{name}_s"] = qw, qz, s
        weights["layers"].append(lw)
    return weights
