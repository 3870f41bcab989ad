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


def make_model_weights_fast(oracle, cfg, seed=0, norm_jitter=0.02):
    """Same distributions as make_model_weights for the large shapes (hidden 2560 / 4096, full vocabulary): the
    random draws, the 4-bit quantisation (per group and column min-max, the oracle quantiser's rule) and the AWQ
    packing run in torch on the GPU; the result comes back as numpy arrays that the oracle and the engine both load."""
    import torch
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    H, D, I, g = cfg.hidden, cfg.head_dim, cfg.inter, cfg.group
    QKV = (cfg.n_q_heads + 2 * cfg.n_kv_heads) * D
    order = (0, 2, 4, 6, 1, 3, 5, 7)

    def pack(v):  # [rows, N] integers 0..15 -> int32 [rows, N/8] in the AWQ nibble order
        rows, N = v.shape
        v = v.view(rows, N // 8, 8).to(torch.int64)
        w = torch.zeros((rows, N // 8), dtype=torch.int64, device=dev)
        for i, o in enumerate(order):
            w |= v[:, :, o] << (4 * i)
        return ((w + 2 ** 31) % 2 ** 32 - 2 ** 31).to(torch.int32).cpu().numpy()

    def quant(K, N):
        W = torch.randn((K, N), generator=gen, device=dev) * 0.02
        Wg = W.view(K // g, g, N)
        mn, mx = Wg.amin(1), Wg.amax(1)
        s16 = ((mx - mn) / 15.0).clamp_min(1e-8).half()
        s = s16.float()
        z = torch.round(-mn / s).clamp_(0, 15)
        q = (torch.round(Wg / s[:, None, :]) + z[:, None, :]).clamp_(0, 15).view(K, N)
        return pack(q), pack(z), s16.view(torch.int16).cpu().numpy().view(np.uint16)

    def bf16(t):
        return t.bfloat16().view(torch.int16).cpu().numpy().view(np.uint16)

    def norm(n):
        return bf16(1.0 + norm_jitter * torch.randn(n, generator=gen, device=dev))

    weights = {
        "embed": bf16(torch.randn((cfg.vocab, H), generator=gen, device=dev) * 0.02),
        "final_norm": norm(H),
        "lm_head": bf16(torch.randn((cfg.vocab, H), generator=gen, device=dev) * 0.02),
        "layers": [],
    }
    for _ in range(cfg.n_layers):
        lw = {"input_norm": norm(H), "post_norm": norm(H), "q_norm": norm(D), "k_norm": norm(D)}
        for name, (K, N) in {"qkv": (H, QKV), "o": (cfg.n_q_heads * D, H), "gu": (H, 2 * I), "down": (I, H)}.items():
            lw[f"{name}_qw"], lw[f"{name}_qz"], lw[f"{name}_s"] = quant(K, N)
        weights["layers"].append(lw)
    torch.cuda.empty_cache()
    return weights


def write_safetensors(path, tensors, metadata=None):
    """Minimal writer of the safetensors container: tensors = {name: (dtype string, numpy array)}; the array's bytes are
    written as they are (BF16 / F16 travel as uint16 bit patterns)."""
    import json
    import struct
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, (dtype, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)


def checkpoint_tensors(cfg, weights):
    """The synthetic model under the tensor names of a Hugging Face AWQ Qwen3 checkpoint: the fused q|k|v and gate|up
    projections are cut back into their separate tensors (packed words hold 8 columns, so cuts fall on word boundaries)."""
    D = cfg.head_dim
    nq, nkv, I = cfg.n_q_heads * D, cfg.n_kv_heads * D, cfg.inter
    out = {"model.embed_tokens.weight": ("BF16", weights["embed"]), "model.norm.weight": ("BF16", weights["final_norm"]),
           "lm_head.weight": ("BF16", weights["lm_head"])}

    def cut(prefix, qw, qz, s, c0, c1):
        out[prefix + ".qweight"] = ("I32", qw[:, c0 // 8:c1 // 8])
        out[prefix + ".qzeros"] = ("I32", qz[:, c0 // 8:c1 // 8])
        out[prefix + ".scales"] = ("F16", s[:, c0:c1])

    for i, lw in enumerate(weights["layers"]):
        p = f"model.layers.{i}"
        out[p + ".input_layernorm.weight"] = ("BF16", lw["input_norm"])
        out[p + ".post_attention_layernorm.weight"] = ("BF16", lw["post_norm"])
        out[p + ".self_attn.q_norm.weight"] = ("BF16", lw["q_norm"])
        out[p + ".self_attn.k_norm.weight"] = ("BF16", lw["k_norm"])
        cut(p + ".self_attn.q_proj", lw["qkv_qw"], lw["qkv_qz"], lw["qkv_s"], 0, nq)
        cut(p + ".self_attn.k_proj", lw["qkv_qw"], lw["qkv_qz"], lw["qkv_s"], nq, nq + nkv)
        cut(p + ".self_attn.v_proj", lw["qkv_qw"], lw["qkv_qz"], lw["qkv_s"], nq + nkv, nq + 2 * nkv)
        cut(p + ".self_attn.o_proj", lw["o_qw"], lw["o_qz"], lw["o_s"], 0, cfg.hidden)
        cut(p + ".mlp.gate_proj", lw["gu_qw"], lw["gu_qz"], lw["gu_s"], 0, I)
        cut(p + ".mlp.up_proj", lw["gu_qw"], lw["gu_qz"], lw["gu_s"], I, 2 * I)
        cut(p + ".mlp.down_proj", lw["down_qw"], lw["down_qz"], lw["down_s"], 0, cfg.hidden)
    return out
