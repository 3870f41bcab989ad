"""Generates tests/golden/qwen3_tiny_hf.npz: an independent cross-check of the oracle's block semantics.

The reference repository holds no golden vector for the decode path, so this fixture does not pin parity
with it.  What it pins is that the oracle's reading of the Qwen3 block (pre-norm, per-head q/k RMSNorm
before rotary, half-split rotary pairing, theta, GQA head mapping, SwiGLU, eps placement) agrees with an
independent implementation: the `transformers` Qwen3 model, random-initialised on the CPU in fp32 and
loaded with the *dequantised* weights of a seeded tiny INT4-AWQ model.  Run from the repository root:

    python tests/golden/make_golden.py

Stored: the packed weights (so the test does not depend on numpy's random streams), the prompt, and the
fp32 logits `transformers` produced for the prompt rows and for 4 cached decode steps.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import make_model_weights  # noqa: E402
from oracle import cpu_oracle as orc  # noqa: E402

CFG = dict(n_layers=2, hidden=128, n_q_heads=2, n_kv_heads=1, head_dim=128, inter=256, vocab=512, max_seq=32, max_batch=1)


def main():
    from transformers import Qwen3Config, Qwen3ForCausalLM
    ocfg = orc.ModelConfig(**CFG)
    w = make_model_weights(orc, ocfg, seed=11, norm_jitter=0.1)
    hf_cfg = Qwen3Config(vocab_size=CFG["vocab"], hidden_size=CFG["hidden"], intermediate_size=CFG["inter"],
                         num_hidden_layers=CFG["n_layers"], num_attention_heads=CFG["n_q_heads"],
                         num_key_value_heads=CFG["n_kv_heads"], head_dim=CFG["head_dim"], rms_norm_eps=1e-6,
                         rope_theta=1e6, max_position_embeddings=64, tie_word_embeddings=False, attention_bias=False,
                         use_sliding_window=False, attn_implementation="eager")
    model = Qwen3ForCausalLM(hf_cfg).float().eval()
    sd = {}
    f = lambda a: torch.from_numpy(orc.bf16_to_f32(a))
    sd["model.embed_tokens.weight"] = f(w["embed"])
    sd["lm_head.weight"] = f(w["lm_head"])
    sd["model.norm.weight"] = f(w["final_norm"])
    Nq, Nkv, D, I = CFG["n_q_heads"], CFG["n_kv_heads"], CFG["head_dim"], CFG["inter"]
    for l, lw in enumerate(w["layers"]):
        deq = lambda n: torch.from_numpy(orc.awq_dequant(lw[f"{n}_qw"], lw[f"{n}_qz"], lw[f"{n}_s"]))  # [K, N]
        p = f"model.layers.{l}."
        qkv, gu = deq("qkv"), deq("gu")
        sd[p + "self_attn.q_proj.weight"] = qkv[:, : Nq * D].T.contiguous()
        sd[p + "self_attn.k_proj.weight"] = qkv[:, Nq * D: (Nq + Nkv) * D].T.contiguous()
        sd[p + "self_attn.v_proj.weight"] = qkv[:, (Nq + Nkv) * D:].T.contiguous()
        sd[p + "self_attn.o_proj.weight"] = deq("o").T.contiguous()
        sd[p + "mlp.gate_proj.weight"] = gu[:, :I].T.contiguous()
        sd[p + "mlp.up_proj.weight"] = gu[:, I:].T.contiguous()
        sd[p + "mlp.down_proj.weight"] = deq("down").T.contiguous()
        sd[p + "self_attn.q_norm.weight"] = f(lw["q_norm"])
        sd[p + "self_attn.k_norm.weight"] = f(lw["k_norm"])
        sd[p + "input_layernorm.weight"] = f(lw["input_norm"])
        sd[p + "post_attention_layernorm.weight"] = f(lw["post_norm"])
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected and all("rotary" in m or "inv_freq" in m for m in missing), (missing, unexpected)

    rng = np.random.default_rng(5)
    prompt = rng.integers(0, CFG["vocab"], 7).astype(np.int64)
    with torch.no_grad():
        out = model(torch.from_numpy(prompt)[None], use_cache=True)
        prompt_logits = out.logits[0].numpy()
        past, tok = out.past_key_values, int(out.logits[0, -1].argmax())
        step_logits, step_tokens = [], []
        for _ in range(4):
            step_tokens.append(tok)
            out = model(torch.tensor([[tok]]), past_key_values=past, use_cache=True)
            past = out.past_key_values
            step_logits.append(out.logits[0, 0].numpy())
            tok = int(out.logits[0, 0].argmax())
    arrays = {"prompt": prompt.astype(np.int32), "prompt_logits": prompt_logits.astype(np.float32),
              "step_tokens": np.array(step_tokens, np.int32), "step_logits": np.stack(step_logits).astype(np.float32),
              "embed": w["embed"], "lm_head": w["lm_head"], "final_norm": w["final_norm"]}
    for l, lw in enumerate(w["layers"]):
        for k, v in lw.items():
            arrays[f"layer{l}.{k}"] = v
    path = os.path.join(ROOT, "tests", "golden", "qwen3_tiny_hf.npz")
    np.savez_compressed(path, **arrays)
    print("wrote", path, os.path.getsize(path), "bytes")

    # immediate check against the oracle
    ref = orc.OracleModel(ocfg, w)
    lg, _ = ref.forward(prompt.astype(np.int32), np.arange(7, dtype=np.int32))
    print("oracle vs transformers, prompt rows: max abs diff", float(np.abs(lg - prompt_logits).max()),
          "of max", float(np.abs(prompt_logits).max()))




def awq_pack_fixture():
    """tests/golden/awq_pack_vllm.npz: a [K, N] nibble matrix and its AWQ packing as produced by an
    independent packer (vllm's quant_utils.awq_pack), pinning the nibble order [0,2,4,6,1,3,5,7]."""
    from vllm.model_executor.layers.quantization.utils.quant_utils import awq_pack
    rng = np.random.default_rng(21)
    K, N = 24, 64
    q = rng.integers(0, 16, (K, N)).astype(np.int32)
    packed = awq_pack(torch.from_numpy(q), 4, K, N).numpy().astype(np.int32)
    path = os.path.join(ROOT, "tests", "golden", "awq_pack_vllm.npz")
    np.savez_compressed(path, q=q.astype(np.uint8), packed=packed)
    print("wrote", path, "oracle agrees:", bool(np.array_equal(orc.awq_pack(q.astype(np.uint8)), packed)))


if __name__ == "__main__":
    main()
    awq_pack_fixture()
