"""CPU-only checks: the oracle against its golden vectors, the host logic, the exported C ABI.

No compute call reaches a GPU here; the CUDA parity tests are the gpu-marked files.
"""
import ctypes as C
import json
import os
import re
import subprocess
import sys

import numpy as np
import pytest

from helpers import awq_random, make_model_weights, rel_err

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


# ----------------------------------------------------------------------------- oracle vs golden vectors
def test_oracle_add_matches_reference_pins(oracle):
    # the reference's only numeric pins: test/test_op/test_op_add.cpp:53-70 (2+3==5) and :72-91 (2.1+3.3~=5.4)
    n = 32 * 151
    assert np.all(oracle.add(np.full(n, 2.0, np.float32), np.full(n, 3.0, np.float32)) == 5.0)
    out = oracle.add(np.full(n * 13, 2.1, np.float32), np.full(n * 13, 3.3, np.float32))
    assert np.abs(out - 5.4).max() <= 1e-4


def test_oracle_awq_packing_matches_independent_packer(oracle):
    # fixture written by tests/golden/make_golden.py from vllm's awq_pack
    g = np.load(os.path.join(GOLDEN, "awq_pack_vllm.npz"))
    assert np.array_equal(oracle.awq_pack(g["q"]), g["packed"])
    assert np.array_equal(oracle.awq_unpack(g["packed"]), g["q"])


def test_oracle_awq_order_by_hand(oracle):
    # nibble i of a word holds logical column 8j + [0,2,4,6,1,3,5,7][i]
    q = np.arange(16, dtype=np.uint8).reshape(1, 16) % 16
    words = oracle.awq_pack(q).view(np.uint32)
    assert words[0, 0] == 0x75316420 and words[0, 1] == 0xFDB9ECA8


def test_oracle_conversions_match_numpy_and_torch(oracle):
    import torch
    rng = np.random.default_rng(0)
    a = (rng.standard_normal(100000) * np.exp(rng.uniform(-20, 11, 100000))).astype(np.float32)
    a[:6] = [0.0, -0.0, 65504.0, 65519.9, 6e-8, -1e-10]
    assert np.array_equal(oracle.f32_to_f16(a), a.astype(np.float16).view(np.uint16))
    want = torch.from_numpy(a).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.f32_to_bf16(a), want)


def test_oracle_dequant_and_gemv_against_numpy(oracle):
    rng = np.random.default_rng(1)
    K, N, g = 384, 96, 128
    q, z, s = awq_random(rng, K, N)
    qw, qz = oracle.awq_pack(q), oracle.awq_pack(z)
    W = oracle.awq_dequant(qw, qz, s.view(np.uint16))
    W_np = (q.astype(np.int32) - np.repeat(z, g, 0).astype(np.int32)).astype(np.float32) * np.repeat(s.astype(np.float32), g, 0)
    assert np.array_equal(W, W_np)
    x = rng.standard_normal((3, K)).astype(np.float32)
    want = x.astype(np.float64) @ W.astype(np.float64)
    assert rel_err(oracle.gemv_f32(x, W), want) <= 1e-6
    assert np.array_equal(oracle.awq_gemv(x, qw, qz, s.view(np.uint16)), oracle.gemv_f32(x, W))
    assert rel_err(oracle.gemv_f32(x, W, acc_double=False), want) <= 1e-5
    # the fp16-operand variant rounds x only
    x16 = x.astype(np.float16).astype(np.float32)
    assert np.array_equal(oracle.awq_gemv(x, qw, qz, s.view(np.uint16), act_round=oracle.ROUND_FP16),
                          oracle.awq_gemv(x16, qw, qz, s.view(np.uint16)))


def test_oracle_quantiser_round_trip(oracle):
    rng = np.random.default_rng(2)
    W = (rng.standard_normal((256, 64)) * 0.02).astype(np.float32)
    qw, qz, s = oracle.awq_quantize(W)
    Wd = oracle.awq_dequant(qw, qz, s)
    step = s.view(np.float16).astype(np.float32).max()
    assert np.abs(Wd - W).max() <= 0.51 * step + 1e-6  # at most half a quantisation step (+ zero-point rounding)
    assert qw.shape == (256, 8) and qz.shape == (2, 8) and s.shape == (2, 64)


def test_oracle_attention_against_numpy(oracle):
    rng = np.random.default_rng(3)
    M, Nq, Nkv, D, S = 2, 4, 2, 128, 40
    q = rng.standard_normal((M, Nq, D)).astype(np.float32)
    kc = oracle.f32_to_bf16(rng.standard_normal((2, Nkv, S, D)).astype(np.float32))
    vc = oracle.f32_to_bf16(rng.standard_normal((2, Nkv, S, D)).astype(np.float32))
    seq, slot = np.array([17, 40], np.int32), np.array([1, 0], np.int32)
    out = oracle.attention(q, kc, vc, seq, slot)
    kf, vf = oracle.bf16_to_f32(kc).astype(np.float64), oracle.bf16_to_f32(vc).astype(np.float64)
    for m in range(M):
        for h in range(Nq):
            k, v = kf[slot[m], h // 2, :seq[m]], vf[slot[m], h // 2, :seq[m]]
            sc = k @ q[m, h].astype(np.float64) / np.sqrt(D)
            p = np.exp(sc - sc.max())
            want = (p / p.sum()) @ v
            assert np.abs(out[m, h] - want).max() <= 1e-5
    empty = oracle.attention(q, kc, vc, np.zeros(2, np.int32), slot)
    assert np.all(empty == 0)


def test_oracle_decoder_matches_transformers_fixture(oracle):
    """Independent cross-check of the block semantics (fixture made by tests/golden/make_golden.py from the
    `transformers` Qwen3 model on the dequantised weights).  The only modelling difference is the oracle's bf16 KV
    cache, hence the 5e-3 band; a wrong rotary pairing, norm placement or head mapping is an O(1) error."""
    g = np.load(os.path.join(GOLDEN, "qwen3_tiny_hf.npz"))
    cfg = oracle.ModelConfig(n_layers=2, hidden=128, n_q_heads=2, n_kv_heads=1, head_dim=128, inter=256, vocab=512,
                             max_seq=32, max_batch=1)
    layers = [{k: np.ascontiguousarray(g[f"layer{l}.{k}"]) for k in oracle.LAYER_FIELDS} for l in range(2)]
    weights = {"embed": np.ascontiguousarray(g["embed"]), "lm_head": np.ascontiguousarray(g["lm_head"]),
               "final_norm": np.ascontiguousarray(g["final_norm"]), "layers": layers}
    model = oracle.OracleModel(cfg, weights)
    n = len(g["prompt"])
    lg, nx = model.forward(g["prompt"], np.arange(n, dtype=np.int32))
    assert rel_err(lg, g["prompt_logits"]) <= 5e-3
    for i, tok in enumerate(g["step_tokens"]):
        lg, nx = model.forward([int(tok)], [n + i])
        assert rel_err(lg[0], g["step_logits"][i]) <= 5e-3
    assert int(g["step_tokens"][0]) == int(np.argmax(g["prompt_logits"][-1]))


def test_oracle_decoder_chunking_is_exact(oracle):
    cfg = oracle.ModelConfig(n_layers=2, hidden=256, n_q_heads=4, n_kv_heads=2, head_dim=128, inter=512, vocab=300,
                             max_seq=32, max_batch=2)
    w = make_model_weights(oracle, cfg, seed=4)
    toks = np.array([5, 6, 7, 8, 9, 10, 11], np.int32)
    one = oracle.OracleModel(cfg, w)
    lg_all, _ = one.forward(toks, np.arange(7, dtype=np.int32))
    two = oracle.OracleModel(cfg, w)
    two.forward(toks[:3], np.arange(3, dtype=np.int32))
    lg_tail, _ = two.forward(toks[3:], np.arange(3, 7, dtype=np.int32))
    assert np.array_equal(lg_tail, lg_all[3:])
    lg_last, nx_last = one.forward(toks, np.arange(7, dtype=np.int32), logit_rows=1)
    assert np.array_equal(lg_last[0], lg_all[-1])


# ----------------------------------------------------------------------------- C ABI and host logic
def _declared(header, macro):
    text = open(os.path.join(ROOT, "include", header)).read()
    # declarations that exist in measurement builds only are not part of the shipped library
    text = re.sub(r"#ifdef KUIPER_TRACE.*?#endif", "", text, flags=re.S)
    return set(re.findall(macro + r"\s+[\w \*]+?(kuiper_\w+)\s*\(", text))


def test_kernel_library_exports_every_declared_symbol():
    from mykuiperllama_b200 import _lib
    lib = _lib.kernels()  # loads without a GPU
    names = _declared("kuiper_b200.h", "KUIPER_API")
    assert names == set(_lib.KERNEL_API), names ^ set(_lib.KERNEL_API)
    for n in names:
        assert getattr(lib, n) is not None
    assert lib.kuiper_version().startswith(b"kuiper_b200")
    assert lib.kuiper_awq_gemv_workspace_bytes(1, 4096, 4096) > 0
    assert lib.kuiper_awq_gemv_workspace_bytes(0, 4096, 4096) == 0


def test_engine_library_exports_every_declared_symbol():
    from mykuiperllama_b200 import _lib
    lib = _lib.host()
    names = _declared("kuiper_llama.h", "KUIPER_LLAMA_API")
    assert names == set(_lib.HOST_API), names ^ set(_lib.HOST_API)
    for n in names:
        assert getattr(lib, n) is not None


def test_kernel_argument_validation_needs_no_gpu():
    # invalid arguments are rejected on the host, before any CUDA call
    from mykuiperllama_b200 import _lib
    lib = _lib.kernels()
    assert lib.kuiper_add_f32(None, None, None, 10, None) == 7
    assert b"null" in lib.kuiper_last_error()
    assert lib.kuiper_awq_gemv_f32(1, 1, 1, 1, 1, None, 1, 100, 64, 128, 1, None, 0, None) == 7  # K % 128 != 0
    assert lib.kuiper_awq_gemv_f32(1, 1, 1, 1, 1, None, 1, 128, 64, 64, 1, None, 0, None) == 7   # group != 128
    assert lib.kuiper_flash_decode(1, 1, 1, 1, 1, 1, 1, 6, 4, 128, 64, 1, -1, None, 0, None) == 7   # Nq % Nkv != 0
    assert lib.kuiper_bf16_gemv_f32(1, 1, 1, 1, 10, 4, None) == 7                                 # K % 8 != 0


def test_host_selftest_cpu_part():
    from mykuiperllama_b200 import _lib
    buf = C.create_string_buffer(16384)
    failed = _lib.host().kuiper_selftest(0, buf, 16384)
    assert failed == 0, buf.value.decode()
    assert b"checks passed" in buf.value


def test_model_create_fails_loudly_without_gpu_or_with_bad_config():
    import torch
    from mykuiperllama_b200 import engine
    bad = engine.EngineConfig(n_layers=1, hidden=128, n_q_heads=3, n_kv_heads=2, head_dim=128, inter=128, vocab=16)
    with pytest.raises(RuntimeError):
        engine.Qwen3Engine(bad)  # heads do not divide
    if not torch.cuda.is_available():
        ok = engine.EngineConfig(n_layers=1, hidden=128, n_q_heads=2, n_kv_heads=1, head_dim=128, inter=128, vocab=16)
        with pytest.raises(BaseException):
            engine.Qwen3Engine(ok)  # no CUDA device: no fallback path exists


def test_bench_accounting():
    sys.path.insert(0, ROOT)
    import bench
    # algorithmic bytes of the single-GEMV workload: 2 097 152 + 65 536 + 16 384
    assert bench.int4_bytes(2048, 2048) == 2097152 + 65536 + 16384
    cfg8 = bench.WORKLOADS["c5"][0]
    w = bench.token_bytes(cfg8, 0)
    assert abs(w - 4853827584) / 4853827584 < 2e-3  # all weights once per token (norm vectors included)
    assert bench.token_bytes(cfg8, 2560) - w == 147456 * 2560


# ----------------------------------------------------------------------------- tensor-parallel sharding (gloo, 2 ranks)
_TP_WORKER = r"""
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "tests"))
from helpers import make_model_weights, rel_err
from oracle import cpu_oracle as orc
from tp_reference import shard_layer

dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
cfg = orc.ModelConfig(n_layers=1, hidden=256, n_q_heads=4, n_kv_heads=2, head_dim=128, inter=512, vocab=64, max_seq=8, max_batch=1)
w = make_model_weights(orc, cfg, seed=9)["layers"][0]
rng = np.random.default_rng(10)
h = rng.standard_normal((1, 256)).astype(np.float32)
xn = rng.standard_normal((1, 256)).astype(np.float32)
att_full = rng.standard_normal((1, 512)).astype(np.float32)
act_full = rng.standard_normal((1, 512)).astype(np.float32)

sh = shard_layer(w, cfg, rank, world)
Hq, Hkv, D, I = cfg.n_q_heads // world, cfg.n_kv_heads // world, 128, cfg.inter // world
# column-split projections give this rank's slice of the full output
qkv_full = orc.awq_gemv(xn, w["qkv_qw"], w["qkv_qz"], w["qkv_s"])
qkv_loc = orc.awq_gemv(xn, sh["qkv_qw"], sh["qkv_qz"], sh["qkv_s"])
want = np.concatenate([qkv_full[:, rank*Hq*D:(rank+1)*Hq*D],
                       qkv_full[:, 4*D + rank*Hkv*D: 4*D + (rank+1)*Hkv*D],
                       qkv_full[:, 6*D + rank*Hkv*D: 6*D + (rank+1)*Hkv*D]], 1)
assert np.array_equal(qkv_loc, want)
gu_full = orc.awq_gemv(xn, w["gu_qw"], w["gu_qz"], w["gu_s"])
gu_loc = orc.awq_gemv(xn, sh["gu_qw"], sh["gu_qz"], sh["gu_s"])
assert np.array_equal(gu_loc, np.concatenate([gu_full[:, rank*I:(rank+1)*I], gu_full[:, 512 + rank*I: 512 + (rank+1)*I]], 1))
# row-split projections: partial sums, residual folded in on rank 0 only, one all-reduce
for name, x_full, width in (("o", att_full, Hq * D), ("down", act_full, I)):
    part = orc.awq_gemv(x_full[:, rank*width:(rank+1)*width], sh[name+"_qw"], sh[name+"_qz"], sh[name+"_s"])
    if rank == 0:
        part = part + h
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)
    full = h + orc.awq_gemv(x_full, w[name+"_qw"], w[name+"_qz"], w[name+"_s"])
    assert rel_err(t.numpy(), full) <= 1e-6, name
dist.barrier()
dist.destroy_process_group()
sys.stdout.write("rank%d-ok\n" % rank)
"""


def test_tensor_parallel_sharding_two_gloo_ranks(tmp_path, oracle):
    script = tmp_path / "tp_worker.py"
    script.write_text(_TP_WORKER.format(root=ROOT))
    env = dict(os.environ, OMP_NUM_THREADS="2")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)],
                         capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "rank0-ok" in res.stdout and "rank1-ok" in res.stdout


def test_python_front_ends_import_without_a_gpu():
    # the torch-tensor front end of the kernel ABI and the engine wrapper are importable on a CPU-only host
    # (they only fail, loudly, when a kernel is called)
    import importlib
    for name in ("mykuiperllama_b200.capi", "mykuiperllama_b200.engine"):
        importlib.import_module(name)


# ----------------------------------------------------------------------------- checkpoint container (host only)
def test_safetensors_header_is_parsed_and_checked(oracle, tmp_path):
    import ctypes as C
    import struct
    from helpers import checkpoint_tensors, make_model_weights, write_safetensors
    from mykuiperllama_b200 import _lib
    lib = _lib.host()
    cfg = oracle.ModelConfig(n_layers=1, hidden=256, n_q_heads=4, n_kv_heads=2, head_dim=128, inter=512, vocab=64, max_seq=8, max_batch=1)
    tensors = checkpoint_tensors(cfg, make_model_weights(oracle, cfg, seed=2))
    path = str(tmp_path / "tiny.safetensors")
    write_safetensors(path, tensors, metadata={"format": "pt", "note": "a \"quoted\" value"})
    buf = C.create_string_buffer(1 << 16)
    assert lib.kuiper_checkpoint_inspect(path.encode(), buf, len(buf)) == 0
    lines = buf.value.decode().splitlines()
    assert "model.layers.0.self_attn.q_proj.qweight I32 [256,64] 65536" in lines
    assert "model.layers.0.mlp.down_proj.scales F16 [4,256] 2048" in lines
    assert "model.embed_tokens.weight BF16 [64,256] 32768" in lines
    assert "__metadata__ format=pt" in lines
    assert len([l for l in lines if not l.startswith("__metadata__")]) == len(tensors)
    # malformed files are refused with a parse error (3) or a path error (2), never read out of bounds
    raw = open(path, "rb").read()
    cases = {
        "missing": None,
        "short": raw[:5],
        "header_too_long": struct.pack("<Q", len(raw)) + raw[8:],
        "truncated_data": raw[:-100],
        "bad_json": raw[:8] + b"{" + b"x" * (struct.unpack("<Q", raw[:8])[0] - 1) + raw[8 + struct.unpack("<Q", raw[:8])[0]:],
    }
    for name, blob in cases.items():
        bad = str(tmp_path / (name + ".safetensors"))
        if blob is not None:
            open(bad, "wb").write(blob)
        rc = lib.kuiper_checkpoint_inspect(bad.encode(), buf, len(buf))
        assert rc in (2, 3), (name, rc)
        assert lib.kuiper_llama_last_error()
