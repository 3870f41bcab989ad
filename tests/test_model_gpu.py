"""The C++ engine (Model::forward / predict, CUDA-graph decode loop) against the CPU oracle decoder."""
import ctypes as C

import numpy as np
import pytest

from helpers import make_model_weights, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def engine_mod(cuda):
    from mykuiperllama_b200 import engine
    return engine


def _mirror(oracle, act_mode):
    """The oracle's operand rounding that mirrors an engine created with this act_mode."""
    return {0: oracle.ROUND_NONE, 1: oracle.ROUND_FP16, 2: oracle.ROUND_ENGINE}[act_mode]


def _pair(oracle, engine_mod, cfg_kwargs, seed, act_mode=1):
    ocfg = oracle.ModelConfig(**cfg_kwargs, act_round=_mirror(oracle, act_mode))
    weights = make_model_weights(oracle, ocfg, seed=seed)
    ref = oracle.OracleModel(ocfg, weights)
    ecfg = engine_mod.EngineConfig(**cfg_kwargs, max_rows=8, act_mode=act_mode)
    eng = engine_mod.Qwen3Engine(ecfg)
    eng.load(weights)
    return ref, eng, weights


TINY = dict(n_layers=2, hidden=256, n_q_heads=4, n_kv_heads=2, head_dim=128, inter=512, vocab=1000, max_seq=64, max_batch=2)


def test_selftest_with_cuda(cuda):
    from mykuiperllama_b200._lib import host
    buf = C.create_string_buffer(16384)
    failed = host().kuiper_selftest(1, buf, 16384)
    assert failed == 0, buf.value.decode()


@pytest.mark.parametrize("act_mode", [2, 1, 0])
def test_tiny_model_logits_and_tokens(oracle, engine_mod, act_mode):
    ref, eng, _ = _pair(oracle, engine_mod, TINY, seed=1, act_mode=act_mode)
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, 1000, 5).astype(np.int32)
    pos = np.arange(5, dtype=np.int32)
    lg_ref, nx_ref = ref.forward(prompt, pos)
    lg, nx = eng.predict(prompt, pos, want_logits=True)
    # fp32 everywhere except the mirrored fp16 rounding of the INT4 matmul operand: what is left is the
    # summation order plus the rare operand whose fp16 rounding flips because of it (2^-11 of one element)
    assert rel_err(lg, lg_ref) <= 2e-3
    assert np.array_equal(nx, nx_ref)
    # a second sequence in slot 1 must not disturb slot 0
    other = rng.integers(0, 1000, 3).astype(np.int32)
    ref.forward(other, np.arange(3, dtype=np.int32), np.ones(3, np.int32))
    eng.predict(other, np.arange(3, dtype=np.int32), np.ones(3, np.int32))
    tok = int(nx[-1])
    for step in range(6):
        lg_ref, nx_ref = ref.forward([tok], [5 + step])
        lg, nx = eng.predict([tok], [5 + step], want_logits=True)
        assert rel_err(lg, lg_ref) <= 2e-3
        assert nx[0] == nx_ref[0]
        tok = int(nx[0])
    # the unrounded oracle is the workload's stated reference: within 1e-2
    ocfg = oracle.ModelConfig(**TINY, act_round=oracle.ROUND_NONE)
    plain = oracle.OracleModel(ocfg, ref._keep)
    lg_plain, _ = plain.forward(prompt, pos)
    lg_again, _ = eng.predict(prompt, pos, want_logits=True)
    assert rel_err(lg_again, lg_plain) <= 1e-2


@pytest.mark.parametrize("act_mode", [2, 1])
def test_prefill_and_graph_decode_match_oracle_greedy(oracle, engine_mod, act_mode):
    ref, eng, _ = _pair(oracle, engine_mod, TINY, seed=3, act_mode=act_mode)
    rng = np.random.default_rng(4)
    prompt = rng.integers(0, 1000, 19).astype(np.int32)  # 19 = two full chunks of 8 + a ragged one
    _, nx_ref = ref.forward(prompt, np.arange(19, dtype=np.int32))
    first = eng.prefill(prompt, slot=0)
    assert first == nx_ref[-1]
    # oracle greedy stream
    want, tok = [], int(nx_ref[-1])
    for i in range(24):
        _, nx = ref.forward([tok], [19 + i])
        want.append(int(nx[0]))
        tok = int(nx[0])
    # device-resident loop: no host interaction between steps
    eng.decode_begin([first], [19], [0])
    got = []
    for i in range(24):
        eng.decode_step(1)
        got.append(int(eng.decode_read(1)[0]))
    assert got == want
    assert eng.kernels_per_step > 0


def test_decode_predict_end_to_end_path(oracle, engine_mod):
    ref, eng, _ = _pair(oracle, engine_mod, TINY, seed=5, act_mode=2)
    prompt = np.array([3, 1, 4, 1, 5, 9, 2, 6], np.int32)
    _, nx_ref = ref.forward(prompt, np.arange(8, dtype=np.int32))
    first = eng.prefill(prompt)
    assert first == nx_ref[-1]
    eng.decode_begin([first], [8], [0])
    tok = first
    for i in range(10):
        _, nx = ref.forward([tok], [8 + i])
        got = eng.decode_predict([tok])
        assert got[0] == nx[0]
        tok = int(nx[0])


def test_batched_decode_two_sequences(oracle, engine_mod):
    ref, eng, _ = _pair(oracle, engine_mod, TINY, seed=6)
    p0 = np.array([7, 8, 9, 10, 11], np.int32)
    p1 = np.array([100, 200, 300], np.int32)
    _, n0 = ref.forward(p0, np.arange(5, dtype=np.int32), np.zeros(5, np.int32))
    _, n1 = ref.forward(p1, np.arange(3, dtype=np.int32), np.ones(3, np.int32))
    f0 = eng.prefill(p0, slot=0)
    f1 = eng.prefill(p1, slot=1)
    assert (f0, f1) == (n0[-1], n1[-1])
    toks, pos = np.array([f0, f1], np.int32), np.array([5, 3], np.int32)
    eng.decode_begin(toks, pos, [0, 1])
    for i in range(8):
        _, nx = ref.forward(toks, pos + i, np.array([0, 1], np.int32))
        eng.decode_step(1)
        got = eng.decode_read(2)
        assert np.array_equal(got, nx)
        toks = nx


def test_engine_rejects_bad_requests(oracle, engine_mod):
    from mykuiperllama_b200._lib import KuiperError
    _, eng, _ = _pair(oracle, engine_mod, TINY, seed=7)
    with pytest.raises(KuiperError) as e:
        eng.predict([1000], [0])  # token id == vocab
    assert e.value.code == 7
    with pytest.raises(KuiperError) as e:
        eng.predict([1], [64])  # position == max_seq
    assert e.value.code == 7
    with pytest.raises(KuiperError):
        eng.predict(np.zeros(9, np.int32), np.arange(9))  # more rows than max_rows
    with pytest.raises(RuntimeError):
        engine_mod.Qwen3Engine(engine_mod.EngineConfig(**{**TINY, "head_dim": 64}))


def test_passes_of_64_rows_or_more_use_the_tensor_core_gemm(oracle, engine_mod):
    """M >= 64 rows switch the INT4 projections to the tcgen05 GEMM (fp16 weights in the product): logits stay
    within the fp16 weight rounding of the oracle, and a chunked prefill (96 + 4 rows) hands the same cache to decode."""
    cfg = {**TINY, "max_seq": 128}
    ocfg = oracle.ModelConfig(**cfg, act_round=oracle.ROUND_FP16)
    weights = make_model_weights(oracle, ocfg, seed=5)
    ref = oracle.OracleModel(ocfg, weights)
    eng = engine_mod.Qwen3Engine(engine_mod.EngineConfig(**cfg, max_rows=96, act_mode=1))
    eng.load(weights)
    rng = np.random.default_rng(6)
    rows = rng.integers(0, 1000, 70).astype(np.int32)
    pos = np.arange(70, dtype=np.int32)
    lg_ref, nx_ref = ref.forward(rows, pos)
    lg, nx = eng.predict(rows, pos, want_logits=True)
    assert rel_err(lg, lg_ref) <= 5e-3
    assert np.mean(nx == nx_ref) >= 0.9  # near-ties may flip under the extra rounding
    prompt = rng.integers(0, 1000, 100).astype(np.int32)
    lg_ref, nx_ref = ref.forward(prompt, np.arange(100, dtype=np.int32), np.ones(100, np.int32))
    first = eng.prefill(prompt, slot=1)
    lg_ref1, nx_ref1 = ref.forward([first], [100], [1])
    lg1, nx1 = eng.predict([first], [100], [1], want_logits=True)
    assert rel_err(lg1, lg_ref1) <= 5e-3
    from mykuiperllama_b200 import capi
    capi.awq_gemm_status()


@pytest.mark.parametrize("act_mode", [2, 1])
def test_qwen3_0p6b_shape_greedy_identity_32_tokens(oracle, engine_mod, act_mode):
    """Config 2 of the workload: Qwen3-0.6B shape, random init, 64-token prompt, greedy tokens identical
    to the oracle's for the first 32 decode steps."""
    cfg = dict(n_layers=28, hidden=1024, n_q_heads=16, n_kv_heads=8, head_dim=128, inter=3072, vocab=151936,
               max_seq=128, max_batch=1)
    ref, eng, _ = _pair(oracle, engine_mod, cfg, seed=0, act_mode=act_mode)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, 151936, 64).astype(np.int32)
    _, nx_ref = ref.forward(prompt, np.arange(64, dtype=np.int32), logit_rows=1)
    first = eng.prefill(prompt)
    assert first == nx_ref[-1]
    eng.decode_begin([first], [64], [0])
    tok, margins = int(first), []
    for i in range(32):
        lg, nx = ref.forward([tok], [64 + i])
        top2 = np.partition(lg[0], -2)[-2:]
        margins.append(float(top2[1] - top2[0]))
        eng.decode_step(1)
        got = int(eng.decode_read(1)[0])
        assert got == nx[0], f"step {i}: engine {got} oracle {nx[0]} (oracle top-1/top-2 margin {margins[-1]:.3e})"
        tok = int(nx[0])
    print("oracle top-1/top-2 logit margins: min %.3e median %.3e" % (min(margins), float(np.median(margins))))


@pytest.mark.parametrize("name,shape", [
    ("qwen3-4b", dict(hidden=2560, n_q_heads=32, n_kv_heads=8, inter=9728)),
    ("qwen3-8b", dict(hidden=4096, n_q_heads=32, n_kv_heads=8, inter=12288)),
])
@pytest.mark.parametrize("act_mode", [2, 1])
def test_two_layer_cuts_of_the_4b_and_8b_shapes_match_oracle(oracle, engine_mod, name, shape, act_mode):
    """Layer widths and the full vocabulary of the Qwen3-4B / 8B shapes, cut to two layers so that the CPU oracle
    finishes in seconds: prompt logits within tolerance and the 32 greedy tokens after it identical."""
    cfg = dict(n_layers=2, head_dim=128, vocab=151936, max_seq=96, max_batch=1, **shape)
    from helpers import make_model_weights_fast
    ocfg = oracle.ModelConfig(**cfg, act_round=_mirror(oracle, act_mode))
    weights = make_model_weights_fast(oracle, ocfg, seed=11)
    ref = oracle.OracleModel(ocfg, weights)
    eng = engine_mod.Qwen3Engine(engine_mod.EngineConfig(**cfg, max_rows=8, act_mode=act_mode))
    eng.load(weights)
    rng = np.random.default_rng(12)
    prompt = rng.integers(0, 151936, 16).astype(np.int32)
    pos = np.arange(16, dtype=np.int32)
    lg_ref, nx_ref = ref.forward(prompt[:8], pos[:8])
    lg, nx = eng.predict(prompt[:8], pos[:8], want_logits=True)
    assert rel_err(lg, lg_ref) <= 2e-3                      # mirrored operand rounding: summation order is what is left
    plain = oracle.OracleModel(oracle.ModelConfig(**cfg, act_round=oracle.ROUND_NONE), weights)
    lg_plain, _ = plain.forward(prompt[:8], pos[:8])
    assert rel_err(lg, lg_plain) <= 1e-2                    # the workload's bound, against the un-rounded oracle
    _, nx_ref = ref.forward(prompt, pos, logit_rows=1)      # rewrites rows 0..7 with the same values
    first = eng.prefill(prompt)
    assert first == nx_ref[-1]
    eng.decode_begin([first], [16], [0])
    tok, margins = int(first), []
    for i in range(32):
        lg_ref, nx = ref.forward([tok], [16 + i])
        top2 = np.partition(lg_ref[0], -2)[-2:]
        margins.append(float(top2[1] - top2[0]))
        eng.decode_step(1)
        got = int(eng.decode_read(1)[0])
        assert got == nx[0], f"{name} step {i}: engine {got} oracle {nx[0]} (oracle top-1/top-2 margin {margins[-1]:.3e})"
        tok = int(nx[0])
    print("%s cut: oracle top-1/top-2 logit margins: min %.3e median %.3e" % (name, min(margins), float(np.median(margins))))
    eng.close()


def test_checkpoint_file_round_trip_reproduces_the_greedy_stream(oracle, engine_mod, tmp_path):
    """The synthetic model written as an AWQ checkpoint (safetensors container, Hugging Face tensor names, separate
    q / k / v and gate / up projections), loaded through the file reader: the 32 greedy tokens of the in-memory
    engine and of the oracle."""
    from helpers import checkpoint_tensors, write_safetensors
    cfg = {**TINY, "max_seq": 96}
    ocfg = oracle.ModelConfig(**cfg, act_round=oracle.ROUND_ENGINE)
    weights = make_model_weights(oracle, ocfg, seed=9)
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, checkpoint_tensors(ocfg, weights), metadata={"format": "pt"})
    ref = oracle.OracleModel(ocfg, weights)
    from_file = engine_mod.Qwen3Engine(engine_mod.EngineConfig(**cfg, max_rows=8, act_mode=2))
    from_file.load_checkpoint(path)
    in_memory = engine_mod.Qwen3Engine(engine_mod.EngineConfig(**cfg, max_rows=8, act_mode=2))
    in_memory.load(weights)
    prompt = np.random.default_rng(10).integers(0, 1000, 11).astype(np.int32)
    _, nx_ref = ref.forward(prompt, np.arange(11, dtype=np.int32), logit_rows=1)
    streams = []
    for eng in (from_file, in_memory):
        first = eng.prefill(prompt)
        assert first == nx_ref[-1]
        eng.decode_begin([first], [11], [0])
        got = []
        for _ in range(32):
            eng.decode_step(1)
            got.append(int(eng.decode_read(1)[0]))
        streams.append(got)
    assert streams[0] == streams[1]
    tok, want = int(nx_ref[-1]), []
    for i in range(32):
        _, nx = ref.forward([tok], [11 + i])
        want.append(int(nx[0]))
        tok = int(nx[0])
    assert streams[0] == want
    # a file that lacks a tensor is refused with a parse error naming it
    from mykuiperllama_b200._lib import KuiperError
    tensors = checkpoint_tensors(ocfg, weights)
    del tensors["model.layers.1.mlp.up_proj.qzeros"]
    write_safetensors(str(tmp_path / "broken.safetensors"), tensors)
    with pytest.raises(KuiperError) as e:
        from_file.load_checkpoint(str(tmp_path / "broken.safetensors"))
    assert e.value.code == 3 and "up_proj" in str(e.value)
