#!/usr/bin/env python
"""Decode-throughput benchmark of the B200 engine.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c5|c4|c2] [--impl reference]

Default workload: config "Qwen3-8B-shaped INT4-AWQ decode, batch 1, 2048-token prompt" of the
workload list (the one the tokens/s target is quoted on); a step is one greedy decode token.
Weights are random-init N(0, 0.02) quantised to INT4-AWQ g128 (synthetic data).

  value      decode tokens/s with everything resident in HBM (CUDA-graph loop, device timed)
  e2e        the same through Model::decode_predict with host token ids in / out every step
  roofline   the INT4-AWQ GEMV launches of one token, timed alone with CUDA events
  cpu_baseline  the CPU oracle's decoder timed on the host cores on a bounded sample

With --gpus N (under torch.distributed.run) the model is tensor-parallel over N ranks.
--impl reference times the CPU oracle (the reference has no implementation of this path to run).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (config kwargs, prompt length, decode tokens of the workload, batch)
    "c2": (dict(n_layers=28, hidden=1024, n_q_heads=16, n_kv_heads=8, head_dim=128, inter=3072, vocab=151936), 64, 256, 1,
           "qwen3-0.6b-shape int4-awq g128, batch 1, 64-token prompt"),
    "c4": (dict(n_layers=36, hidden=2560, n_q_heads=32, n_kv_heads=8, head_dim=128, inter=9728, vocab=151936), 512, 512, 1,
           "qwen3-4b-shape int4-awq g128, batch 1, 512-token prompt"),
    "c5": (dict(n_layers=36, hidden=4096, n_q_heads=32, n_kv_heads=8, head_dim=128, inter=12288, vocab=151936), 2048, 1024, 1,
           "qwen3-8b-shape int4-awq g128, batch 1, 2048-token prompt"),
}
AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)
NOMINAL_HBM_GBS = 8000.0
NCU_TRAFFIC_RATIO = 1.002  # dram__bytes_read + write over algorithmic bytes, INT4 GEMV, from the committed ncu summary


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def int4_bytes(K, N, g=128):
    return K * N // 2 + (K // g) * N * 2 + (K // g) * N // 2


def layer_shapes(cfg, tp=1):
    H, D = cfg["hidden"], cfg["head_dim"]
    Hq, Hkv, I = cfg["n_q_heads"] // tp, cfg["n_kv_heads"] // tp, cfg["inter"] // tp
    return {"qkv": (H, (Hq + 2 * Hkv) * D), "o": (Hq * D, H), "gu": (H, 2 * I), "down": (I, H)}


def token_bytes(cfg, ctx, batch=1):
    """Algorithmic HBM bytes of one decode step: every weight once + the KV rows read."""
    w = cfg["n_layers"] * sum(int4_bytes(K, N) for K, N in layer_shapes(cfg).values())
    w += cfg["vocab"] * cfg["hidden"] * 2 + (2 * cfg["n_layers"] + 1) * cfg["hidden"] * 2
    kv = cfg["n_layers"] * 2 * cfg["n_kv_heads"] * cfg["head_dim"] * 2 * ctx * batch
    return w + kv


# --------------------------------------------------------------------------- synthetic weights
def quantize_awq_torch(W, g=128):
    """Harness quantiser (per group/column min-max, 4 bit), same rule as the oracle's orc_awq_quantize."""
    import torch
    K, N = W.shape
    Wg = W.view(K // g, g, N)
    mn, mx = Wg.amin(1), Wg.amax(1)
    s16 = ((mx - mn) / 15.0).clamp_min(1e-8).half()
    s = s16.float()
    z = torch.round(-mn / s).clamp_(0, 15)
    q = (torch.round(Wg / s[:, None, :]) + z[:, None, :]).clamp_(0, 15).to(torch.int64).view(K, N)

    def pack(v):
        rows = v.shape[0]
        v = v.view(rows, N // 8, 8)
        w = torch.zeros((rows, N // 8), dtype=torch.int64, device=v.device)
        for i, o in enumerate(AWQ_ORDER):
            w |= v[:, :, o] << (4 * i)
        return ((w + 2 ** 31) % 2 ** 32 - 2 ** 31).to(torch.int32).contiguous()

    return pack(q), pack(z.to(torch.int64)), s16.contiguous()


def make_layer_torch(cfg, gen, device):
    import torch
    H, D = cfg["hidden"], cfg["head_dim"]
    lw = {}
    for name, n in (("input_norm", H), ("post_norm", H), ("q_norm", D), ("k_norm", D)):
        lw[name] = (1.0 + 0.02 * torch.randn(n, generator=gen, device=device)).bfloat16()
    for name, (K, N) in layer_shapes(cfg).items():
        W = torch.randn((K, N), generator=gen, device=device) * 0.02
        lw[f"{name}_qw"], lw[f"{name}_qz"], lw[f"{name}_s"] = quantize_awq_torch(W)
        del W
    return lw


def make_globals_torch(cfg, gen, device):
    import torch
    V, H = cfg["vocab"], cfg["hidden"]
    embed = (torch.randn((V, H), generator=gen, device=device) * 0.02).bfloat16()
    lm_head = (torch.randn((V, H), generator=gen, device=device) * 0.02).bfloat16()
    final_norm = (1.0 + 0.02 * torch.randn(H, generator=gen, device=device)).bfloat16()
    return embed, final_norm, lm_head


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """nvidia-smi samples (SM clock, throttle reasons) taken while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index, self.samples, self._stop, self._t = gpu_index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                      "-i", str(self.gpu_index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        mhz = sorted(float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit())
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        mx = [float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit()]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


# --------------------------------------------------------------------------- CPU oracle timing
def make_cpu_weights(orc, ocfg, seed=0):
    """Cheap synthetic weights for CPU timing: uniform nibbles / zeros, fp16 scales in [0.002, 0.02]
    (the single-GEMV workload's distribution); bf16 tables tiled from a small random block."""
    rng = np.random.default_rng(seed)
    H, D, I, V = ocfg.hidden, ocfg.head_dim, ocfg.inter, ocfg.vocab
    QKV = (ocfg.n_q_heads + 2 * ocfg.n_kv_heads) * D

    def quant(K, N):
        qw = rng.integers(-2 ** 31, 2 ** 31, (K, N // 8), dtype=np.int64).astype(np.int32)
        qz = rng.integers(-2 ** 31, 2 ** 31, (K // 128, N // 8), dtype=np.int64).astype(np.int32)
        s = rng.uniform(0.002, 0.02, (K // 128, N)).astype(np.float16).view(np.uint16)
        return qw, qz, s

    def norm(n):
        return orc.f32_to_bf16(np.ones(n, np.float32))

    block = orc.f32_to_bf16((rng.standard_normal((1024, H)) * 0.02).astype(np.float32))
    table = np.ascontiguousarray(np.tile(block, ((V + 1023) // 1024, 1))[:V])
    weights = {"embed": table, "final_norm": norm(H), "lm_head": table, "layers": []}
    for _ in range(ocfg.n_layers):
        lw = {"input_norm": norm(H), "post_norm": norm(H), "q_norm": norm(D), "k_norm": norm(D)}
        for name, (K, N) in {"qkv": (H, QKV), "o": (ocfg.n_q_heads * D, H), "gu": (H, 2 * I), "down": (I, H)}.items():
            lw[f"{name}_qw"], lw[f"{name}_qz"], lw[f"{name}_s"] = quant(K, N)
        weights["layers"].append(lw)
    return weights


def cpu_decode_sample(cfg, n_layers_sample, steps, warmup, seed=0):
    """Times the CPU oracle's decoder (fp32 accumulation, OpenMP over all host cores) on a model
    truncated to n_layers_sample layers and extrapolates to the full depth.  Returns tokens/s."""
    from oracle import cpu_oracle as orc
    orc.build()
    # the launcher may have exported OMP_NUM_THREADS=1 (torch.distributed.run does): the CPU arm takes every core it
    # is allowed to run on regardless
    orc.set_num_threads(host_cores())
    ocfg = orc.ModelConfig(**{**cfg, "n_layers": n_layers_sample}, max_seq=max(64, steps + warmup + 8), max_batch=1,
                           act_round=orc.ROUND_FP16)
    weights = make_cpu_weights(orc, ocfg, seed=seed)
    model = orc.OracleModel(ocfg, weights)
    tok, times = 1, []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        _, nx = model.forward([tok], [i], acc_double=False, want_logits=False)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
        tok = int(nx[0])
    t_step = float(np.mean(times))
    # head (final norm + lm_head + argmax) is paid once per token, layers scale with depth
    t0 = time.perf_counter()
    orc.bf16_gemv(np.ones((1, cfg["hidden"]), np.float32), weights["lm_head"], acc_double=False)
    t_head = time.perf_counter() - t0
    t_layers = max(t_step - t_head, 1e-9) / n_layers_sample
    t_token = t_layers * cfg["n_layers"] + t_head
    return 1.0 / t_token, t_step


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def run_reference(args, cfg, desc, rank, world):
    """Reference arm: the reference ships no code for this path, so its CPU side is the oracle port."""
    if rank != 0:
        return
    n_sample = 2 if cfg["hidden"] >= 2560 else 4
    steps, warmup = max(1, min(args.steps, 12)), max(1, min(args.warmup, 2))
    t0 = time.perf_counter()
    tps, t_step = cpu_decode_sample(cfg, n_sample, steps, warmup)
    sample = (f"{steps} greedy decode tokens (after {warmup} warm-up) of a {n_sample}-layer slice of the model at "
              f"context < 32, fp32 accumulation, OpenMP; per-layer time scaled to {cfg['n_layers']} layers + full lm_head")
    line = {
        "impl": "reference", "metric": "Qwen3 INT4 decode tokens/s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 / tps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int4 weights, fp32 accumulate",
        "data": "synthetic", "config": {"workload": desc, "timed_steps_used": steps},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": host_cores(), "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def gemv_roofline(cfg, tp, layers_kept, iters=3):
    """INT4-AWQ GEMV launches of one token (4 shapes x n_layers), over distinct weights, timed alone.  Every launch
    has its own balance counters, as every layer object of the engine has."""
    import torch
    from mykuiperllama_b200 import capi
    shapes = layer_shapes(cfg, tp)
    x = {n: torch.randn((1, K), device="cuda") for n, (K, N) in shapes.items()}
    y = {n: torch.zeros((1, N), device="cuda") for n, (K, N) in shapes.items()}
    L = cfg["n_layers"]
    tickets = [[capi.awq_gemv_tickets() for _ in range(4)] for _ in range(L)]

    def one_token():
        for l in range(L):
            lw = layers_kept[l % len(layers_kept)]
            for j, n in enumerate(("qkv", "o", "gu", "down")):
                capi.awq_gemv_accum_balanced(x[n], lw[f"{n}_qw"], lw[f"{n}_qz"], lw[f"{n}_s"], y[n], tickets[l][j],
                                             act_mode=capi.ACT_INT16_BLOCK)  # the engine's path

    one_token()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        one_token()
    best = None
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        best = ms if best is None else min(best, ms)
    launches = 4 * L
    total_bytes = L * sum(int4_bytes(K, N) + 4 * K + 4 * N for K, N in shapes.values())
    return total_bytes / launches, best * 1e-3 / launches, launches


def gemv_set(K, N, n, grouped, iters=5, seed=0):
    """One INT4 GEMV shape over n distinct weight sets (more than L2 in total), visited in turn: as n balanced launches
    inside a CUDA graph, or as ONE grouped launch.  Returns (bytes per matrix, seconds per matrix)."""
    import torch
    from mykuiperllama_b200 import capi
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    qw = [torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), dtype=torch.int32, device="cuda", generator=gen) for _ in range(n)]
    qz = [torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 128, N // 8), dtype=torch.int32, device="cuda", generator=gen) for _ in range(n)]
    sc = [(torch.rand((K // 128, N), device="cuda", generator=gen) * 0.018 + 0.002).half() for _ in range(n)]
    x = torch.randn((1, K), device="cuda", generator=gen)
    ys = [torch.zeros((1, N), device="cuda") for _ in range(n)]
    if grouped:
        grp = capi.GemvGroup([dict(x=x, qweight=qw[i], qzeros=qz[i], scales=sc[i], y=ys[i]) for i in range(n)])
        run = grp.run
    else:
        tk = [capi.awq_gemv_tickets() for _ in range(n)]

        def run():
            for i in range(n):
                capi.awq_gemv_accum_balanced(x, qw[i], qz[i], sc[i], ys[i], tk[i], act_mode=capi.ACT_INT16_BLOCK)
    run()
    torch.cuda.synchronize()
    passes = 4  # one pass over the set is short: several of them per timed graph replay
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(passes):
            run()
    g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    per = int4_bytes(K, N) + 4 * K + 4 * N
    return per, float(np.median(times)) * 1e-3 / (n * passes)


def gemv_sub_record(K, N, n, grouped, peak):
    per, sec = gemv_set(K, N, n, grouped)
    gbs = per / sec / 1e9
    return {"shape": f"{K}x{N}", "achieved": gbs, "unit": "GB/s", "frac": gbs / peak, "frac_of_nominal_8TBs": gbs / NOMINAL_HBM_GBS,
            "matrices_visited": n, "us_per_matrix": sec * 1e6, "bytes_per_matrix": per,
            "launch": "one grouped persistent launch over all matrices" if grouped else "one launch per matrix inside a CUDA graph",
            "l2_policy": f"{n} distinct weight sets ({per * n >> 20} MiB) visited in turn: larger than L2"}


def tp1_stream_check(cfg, ecfg, prompt, ids, device):
    """Rank 0 of a tensor-parallel run: the same weights (same seed) on a single-GPU engine, the same prompt, and
    the number of leading greedy tokens on which the two engines agree.  At the first disagreement the single-GPU
    engine's top-1 / top-2 logit margin is reported (a near-tie that the different summation order flipped)."""
    import torch
    from mykuiperllama_b200 import engine as eng_mod
    one = eng_mod.Qwen3Engine(eng_mod.EngineConfig(**{**ecfg.__dict__, "tp_rank": 0, "tp_size": 1, "max_batch": 1}))
    gen = torch.Generator(device=device)
    gen.manual_seed(1234)
    for l in range(cfg["n_layers"]):
        one.load_layer(l, make_layer_torch(cfg, gen, device))
    one.load_globals(*make_globals_torch(cfg, gen, device))
    tok = one.prefill(prompt, slot=0)
    matching, margin, one_margin = 0, None, None
    for i, want in enumerate(ids):
        if tok != want:
            margin = one_margin
            break
        matching += 1
        if i + 1 == len(ids):
            break
        lg, nx = one.predict([tok], [len(prompt) + i], want_logits=True)
        top2 = np.partition(lg[0], -2)[-2:]
        one_margin = float(top2[1] - top2[0])
        tok = int(nx[0])
    one.close()
    del one
    torch.cuda.empty_cache()
    return {"tokens_compared": len(ids), "matching_leading": matching, "tp1_margin_at_first_mismatch": margin}



def _trace_stat(x):
    return "min %.2f  median %.2f  p90 %.2f  max %.2f" % (x.min(), np.median(x), np.percentile(x, 90), x.max())


def print_trace_summary(kind, trace, sm_mhz):
    """Per-CTA timestamps of the measurement build (slot 0: global timer in ns at entry, slot 1: SM clock at entry, other
    slots: SM clock at a milestone, 0 if not reached), summarised on stderr as microseconds since the CTA's entry and on
    a common time axis.  Entries left from earlier launches (more than 30 us before the latest entry) are dropped."""
    names = {"flash": {2: "early fetch issued", 3: "dependency wait passed", 4: "q ready", 5: "rows done",
                       6: "partials visible", 7: "arrival counter answered", 8: "combine done", 9: "exit"},
             "gemv": {8: "first weight unit issued", 6: "activation warp saw first descriptor", 2: "consumers past the wait",
                      7: "first fragments written", 3: "first unit ready", 9: "last weight unit issued",
                      4: "last unit consumed", 5: "consumer exit"}}[kind]
    act = trace[trace[:, 1] != 0]
    if len(act) == 0:
        print(f"[{kind} trace] empty", file=sys.stderr)
        return
    act = act[act[:, 0] >= act[:, 0].max() - 30000]
    t0 = act[:, 0].min()
    per_us = sm_mhz  # SM cycles per microsecond
    print(f"[{kind} trace] {len(act)} CTAs, SM clock {sm_mhz:.0f} MHz; entry spread (us): {_trace_stat((act[:, 0] - t0) / 1e3)}",
          file=sys.stderr)
    for slot, label in names.items():
        w = act[(act[:, slot] > act[:, 1]) & (act[:, slot] < act[:, 1] + 1000 * per_us)]  # older launches' values dropped
        if len(w) == 0:
            continue
        rel = (w[:, slot] - w[:, 1]) / per_us
        print(f"[{kind} trace]   {label:38s} since entry: {_trace_stat(rel)} | common axis: {_trace_stat((w[:, 0] - t0) / 1e3 + rel)}  (n={len(w)})",
              file=sys.stderr)

def run_engine(args, cfg, prompt_len, desc, rank, world):
    import torch
    import torch.distributed as dist
    from mykuiperllama_b200 import engine as eng_mod

    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    B = max(1, args.batch)
    steps_total = args.warmup + args.steps
    n_ids = 32  # greedy ids printed with the line (the first tokens after the prompt, read back step by step)
    max_seq = prompt_len + n_ids + 2 * steps_total + 16
    ecfg = eng_mod.EngineConfig(**cfg, max_seq=max_seq, max_batch=B, max_rows=max(int(os.environ.get('KUIPER_BENCH_MAX_ROWS', '2048')), B), tp_rank=rank, tp_size=world,
                                act_mode=args.act_mode)
    eng = eng_mod.Qwen3Engine(ecfg)

    gen = torch.Generator(device=device)
    gen.manual_seed(1234)  # same weights on every rank
    keep = []
    for l in range(cfg["n_layers"]):
        lw = make_layer_torch(cfg, gen, device)
        eng.load_layer(l, lw)
        if l < 4 and world == 1:
            keep.append(lw)
    embed, final_norm, lm_head = make_globals_torch(cfg, gen, device)
    eng.load_globals(embed, final_norm, lm_head)
    del embed, lm_head, lw
    torch.cuda.empty_cache()

    if world > 1:
        uid = torch.zeros(128, dtype=torch.uint8, device=device)
        if rank == 0:
            uid.copy_(torch.frombuffer(bytearray(eng_mod.Qwen3Engine.tp_unique_id()), dtype=torch.uint8))
        dist.broadcast(uid, 0)
        eng.init_tp(bytes(uid.cpu().numpy().tobytes()))

    rng = np.random.default_rng(7)
    prompt = rng.integers(0, cfg["vocab"], prompt_len).astype(np.int32)
    eng.prefill(prompt, slot=0)  # first use (module load, kernel attributes, NCCL channels) stays out of the prefill time
    eng.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    firsts = [eng.prefill(np.roll(prompt, b), slot=b) for b in range(B)]  # a different prompt per sequence
    prefill_s = time.perf_counter() - t0

    stream = torch.cuda.ExternalStream(eng.stream, device=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- the first n_ids greedy tokens of sequence 0, read back one step at a time: every N prints them, and for
    #      N > 1 rank 0 also runs the single-GPU engine on the same weights and counts the leading tokens that agree
    eng.decode_begin(firsts, [prompt_len] * B, list(range(B)))
    ids = [int(firsts[0])]
    for _ in range(n_ids - 1):
        eng.decode_step(1)
        ids.append(int(eng.decode_read(B)[0]))
    eng.decode_step(1)
    firsts = [int(t) for t in eng.decode_read(B)]
    prompt_tokens = prompt_len
    prompt_len += n_ids
    tp_parity = None
    if world > 1:
        tp_parity = tp1_stream_check(cfg, ecfg, prompt, ids, device) if rank == 0 else None
        barrier()

    # ---- device-resident loop: value
    eng.decode_begin(firsts, [prompt_len] * B, list(range(B)))
    eng.decode_step(args.warmup)
    eng.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        if args.profile_range:
            torch.cuda.profiler.start()  # a profiler started with "profile from start off" sees only the timed steps
        e0.record(stream)
        eng.decode_step(args.steps)
        e1.record(stream)
        eng.synchronize()
        if args.profile_range:
            torch.cuda.profiler.stop()
        barrier()
    if world > 1:
        eng.tp_status()  # raises if a bounded wait of the peer exchange ran out during the timed loop
    if args.flash_trace:
        # measurement build (KUIPER_TRACE=1): per-CTA clock readings of the step's last attention launch
        from mykuiperllama_b200._lib import kernels
        trace = np.zeros((1024, 10), np.int64)
        got = kernels().kuiper_flash_trace_read(trace.ctypes.data, trace.size)
        np.save(args.flash_trace, trace[: max(got, 0) // 10])
        print_trace_summary("flash", trace[: max(got, 0) // 10], clocks.summary().get("sm_mhz") or 1965.0)
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    value = args.steps * B / (ms * 1e-3)
    tok_after = eng.decode_read(B)

    # ---- end to end: host token in, host token out, every step, over the same positions as the device-resident loop
    #      (so that the two numbers differ by the host round trip only, not by the context length)
    eng.decode_begin(firsts, [prompt_len] * B, list(range(B)))
    tok = np.array(firsts, np.int32)
    for _ in range(args.warmup):
        tok = eng.decode_predict(tok)
    barrier()
    t0 = time.perf_counter()
    marks = [t0]
    for _ in range(args.steps):
        tok = eng.decode_predict(tok)
        marks.append(time.perf_counter())
    barrier()
    e2e_s = time.perf_counter() - t0
    per_step_ms = np.diff(np.array(marks)) * 1e3  # spread of the host-side step times (the value uses the whole loop)
    if os.environ.get("KUIPER_BENCH_VERBOSE"):
        print("[e2e] per-step ms:", " ".join("%.3f" % v for v in per_step_ms), file=sys.stderr)
    if world > 1:
        eng.tp_status()
    t = torch.tensor([e2e_s], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = args.steps * B / float(t.item())

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    ctx_mid = prompt_len + args.warmup + args.steps // 2
    peak, peak_kind = measured_peak_gbs()
    step_bytes = token_bytes(cfg, ctx_mid, B) / world  # per GPU under tensor parallelism (the lm_head is split over the vocabulary)
    roof_tps = peak * 1e9 / step_bytes
    line = {
        "metric": "Qwen3 INT4 decode tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": ("int4 weights (AWQ g128), 16-bit block-scaled integer x operand for one-row passes (u8 x s8 mma, exact sums per 32 rows), "
                  "fp16 x operand otherwise, fp32 accumulate") if args.act_mode == 2 else "int4 weights (AWQ g128), fp16 x operand, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": desc if B == 1 else desc.replace("batch 1", f"batch {B}"), "batch": B, "prompt_tokens": prompt_tokens, "context_during_timing": ctx_mid,
                   "parallelism": f"tp{world}", "l2_policy": "inputs larger than L2 (weights streamed once per token)",
                   "prefill_s": round(prefill_s, 3), "greedy_ids_first32": ids, "tp1_stream_check": tp_parity},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B,
                "ms_per_step_min_median_max": [float(per_step_ms.min()), float(np.median(per_step_ms)), float(per_step_ms.max())]},
        "gpu_launches": eng.kernels_per_step * args.steps,
        "clocks": clocks.summary(),
        "decode_roofline": {"bytes_per_token_per_gpu": int(step_bytes), "tokens_per_s_at_peak": roof_tps,
                            "frac_of_" + peak_kind: value / roof_tps,
                            "frac_of_nominal_8TBs": value / (NOMINAL_HBM_GBS * 1e9 / step_bytes)},
    }
    if world == 1:
        per_launch_bytes, per_launch_s, launches = gemv_roofline(cfg, 1, keep)
        achieved = per_launch_bytes / per_launch_s / 1e9
        # DRAM traffic per launch: an ncu capture of the largest shape read 52.45 MB and wrote 0.05 MB for 52.41 MB of
        # algorithmic bytes; traffic grows with the matrix, so the ratio is applied to the average launch of the four
        # shapes timed here
        line["roofline"] = {"bound": "hbm", "kernel": "awq_gemv_mma_kernel<1 row, 3 stages, accumulate, integer operand>", "achieved": achieved, "peak": peak,
                            "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                            "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
                            "traffic": int(per_launch_bytes * NCU_TRAFFIC_RATIO),
                            "traffic_source": "ncu dram bytes / algorithmic bytes = 1.002 on K=4096 N=24576, scaled",
                            "launches_per_token": launches, "avg_bytes_per_launch": int(per_launch_bytes),
                            "avg_us_per_launch": per_launch_s * 1e6}
        del keep
        torch.cuda.empty_cache()
        # the single-GEMV half of the metric: the 2048 x 2048 workload over 256 weight sets (one grouped launch), and the
        # widest projection of this model over 10 weight sets, four passes over the set per timed graph replay
        line["gemv_c1"] = gemv_sub_record(2048, 2048, 256, True, peak)
        torch.cuda.empty_cache()
        Kl, Nl = max(layer_shapes(cfg).values(), key=lambda kn: kn[0] * kn[1])
        line["gemv_largest"] = gemv_sub_record(Kl, Nl, 10, False, peak)
        torch.cuda.empty_cache()
        n_sample = 2 if cfg["hidden"] >= 2560 else 4
        tps_cpu, _ = cpu_decode_sample(cfg, n_sample, steps=3, warmup=1)
        line["cpu_baseline"] = {
            "value": tps_cpu, "unit": "tokens/s", "cores": host_cores(), "kind": "port",
            "sample": f"3 decode tokens of a {n_sample}-layer slice at context < 8 on the CPU oracle (fp32 accumulate, "
                      f"OpenMP), per-layer time scaled to {cfg['n_layers']} layers + full lm_head"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# --------------------------------------------------------------------------- kernel microbenchmarks
def run_gemv_micro(args):
    """INT4-AWQ GEMV alone (config 1 of the workload list and the model-sized shapes): M=1, distinct weight
    matrices totalling more than L2 are visited in turn inside one CUDA graph, so every launch streams from HBM."""
    import torch
    from mykuiperllama_b200 import capi
    torch.cuda.set_device(0)
    K, N = (int(v) for v in args.shape.lower().split("x"))
    if args.gemv_impl is None:
        args.gemv_impl = 2
    if args.gemv_impl in (0, 1):
        capi.set_tuning("gemv_impl", args.gemv_impl)
    if args.gemv_impl == 3:  # the first-generation persistent kernel (SIMT products), accumulate mode
        capi.set_tuning("gemv_impl", 2)
        args.gemv_impl = 2
    per = int4_bytes(K, N) + 4 * K + 4 * N
    n = args.mats or max(2, min(256, (512 << 20) // per))
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    qw = [torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), dtype=torch.int32, device="cuda", generator=gen) for _ in range(n)]
    qz = [torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 128, N // 8), dtype=torch.int32, device="cuda", generator=gen) for _ in range(n)]
    sc = [(torch.rand((K // 128, N), device="cuda", generator=gen) * 0.018 + 0.002).half() for _ in range(n)]
    x = torch.randn((1, K), device="cuda", generator=gen)
    y = torch.zeros((1, N), device="cuda")
    ws = capi.awq_gemv_workspace(1, K, N)
    tk = [capi.awq_gemv_tickets() for _ in range(n)]
    grp = capi.GemvGroup([dict(x=x, qweight=qw[i], qzeros=qz[i], scales=sc[i], y=y) for i in range(n)], act_mode=args.act_mode,
                         balanced=args.group_tickets) if args.gemv_impl == 5 else None

    def sweep():
        if args.gemv_impl == 5:
            grp.run()
            return
        for i in range(n):
            if args.gemv_impl == 2:
                capi.awq_gemv_accum_balanced(x, qw[i], qz[i], sc[i], y, tk[i], act_mode=args.act_mode)
            elif args.gemv_impl == 6:
                capi.awq_gemv_accum_balanced(x, qw[i], qz[i], sc[i], y, None, act_mode=args.act_mode)
            else:
                capi.awq_gemv(x, qw[i], qz[i], sc[i], workspace=ws, out=y)

    for _ in range(args.warmup):
        sweep()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        sweep()
    graph.replay()
    torch.cuda.synchronize()
    times = []
    with ClockSampler(0) as clocks:
        for _ in range(args.steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
    if args.gemv_trace:
        # measurement build (KUIPER_TRACE=1): per-CTA clock readings of the sweep's last launch
        from mykuiperllama_b200._lib import kernels
        trace = np.zeros((304, 10), np.int64)
        kernels().kuiper_gemv_trace_read(trace.ctypes.data, trace.size)
        np.save(args.gemv_trace, trace)
        print_trace_summary("gemv", trace, clocks.summary().get("sm_mhz") or 1965.0)
    ms = float(np.median(times))
    gbs = per * n / (ms * 1e-3) / 1e9
    peak, kind = measured_peak_gbs()
    print(json.dumps({
        "metric": "INT4-AWQ GEMV HBM GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 weights (AWQ g128), fp16 x operand, fp32 accumulate", "data": "synthetic",
        "config": {"workload": f"single INT4-AWQ GEMV M=1 K={K} N={N} g128", "distinct_matrices": n,
                   "l2_policy": f"{n} matrices ({per * n >> 20} MiB) visited in turn: larger than L2"},
        "roofline": {"bound": "hbm", "kernel": "awq_gemv", "achieved": gbs, "peak": peak, "peak_kind": kind, "unit": "GB/s",
                     "frac": gbs / peak, "frac_of_nominal_8TBs": gbs / NOMINAL_HBM_GBS,
                     "traffic": int(per * NCU_TRAFFIC_RATIO) if args.gemv_impl in (2, 5, 6) else None,
                     "avg_us_per_launch": ms * 1e3 / n, "avg_bytes_per_launch": per},
        "gpu_launches": n * args.steps, "clocks": clocks.summary()}), flush=True)


def run_gemm_micro(args):
    """INT4-AWQ GEMM on the tcgen05 tensor cores alone (M >= 16 token rows): distinct weight matrices are visited in
    turn inside one CUDA graph.  Reports TFLOP/s (2*M*K*N per launch) against the measured dense bf16 peak."""
    import torch
    from mykuiperllama_b200 import capi
    torch.cuda.set_device(0)
    K, N = (int(v) for v in args.shape.lower().split("x"))
    M = max(16, args.rows)
    per = int4_bytes(K, N)
    n = args.mats or max(2, min(64, (256 << 20) // per))
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    qw = [torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), dtype=torch.int32, device="cuda", generator=gen) for _ in range(n)]
    qz = [torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 128, N // 8), dtype=torch.int32, device="cuda", generator=gen) for _ in range(n)]
    sc = [(torch.rand((K // 128, N), device="cuda", generator=gen) * 0.018 + 0.002).half() for _ in range(n)]
    x = torch.randn((M, K), device="cuda", generator=gen)
    y = torch.zeros((M, N), device="cuda")
    ws = capi.awq_gemm_workspace(M, K)

    def sweep():
        for i in range(n):
            capi.awq_gemm(x, qw[i], qz[i], sc[i], y=y, workspace=ws)

    for _ in range(args.warmup):
        sweep()
    torch.cuda.synchronize()
    capi.awq_gemm_status()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        sweep()
    graph.replay()
    torch.cuda.synchronize()
    times = []
    with ClockSampler(0) as clocks:
        for _ in range(args.steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
    ms = float(np.median(times))
    tflops = 2.0 * M * K * N * n / (ms * 1e-3) / 1e12
    peak, kind = 1590.0, "fallback"
    try:
        peak, kind = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]), "measured"
    except Exception:
        pass
    print(json.dumps({
        "metric": "INT4-AWQ GEMM TFLOP/s", "value": tflops, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 weights (AWQ g128) dequantised to fp16, fp16 x operand, fp32 accumulate in tensor memory",
        "data": "synthetic",
        "config": {"workload": f"single INT4-AWQ GEMM M={M} K={K} N={N} g128", "distinct_matrices": n,
                   "l2_policy": f"{n} matrices ({per * n >> 20} MiB) visited in turn"},
        "roofline": {"bound": "tensor", "kernel": "awq_gemm_tc_kernel", "achieved": tflops, "peak": peak, "peak_kind": kind,
                     "unit": "TFLOP/s", "frac": tflops / peak, "traffic": None, "avg_us_per_launch": ms * 1e3 / n,
                     "weight_gbs": per * n / (ms * 1e-3) / 1e9},
        "gpu_launches": n * args.steps, "clocks": clocks.summary()}), flush=True)


def run_attn_micro(args):
    """GQA flash-decoding alone (config 3 of the workload list): 32 query heads over 8 KV heads, head_dim 128, bf16
    cache ~N(0,1); distinct caches totalling more than L2 are visited in turn, so the KV rows stream from HBM."""
    import torch
    from mykuiperllama_b200 import capi
    torch.cuda.set_device(0)
    B, L, Nq, Nkv, D = max(1, args.batch), args.kv_len, 32, 8, 128
    kv_bytes = B * 2 * Nkv * L * D * 2
    n = max(2, min(64, (384 << 20) // kv_bytes + 1))
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    kc = [torch.randn((B, Nkv, L, D), device="cuda", generator=gen).bfloat16() for _ in range(n)]
    vc = [torch.randn((B, Nkv, L, D), device="cuda", generator=gen).bfloat16() for _ in range(n)]
    q = torch.randn((B, Nq, D), device="cuda", generator=gen)
    out = torch.empty_like(q)
    seq = torch.full((B,), L, dtype=torch.int32, device="cuda")
    slot = torch.arange(B, dtype=torch.int32, device="cuda")
    ws = capi.flash_decode_workspace(B, Nq, D, L)

    if args.fused:
        # the engine's decode call: q/k-norm + rotary + KV append + attention in one kernel, from a raw projection row
        # (the row is rewritten before every launch because the kernel clears it; that copy is part of the timed graph)
        qkv0 = torch.randn((B, (Nq + 2 * Nkv) * D), device="cuda", generator=gen)
        qkv = qkv0.clone()
        ones = torch.ones(D, device="cuda").bfloat16()
        half = torch.arange(D // 2, device="cuda", dtype=torch.float64)
        ang = torch.arange(L, device="cuda", dtype=torch.float64)[:, None] * torch.pow(torch.tensor(1e6, dtype=torch.float64, device="cuda"), -2.0 * half / D)[None, :]
        cos_t, sin_t = torch.cos(ang).float().contiguous(), torch.sin(ang).float().contiguous()
        pos = torch.full((B,), L - 1, dtype=torch.int32, device="cuda")

        def sweep():
            for i in range(n):
                qkv.copy_(qkv0)
                capi.rope_flash_decode(qkv, ones, ones, cos_t, sin_t, pos, seq, slot, Nq, Nkv, D, 1e-6, kc[i], vc[i], workspace=ws,
                                       out=out, fresh_rows=1, clear_input=True)
    else:
        def sweep():
            for i in range(n):
                capi.flash_decode(q, kc[i], vc[i], seq, slot, workspace=ws, out=out)

    for _ in range(args.warmup):
        sweep()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        sweep()
    graph.replay()
    torch.cuda.synchronize()
    times = []
    with ClockSampler(0) as clocks:
        for _ in range(args.steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
    ms = float(np.median(times))
    gbs = kv_bytes * n / (ms * 1e-3) / 1e9
    peak, kind = measured_peak_gbs()
    print(json.dumps({
        "metric": "GQA flash-decoding KV-read GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 KV cache, bf16 x bf16 -> fp32 mma (q and probabilities as bf16 high + low parts), fp32 softmax", "data": "synthetic",
        "config": {"workload": f"flash-decoding batch {B}, 32 q heads / 8 kv heads, head_dim 128, KV length {L}",
                   "distinct_caches": n, "l2_policy": f"{n} caches ({kv_bytes * n >> 20} MiB) visited in turn: larger than L2"},
        "roofline": {"bound": "hbm", "kernel": "flash_decode_mma_kernel<4 heads per kv head%s>" % (", fused rotary" if args.fused else ""), "achieved": gbs, "peak": peak, "peak_kind": kind,
                     "unit": "GB/s", "frac": gbs / peak, "frac_of_nominal_8TBs": gbs / NOMINAL_HBM_GBS,
                     # an ncu capture at batch 16, 4096 rows: dram bytes / KV bytes = 1.01
                     "traffic": int(kv_bytes * 1.01),
                     "avg_us_per_launch": ms * 1e3 / n, "avg_bytes_per_launch": kv_bytes},
        "gpu_launches": n * args.steps, "clocks": clocks.summary()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--workload", default="c5", choices=sorted(WORKLOADS) + ["gemv", "gemm", "attn"])
    ap.add_argument("--kv-len", type=int, default=4096, help="KV length of the attn microbenchmark")
    ap.add_argument("--shape", default="2048x2048", help="KxN of the gemv microbenchmark")
    ap.add_argument("--rows", type=int, default=2048, help="token rows M of the gemm microbenchmark")
    ap.add_argument("--mats", type=int, default=0, help="distinct weight matrices in the gemv microbenchmark (0 = 512 MiB worth)")
    ap.add_argument("--gemv-impl", type=int, default=None, help="2 accumulate mode of the tensor-core GEMV with ticket balancing (engine path, default), 6 the same dealt statically, "
                         "5 all matrices in one grouped launch, 0 the ordered combine, "
                         "1 register-staged kernel, 3 first-generation persistent SIMT kernel (accumulate)")
    ap.add_argument("--impl", default="engine", choices=["engine", "reference"])
    ap.add_argument("--batch", type=int, default=1, help="sequences decoded together (config 4 of the workload list uses 16)")
    ap.add_argument("--profile-range", action="store_true",
                    help="bracket the timed decode steps with cudaProfilerStart/Stop (for a profiler run with profile-from-start off)")
    ap.add_argument("--act-mode", type=int, default=2, help="INT4 matmul operand: 2 block-scaled 16-bit integers for one-row passes "
                    "(integer tensor-core kernel; fp16 for passes of several rows), 1 fp16 everywhere")
    ap.add_argument("--fused", action="store_true", help="attn workload: the fused rotary + append + attention call of the decode step")
    ap.add_argument("--group-tickets", action="store_true", help="gemv-impl 5: hand the tail of the grouped launch out by ticket")
    ap.add_argument("--gemv-trace", default=None, metavar="FILE.npy",
                    help="gemv workload with the KUIPER_TRACE=1 build: save the per-CTA clock readings of the last GEMV launch")
    ap.add_argument("--flash-trace", default=None, metavar="FILE.npy",
                    help="with the KUIPER_TRACE=1 build: save the per-CTA clock readings of the last attention launch")
    ap.add_argument("--prompt", type=int, default=None, help="override the workload's prompt length (profiling aid)")
    ap.add_argument("--tuning", action="append", default=[], metavar="KEY=VALUE",
                    help="kernel tuning switch applied before the run (profiling aid), e.g. flash_mma_fused=0")
    args = ap.parse_args()
    if args.tuning and args.impl == "engine":
        from mykuiperllama_b200 import capi
        for kv in args.tuning:
            key, _, value = kv.partition("=")
            capi.set_tuning(key, int(value))
    if args.warmup < 3 and args.impl == "engine":
        args.warmup = 3
    if args.workload == "gemv":
        run_gemv_micro(args)
        return
    if args.workload == "gemm":
        run_gemm_micro(args)
        return
    if args.workload == "attn":
        run_attn_micro(args)
        return
    cfg, prompt_len, _, _, desc = WORKLOADS[args.workload]
    if args.prompt is not None:
        prompt_len = args.prompt
        desc += f" (prompt overridden to {prompt_len} tokens)"
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, cfg, desc, rank, world)
        return
    if world != args.gpus:
        if args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torch.distributed.run with {args.gpus} ranks (WORLD_SIZE={world})")
    run_engine(args, cfg, prompt_len, desc, rank, world)


if __name__ == "__main__":
    main()
