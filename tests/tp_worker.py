"""Rank body of the tensor-parallel GPU test: a tiny Qwen3-shaped model sharded over WORLD_SIZE GPUs must give the
oracle's logits and greedy tokens on every rank."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import make_model_weights, rel_err  # noqa: E402
from mykuiperllama_b200 import engine  # noqa: E402
from oracle import cpu_oracle as orc  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("gloo")  # host plumbing only; the engine talks NCCL itself
    # 8 kv heads and an intermediate width of 8 groups: shards evenly over 2, 4 and 8 ranks
    cfg = dict(n_layers=2, hidden=512, n_q_heads=16, n_kv_heads=8, head_dim=128, inter=1024, vocab=1000, max_seq=64,
               max_batch=1)
    act_mode = int(os.environ.get("KUIPER_TEST_ACT_MODE", "2"))
    ocfg = orc.ModelConfig(**cfg, act_round=orc.ROUND_ENGINE if act_mode == 2 else orc.ROUND_FP16)
    weights = make_model_weights(orc, ocfg, seed=21)
    ref = orc.OracleModel(ocfg, weights)
    eng = engine.Qwen3Engine(engine.EngineConfig(**cfg, tp_rank=rank, tp_size=world, act_mode=act_mode))
    eng.load(weights)  # every rank gets the unsharded weights; the engine slices its part
    uid = [engine.Qwen3Engine.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, 0)
    eng.init_tp(uid[0])

    prompt = np.array([11, 7, 993, 2, 400, 5, 77, 12, 9, 31], np.int32)  # two chunks
    lg_ref, nx_ref = ref.forward(prompt, np.arange(10, dtype=np.int32))
    first = eng.prefill(prompt)
    assert first == nx_ref[-1], (rank, first, nx_ref[-1])
    lg, nx = eng.predict(prompt[:5], np.arange(5, dtype=np.int32), want_logits=True)
    assert rel_err(lg, lg_ref[:5]) <= 2e-3, (rank, rel_err(lg, lg_ref[:5]))
    eng.prefill(prompt)  # restore the cache rows the predict call rewrote (same values)
    eng.decode_begin([first], [10], [0])
    tok = first
    for i in range(8):
        _, nx = ref.forward([tok], [10 + i])
        eng.decode_step(1)
        got = int(eng.decode_read(1)[0])
        assert got == nx[0], (rank, i, got, nx[0])
        tok = got
    eng.tp_status()
    dist.barrier()
    sys.stdout.write("tp-rank%d-ok one-shot=%d\n" % (rank, int(eng.tp_one_shot())))
    eng.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
