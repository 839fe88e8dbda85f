"""Run a few eager decode steps of a full-width (few-layer) dense decoder between
cudaProfilerStart/Stop, for per-kernel timing with

    ncu --metrics gpu__time_duration.sum --clock-control none --profile-from-start off \
        --csv --log-file launches.csv python benchmarks/decode_step_profile.py

Without ncu it prints the wall time per decode step (eager launches, so host-bound)."""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vllm_kunlun_b200 import LLM, SamplingParams  # noqa: E402
from vllm_kunlun_b200.config import PRESETS, tiny  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--model", default="llama-3.1-8b")
ap.add_argument("--layers", type=int, default=4)
ap.add_argument("--batch", type=int, default=16)
ap.add_argument("--ctx", type=int, default=2048)
ap.add_argument("--steps", type=int, default=3)
a = ap.parse_args()

cfg = tiny(PRESETS[a.model](), num_layers=a.layers)
llm = LLM(cfg, device="cuda", block_size=64, max_model_len=a.ctx + 256, max_num_seqs=a.batch,
          max_num_batched_tokens=8192, enforce_eager=True)
eng = llm.engine
g = torch.Generator().manual_seed(0)
for _ in range(a.batch):
    eng.add_request(torch.randint(0, cfg.vocab_size, (a.ctx,), generator=g).tolist(),
                    SamplingParams(max_tokens=64, ignore_eos=True))
while any(r.num_computed_tokens < a.ctx for r in eng.scheduler.running) or eng.scheduler.waiting:
    eng.step()
for _ in range(3):
    eng.step()
torch.cuda.synchronize()
torch.cuda.profiler.start()
t0 = time.perf_counter()
for _ in range(a.steps):
    eng.step()
torch.cuda.synchronize()
t1 = time.perf_counter()
torch.cuda.profiler.stop()
print(f"decode step (eager, {a.layers} layers): {(t1 - t0) / a.steps * 1e3:.3f} ms")
