"""Headline benchmark: output tok/s at 16-way concurrency, 2048-token prompts, 2048 generated tokens.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--model llama-3.1-8b]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

One *step* is one complete serving round: 16 concurrent requests, each a 2048-token prompt of
uniform random ids, greedy generation of 2048 tokens with ignore_eos, run through the framework's
own engine (scheduler, paged KV cache, chunked prefill, CUDA-graph decode).  Weights are random-init
N(0, 0.02) of the named architecture; N GPUs = tensor parallel over N ranks (strong scaling: the
request set is fixed).

Two measurements, each of exactly K steps after W warm-up steps:
  value  device time: CUDA events on the launching stream around the K steps, barrier +
         synchronize on both sides, max over ranks;
  e2e    the public API (``LLM.generate`` on host token lists): wall clock around the call,
         including every step's host->device copy of its inputs from pinned memory and the
         device->host read of the sampled tokens.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_TOK_S = {  # published by the reference (Kunlun3 P800), 16-way, 2048/2048
    "llama-3.1-8b": 1779.8,   # closest published analogue: Qwen3-8B, TP=1
    "qwen3-8b": 1779.8,
    "qwen3-30b-a3b": 1927.4,  # Qwen3-30B-A3B, TP=2
    # nothing is published for DeepSeek-V3 / V3.2; the nearest chart entry by size is Qwen3-235B-A22B at TP=8
    "deepseek-v3": 927.5,
}


BASELINE_REF = {
    "llama-3.1-8b": "Qwen3-8B TP=1 on Kunlun3 P800 (closest published analogue)",
    "qwen3-8b": "Qwen3-8B TP=1 on Kunlun3 P800",
    "qwen3-30b-a3b": "Qwen3-30B-A3B TP=2 on 2x Kunlun3 P800",
    "deepseek-v3": "none published for DeepSeek-V3; Qwen3-235B-A22B TP=8 on 8x Kunlun3 P800 is the nearest chart entry",
    "deepseek-v3.2": "none published",
}

# The benchmark configurations by number: 2 is the default (the driver's command line does not change).
CONFIGS = {
    2: dict(model="llama-3.1-8b", in_len=2048, out_len=2048, ep=False, spec=None, kv_cache_dtype="auto"),
    3: dict(model="qwen3-30b-a3b", in_len=2048, out_len=2048, ep=True, spec=None, kv_cache_dtype="auto"),
    4: dict(model="deepseek-v3", in_len=2048, out_len=2048, ep=True, spec="mtp", kv_cache_dtype="auto"),
    5: dict(model="deepseek-v3.2", in_len=32768, out_len=1024, ep=True, spec=None, kv_cache_dtype="auto"),
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=sorted(CONFIGS),
                    help="benchmark configuration: 2 Llama-3.1-8B bf16 (default), 3 Qwen3-30B-A3B fp8 TP+EP, "
                         "4 DeepSeek-V3 fp8 TP+EP+MTP, 5 DeepSeek-V3.2 sparse attention at 32k context")
    ap.add_argument("--model", default=None, help="override the model of the configuration")
    ap.add_argument("--concurrency", type=int, default=16)
    ap.add_argument("--in-len", type=int, default=None)
    ap.add_argument("--out-len", type=int, default=None)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--ep", action="store_true", help="expert parallelism for MoE models (whole experts per rank)")
    ap.add_argument("--spec", default=None, help="speculative method (mtp | ngram | eagle), one draft token")
    ap.add_argument("--kv-cache-dtype", default=None)
    ap.add_argument("--tp", type=int, default=0,
                    help="tensor-parallel size (0 = choose); the remaining ranks form data-parallel replicas that share "
                         "the concurrent requests")
    ap.add_argument("--layers", type=int, default=0,
                    help="debugging only: run with this many layers (the JSON line then says so and is not a result)")
    a = ap.parse_args()
    c = CONFIGS[a.config]
    a.model = a.model or c["model"]
    a.in_len = a.in_len or c["in_len"]
    a.out_len = a.out_len or c["out_len"]
    a.ep = a.ep or c["ep"]
    a.spec = a.spec or c["spec"]
    a.kv_cache_dtype = a.kv_cache_dtype or c["kv_cache_dtype"]
    return a


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region (read-only queries)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "200", "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self) -> dict:
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, pw = [], [], []
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.f.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2])); pw.append(float(parts[3]))
            except ValueError:
                continue
            for n, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.unlink(self.f.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(pw),
                "samples": len(sm), "reasons": sorted(reasons)}


def reference_arm(args):
    """The reference arm: the unmodified reference through its own public API, or one ``unavailable`` line.

    Two independent facts keep it from running here (``baseline/probe_reference.py`` reproduces the second):
    * its offline install (``pip install --no-index --no-build-isolation --find-links /opt/wheelhouse --target
      baseline/_ref``) fails because the build backend ``hatchling`` is not in the wheelhouse;
    * a plain copy of the package with empty stand-ins for the closed Kunlun wheels registers its platform, but the
      modules behind it do not import on the installed vLLM 0.22 (the reference pins 0.15.1): the first failures are
      ``from vllm.v1.attention.backends.tree_attn import TreeAttentionMetadata`` (``v1/sample/spec_decode/eagle.py:10``,
      reached from ``vllm_kunlun.ops`` and from the attention backend) and ``from vllm.attention.backends.abstract
      import AttentionBackend`` (``v1/worker/utils.py:8``); both modules are gone from vLLM 0.22.
    """
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference pins vLLM 0.15.1 and does not import on the installed vLLM 0.22 "
                      "(ModuleNotFoundError: vllm.v1.attention.backends.tree_attn, vllm.attention); its kernels are "
                      "closed Kunlun wheels (kunlun_ops/xspeedgate_ops/cocopod) and its hatchling build backend is "
                      "absent offline, so baseline/_ref could not be installed"}))
    return 0


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    import torch
    import torch.distributed as dist

    from vllm_kunlun_b200 import LLM, SamplingParams
    from vllm_kunlun_b200.ops import _ext

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local)
    C, IN, OUT = args.concurrency, args.in_len, args.out_len
    # Parallel layout.  The dense 8B model at 16 concurrent requests stops gaining from tensor parallelism beyond 4
    # ranks (64 all-reduces per step across 8 ranks cost what the smaller per-rank GEMMs save): 8 GPUs run as two
    # replicas of 4, each serving half of the requests.  The MoE configurations keep TP = EP = all ranks.
    tp = args.tp or (4 if (args.config == 2 and world == 8 and C % 2 == 0) else world)
    if world % tp or C % (world // tp):
        raise SystemExit(f"--tp {tp} does not divide {world} ranks / {C} requests")
    dp = world // tp
    C_local = C // dp
    spec = {"method": args.spec, "num_speculative_tokens": 1} if args.spec else None
    model = args.model
    if args.layers:
        import dataclasses

        from vllm_kunlun_b200.config import PRESETS
        mc = PRESETS[args.model]()
        model = dataclasses.replace(mc, num_layers=args.layers,
                                    first_dense_layers=min(mc.first_dense_layers, max(1, args.layers // 2)))
    llm = LLM(model, tensor_parallel_size=tp, data_parallel_size=dp, device="cuda", block_size=64,
              max_model_len=IN + OUT + 64, max_num_seqs=C_local, max_num_batched_tokens=8192,
              gpu_memory_utilization=0.9, seed=0, enable_expert_parallel=args.ep and tp > 1, speculative_config=spec,
              kv_cache_dtype=args.kv_cache_dtype)
    eng = llm.engine
    dp_rank = eng.pstate.dp_rank if dp > 1 else 0
    vocab = eng.cfg.model.vocab_size
    g = torch.Generator().manual_seed(1234)
    # prompts live in pinned host memory; every round draws a fresh set so nothing is cached
    n_rounds = args.warmup + 2 * args.steps
    prompt_bank = torch.randint(0, vocab, (n_rounds, C, IN), generator=g, dtype=torch.int64).pin_memory()
    sp = SamplingParams(max_tokens=OUT, temperature=0.0, ignore_eos=True)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local])
        torch.cuda.synchronize()

    ttfts, tpots = [], []

    def one_round(i, collect=False):
        # every replica serves its own share of the round's prompts
        outs = llm.generate([prompt_bank[i, c].tolist() for c in range(dp_rank * C_local, (dp_rank + 1) * C_local)], sp)
        assert all(len(o.token_ids) == OUT for o in outs)
        if collect:
            ttfts.extend(o.ttft for o in outs)
            tpots.extend(o.tpot for o in outs)
        return outs

    r = 0
    for _ in range(args.warmup):
        one_round(r); r += 1
    # ---------------- device-timed region
    sampler = ClockSampler(local)
    barrier()
    k0 = _ext.C().launch_count()
    g0 = eng.runner.graphs.replayed_kernels if eng.runner.graphs else 0
    h0, d0 = eng.runner.h2d_bytes, eng.runner.d2h_bytes
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        one_round(r, collect=True); r += 1
    e1.record()
    barrier()
    clocks = sampler.stop()
    dev_ms = e0.elapsed_time(e1)
    launches = (_ext.C().launch_count() - k0) + ((eng.runner.graphs.replayed_kernels - g0) if eng.runner.graphs else 0)
    h2d = (eng.runner.h2d_bytes - h0) / args.steps
    d2h = (eng.runner.d2h_bytes - d0) / args.steps
    # ---------------- end-to-end region (public API, wall clock)
    e2e_ms = None
    if not args.no_e2e:
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            one_round(r); r += 1
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
    t = torch.tensor([dev_ms, e2e_ms or 0.0], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_max = t.tolist()
    if dp > 1:
        # latencies and byte / launch counts of every replica (one reporter per replica: its first rank)
        part = (ttfts, tpots, h2d, d2h, launches) if eng.pstate.tp_rank == 0 and eng.pstate.pp_rank == 0 else None
        parts = [None] * world
        dist.all_gather_object(parts, part)
        parts = [x for x in parts if x is not None]
        ttfts = [v for x in parts for v in x[0]]
        tpots = [v for x in parts for v in x[1]]
        h2d, d2h, launches = (sum(x[k] for x in parts) for k in (2, 3, 4))
    from vllm_kunlun_b200.ops.gemm_cuda import check_status
    check_status()
    # every status word of the peer-memory collectives and the expert exchange must be clean as well: a number
    # from a run in which a bounded wait gave up would come from wrong data
    for comm in (eng.pstate.tp_comm, eng.pstate.ep_comm, eng.pstate.dcp_comm):
        peer = getattr(comm, "peer", None) if comm is not None else None
        if peer is not None:
            peer.check_status()
    a2a = getattr(eng.pstate, "ep_a2a", None)
    if a2a is not None:
        a2a.check_status()
    if rank == 0:
        tokens = C * OUT * args.steps
        value = tokens / (dev_ms / 1e3)
        base = BASELINE_TOK_S.get(args.model)
        out = {
            "metric": f"output tok/s at {C} concurrency, {IN} in/{OUT} out", "value": round(value, 1), "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dev_ms / args.steps, 2),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": round(value / base, 3) if base else None,
            "dtype": "fp8 weights (128x128 block scales), bf16 activations" if eng.cfg.model.quantization == "fp8" else "bf16",
            "data": "synthetic (uniform random token ids, random-init N(0,0.02) weights)",
            "impl": "ours",
            "config": {"model": args.model, "bench_config": args.config, "global_batch": C, "seq_len": IN + OUT,
                       "in_len": IN, "out_len": OUT,
                       "parallelism": f"tp{tp}" + (f"+dp{dp}" if dp > 1 else "") + ("+ep" if args.ep and tp > 1 else "") +
                                      (f"+{args.spec}" if args.spec else ""),
                       "step": f"one full serving round of {C} requests",
                       **({"reduced_layers": args.layers, "valid": False} if args.layers else {}),
                       **({"spec_acceptance": round(eng.stats["spec_accepted"] / max(1, eng.stats["spec_proposed"]), 3)}
                          if args.spec else {}),
                       "l2": "inputs larger than L2: every decode step streams the active weight set and the KV cache "
                             "(16 GB of bf16 weights for the 8B dense model)",
                       "baseline_ref": BASELINE_REF.get(args.model, "none published")},
            "p50_ttft_ms": round(statistics.median(ttfts) * 1e3, 1) if ttfts else None,
            "p50_tpot_ms": round(statistics.median(tpots) * 1e3, 3) if tpots else None,
            "clocks": clocks, "gpu_launches": int(launches),
        }
        if e2e_ms is not None:
            out["e2e"] = {"value": round(tokens / (e2e_max / 1e3), 1), "unit": "tok/s",
                          "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                          "ms_per_step": round(e2e_max / args.steps, 2)}
        print(json.dumps(out), flush=True)
    if world > 1:
        # orderly teardown: drop the captured graphs first (they hold references into the communicators'
        # buffers), then the peer mappings, then the process group
        torch.cuda.synchronize()
        dist.barrier(device_ids=[local])
        sys.stdout.flush()
        try:
            if eng.runner.graphs is not None:
                eng.runner.graphs.graphs.clear()
                eng.runner.graphs = None
            torch.cuda.synchronize()
            from vllm_kunlun_b200.parallel.state import destroy_model_parallel
            destroy_model_parallel()
            dist.barrier(device_ids=[local])
            dist.destroy_process_group()
        except Exception as e:  # a failed teardown must not turn a measured run into a failed one
            print(f"[bench] teardown: {e!r}", file=sys.stderr, flush=True)
            os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
