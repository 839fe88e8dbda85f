"""Serving benchmark client for the OpenAI-compatible server: N requests at a fixed concurrency, fixed input /
output lengths, streamed completions; reports TTFT, TPOT and output-token throughput.

    python -m vllm_kunlun_b200.entrypoints.openai_server --model llama-3.1-8b --port 8000 &
    python benchmarks/bench_serving.py --port 8000 --num-prompts 16 --max-concurrency 16 \\
        --random-input-len 2048 --random-output-len 2048

Counterpart of the ``vllm bench serve`` runs the reference documents
(``docs/source/developer_guide/performance/performance_benchmark/benchmark_server.md:36-104``) and of its
CI perf script (``ci/scripts/perf``)."""
import argparse
import asyncio
import json
import random
import statistics
import time


async def one_request(session, url, model, prompt_ids, out_len, result):
    body = {"model": model, "prompt": prompt_ids, "max_tokens": out_len, "temperature": 0, "ignore_eos": True, "stream": True}
    t0 = time.perf_counter()
    first = last = None
    n = 0
    async with session.post(url, json=body) as resp:
        async for raw in resp.content:
            line = raw.decode().strip()
            if not line.startswith("data: ") or line == "data: [DONE]":
                continue
            chunk = json.loads(line[6:])
            text = chunk["choices"][0].get("text", "")
            if text:
                now = time.perf_counter()
                first = first or now
                last = now
                n += len(text.split())
    if first is None:
        result.append(None)
        return
    result.append({"ttft": first - t0, "tpot": (last - first) / max(1, n - 1), "tokens": n, "latency": last - t0})


async def run(a):
    import aiohttp
    rng = random.Random(a.seed)
    prompts = [[rng.randrange(10, a.vocab_size) for _ in range(a.random_input_len)] for _ in range(a.num_prompts)]
    url = f"http://{a.host}:{a.port}/v1/completions"
    sem = asyncio.Semaphore(a.max_concurrency)
    results: list = []
    timeout = aiohttp.ClientTimeout(total=None)
    async with aiohttp.ClientSession(timeout=timeout) as session:
        async def guarded(p):
            async with sem:
                await one_request(session, url, a.model, p, a.random_output_len, results)
        t0 = time.perf_counter()
        await asyncio.gather(*(guarded(p) for p in prompts))
        dur = time.perf_counter() - t0
    ok = [r for r in results if r]
    out = {"completed": len(ok), "failed": len(results) - len(ok), "duration_s": round(dur, 3),
           "output_tok_per_s": round(sum(r["tokens"] for r in ok) / dur, 1),
           "mean_ttft_ms": round(1e3 * statistics.mean(r["ttft"] for r in ok), 2) if ok else None,
           "p50_ttft_ms": round(1e3 * statistics.median(r["ttft"] for r in ok), 2) if ok else None,
           "mean_tpot_ms": round(1e3 * statistics.mean(r["tpot"] for r in ok), 3) if ok else None,
           "p50_tpot_ms": round(1e3 * statistics.median(r["tpot"] for r in ok), 3) if ok else None,
           "concurrency": a.max_concurrency, "input_len": a.random_input_len, "output_len": a.random_output_len}
    print(json.dumps(out))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--model", default="model")
    ap.add_argument("--num-prompts", type=int, default=16)
    ap.add_argument("--max-concurrency", type=int, default=16)
    ap.add_argument("--random-input-len", type=int, default=2048)
    ap.add_argument("--random-output-len", type=int, default=2048)
    ap.add_argument("--vocab-size", type=int, default=32000)
    ap.add_argument("--seed", type=int, default=0)
    return asyncio.run(run(ap.parse_args(argv)))


if __name__ == "__main__":
    main()
