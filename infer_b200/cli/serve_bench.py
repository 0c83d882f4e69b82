"""Throughput against latency across slot counts, in the manner of the reference's main_serve_bench
(src/main_serve_bench.cpp:1-27,74-239): a fixed request set goes through the scheduler once per slot count, with
continuous and static batching.

    bin/serve_bench --model DIR | random=SPEC [key=value ...]
      random=          a preset name, a config.json or a JSON object: seeded random weights instead of --model
      n=64             requests                 slots=1,2,4,8,16,32
      max_new=48       spread over max_new/2 .. 3*max_new/2 (src/main_serve_bench.cpp:137)
      max_seq=192      per-sequence cap         budget_mb=0 (0 = reserve slots x max_seq)
      kv_blocks=0      size of the page pool in pages, instead of budget_mb
      prompt_len=12    prompts are seeded random ids of 5..prompt_len tokens (the reference cycles five fixed prompts)
      prefix=0         that many shared random tokens in front of every prompt (the reference's long-context switch)
      chunk=512        token budget of one step
      modes=both|continuous|static
      gemm=mine|plain  attn=split|plain         dtype=bfloat16|float32
      events=<path>    write the last continuous run's scheduler event log (JSON lines)
      tag=<text>       copied into the record
Prints a table and one JSON record per configuration: tok/s, mean step ms, token latency, request p50/p95,
TTFT p50, steps, peak pages, preemptions.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="serve_bench", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default=os.environ.get("LLM_MODEL"))
    ap.add_argument("kv", nargs="*")
    args = ap.parse_args(argv)
    opt = dict(n="64", slots="1,2,4,8,16,32", max_new="48", max_seq="192", budget_mb="0", prompt_len="12", chunk="512",
               modes="both", gemm="mine", attn="split", dtype="bfloat16", events="", tag="", random="", kv_blocks="0",
               prefix="0", weights_seed="0")
    for kv in args.kv:
        k, _, v = kv.partition("=")
        if k not in opt:
            ap.error(f"unknown option {k}")
        opt[k] = v
    if not args.model and not opt["random"]:
        ap.error("no model: give --model DIR, random=SPEC, or set LLM_MODEL")
    import numpy as np
    import torch
    from infer_b200.engine.generation import LLM
    from infer_b200.engine.scheduler import Request, SampleParams
    spec = weights = None
    if opt["random"]:
        from infer_b200.config import parse_config
        from infer_b200.models import load_preset
        from infer_b200.weights import random_weights
        arch, typed = parse_config(load_preset(opt["random"]))
        spec = arch.to_spec(typed)
        weights = random_weights(spec, int(opt["weights_seed"]), torch.bfloat16, device="cuda")
    kernels = {}
    if opt["gemm"] == "plain":
        kernels["linear"] = "plain"
    if opt["attn"] == "plain":
        kernels["attention"] = "plain"
    n, max_new_base, max_seq = int(opt["n"]), int(opt["max_new"]), int(opt["max_seq"])
    print(f"{'slots':>5} {'mode':>10} {'tok/s':>9} {'step ms':>8} {'tok lat ms':>10} {'req p50':>9} {'req p95':>9} "
          f"{'ttft p50':>8} {'steps':>6} {'pages':>7} {'peak':>7} {'preempt':>7}")
    records = []
    for slots in [int(s) for s in opt["slots"].split(",")]:
        llm = LLM(None if spec is not None else args.model, dtype=opt["dtype"], slots=slots, max_seq=max_seq,
                  budget_mb=int(opt["budget_mb"]), kv_blocks=int(opt["kv_blocks"]), max_batch_tokens=int(opt["chunk"]),
                  kernels=kernels, spec=spec, weights=weights)
        V = llm.engine.spec.vocab_size
        rng = np.random.default_rng(0)
        prefix = rng.integers(0, V, int(opt["prefix"])).tolist()
        prompts = [prefix + rng.integers(0, V, int(rng.integers(5, max(6, int(opt["prompt_len"]) + 1)))).tolist() for _ in range(5)]
        reqs = [(i, prompts[i % 5], max_new_base // 2 + (i * 7) % (max_new_base + 1)) for i in range(n)]
        for continuous in (True, False):
            if opt["modes"] == "continuous" and not continuous or opt["modes"] == "static" and continuous:
                continue
            warm = llm.new_scheduler(eos_id=-1)
            warm.submit(Request("warm", prompts[0], 4))
            warm.run_until_idle()
            sch = llm.new_scheduler(continuous=continuous, eos_id=-1)
            for i, p, mn in reqs:
                sch.submit(Request(i, list(p), max(1, mn), 0, SampleParams()))
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            sch.run_until_idle()
            torch.cuda.synchronize()
            wall = time.perf_counter() - t0
            total = sum(len(c.tokens) for c in sch.completed)
            lat = sorted(c.finished_ms for c in sch.completed)
            ttft = sorted(c.first_token_ms for c in sch.completed)
            pool = llm.engine.cache.groups[0].pool if llm.engine.cache.groups else None
            rec = dict(slots=slots, mode="continuous" if continuous else "static", tok_s=total / wall,
                       step_ms=wall * 1e3 / max(1, sch.steps),
                       token_latency_ms=sum((c.finished_ms - c.first_token_ms) / max(1, len(c.tokens) - 1) for c in sch.completed) / max(1, len(sch.completed)),
                       req_p50_ms=lat[len(lat) // 2], req_p95_ms=lat[min(len(lat) - 1, int(len(lat) * 0.95))],
                       ttft_p50_ms=ttft[len(ttft) // 2], steps=sch.steps, pages=pool.n_pages if pool else 0,
                       peak_pages=pool.peak_in_use if pool else 0, preemptions=sch.preemptions, tag=opt["tag"],
                       n=n, tokens=total, dtype=opt["dtype"])
            records.append(rec)
            print(f"{slots:>5} {rec['mode']:>10} {rec['tok_s']:>9.1f} {rec['step_ms']:>8.3f} {rec['token_latency_ms']:>10.3f} "
                  f"{rec['req_p50_ms']:>9.1f} {rec['req_p95_ms']:>9.1f} {rec['ttft_p50_ms']:>8.1f} {rec['steps']:>6} "
                  f"{rec['pages']:>7} {rec['peak_pages']:>7} {rec['preemptions']:>7}")
            if opt["events"] and continuous:
                sch.events.write_jsonl(opt["events"])
        del llm
        torch.cuda.empty_cache()
    for r in records:
        print(json.dumps(r))
    return 0


if __name__ == "__main__":
    sys.exit(main())
