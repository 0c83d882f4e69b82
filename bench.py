"""Headline benchmark: decode tokens/s (and prefill tokens/s at 2,048 tokens) at Qwen2.5-1.5B layer sizes with
random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 2048] [--layers L] [--impl reference]

Prints ONE JSON line. "value" is decoded tokens per second of the step function, timed on the device with CUDA
events around K decode steps of a batch of 8 requests whose 2,048-token contexts already lie in the paged cache
(the cache is filled with random keys and values: throughput does not depend on their values). "e2e" is the same
through the Python entry point's scheduler: host token ids in, sampled host token ids out, every step.
Every step reads all weights (3.1 GB) and the live requests' cache (0.47 GB at batch 8): far more than the 126 MB
L2, so no flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The benchmark configurations are the config.json presets of the package (no weights): Qwen2.5-1.5B layer sizes by
# default, 7B and 14B with --sizes.
def _preset(name):
    with open(os.path.join(ROOT, "infer_b200", "models", "presets", name + ".json")) as f:
        return json.load(f)


SIZES = {"1.5b": _preset("qwen2.5-1.5b"), "7b": _preset("qwen2.5-7b"), "14b": _preset("qwen2.5-14b")}
CONFIG = SIZES["1.5b"]
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    src = "fallback"
    p = dict(FALLBACK_PEAKS)
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            flat = {}

            def walk(d):
                for k, v in d.items():
                    if isinstance(v, dict):
                        walk(v)
                    elif isinstance(v, (int, float)):
                        flat.setdefault(k, float(v))
            walk(raw)
            for k in p:
                if k in flat:
                    p[k] = flat[k]
            src = "measured"
        except Exception:
            pass
    p["source"] = src
    return p


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs (reads only)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])), mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# The reference's own published decode throughput for the 1.5B model under continuous batching, by concurrent
# sequences (bench/stage11_slots_15b_bf16_1.5B.json, README.md:68 of RyanXiaoo/infer): one RTX 5070 Ti, real weights,
# prompts of 5-12 tokens. It publishes nothing on a B200, at 2,048-token contexts or at batch 64.
PUBLISHED_TOK_S = {1: 178.4, 4: 554.5, 8: 891.6, 16: 1339.2, 32: 1360.8}
PUBLISHED_NOTE = "reference's published tok/s at the same number of sequences on one RTX 5070 Ti with short contexts"


def build_engine(n_layers, batch, context, steps_total, dtype="bfloat16"):
    import torch
    from infer_b200.config import parse_config
    from infer_b200.engine import Engine
    from infer_b200.weights import random_weights
    import infer_b200.models  # noqa: F401
    cfg = dict(CONFIG, num_hidden_layers=n_layers)
    arch, typed = parse_config(cfg)
    spec = arch.to_spec(typed)
    W = random_weights(spec, 0, torch.bfloat16, device="cuda")
    max_seq = context + steps_total + 16
    eng = Engine(spec, W, dtype=dtype, max_tokens=batch * (max_seq + 16), max_requests=batch, max_seq_len=max_seq)
    del W
    torch.cuda.empty_cache()
    return eng


def fill_contexts(eng, batch, context):
    """Admits `batch` requests and gives each a context of `context` positions of random keys and values."""
    import torch
    for g in eng.cache.groups:
        g.k.normal_(0, 0.5)
        g.v.normal_(0, 0.5)
    for r in range(batch):
        eng.add_request(r)
        assert eng.cache.reserve(r, context)
        eng.cache.advance(r, context)
    torch.cuda.synchronize()


def release_all(eng):
    for r in list(eng.cache.requests):
        eng.end_request(r)


def decode_bytes(eng, batch, context_mid):
    """Bytes one decode step has to read: every weight once (the token table only as the output matrix when tied,
    plus `batch` rows), and the cache of the live requests."""
    spec = eng.spec
    w = eng.model.weight_bytes()
    item = 2 if str(eng.rt.dtype).endswith("bfloat16") else 4
    table = eng.model.embedding.table()
    head_w = getattr(getattr(eng.model.head, "linear", None), "weight", None)
    if table is not None and (head_w is None or head_w.data_ptr() != table.data_ptr()):
        w -= table.numel() * item - batch * spec.hidden_size * item         # an untied table is read row by row only
    kv = sum(2 * len(g.cache_ids) * g.need.num_kv_heads * g.need.head_dim * item for g in eng.cache.groups)
    return w + batch * context_mid * kv, w, kv


def time_decode(eng, batch, context, steps, warmup, kernel_counter):
    """Device-timed decode steps of the step function: greedy ids are fed back on the device side of the engine's
    inputs only through the host packing of token ids (the ids fed are fixed: throughput does not depend on them)."""
    import torch
    from infer_b200.engine import StepEntry
    fill_contexts(eng, batch, context)
    ids = [(7 * r + 1) % eng.spec.vocab_size for r in range(batch)]

    def one():
        return eng.step([StepEntry(r, [ids[r]], [0]) for r in range(batch)])
    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    n0 = kernel_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    eng.check_status()
    launches = kernel_counter() - n0
    release_all(eng)
    return ms / steps, launches


def time_prefill(eng, tokens, reps, warmup):
    import torch
    from infer_b200.engine import StepEntry
    import numpy as np
    ids = np.random.default_rng(0).integers(0, eng.spec.vocab_size, tokens).tolist()
    times = []
    for i in range(warmup + reps):
        eng.add_request("p")
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.step([StepEntry("p", ids, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        eng.end_request("p")
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def serve_workload(eng, n_requests, len_lo, len_hi, max_new, chunk, seed=0):
    """Continuous batching through the scheduler of the Python entry point: `n_requests` requests, all submitted at
    once, with seeded random prompt lengths in [len_lo, len_hi] and `max_new` generated tokens each, prompts cut into
    portions of at most `chunk` tokens beside the decode tokens of the running requests. Host token ids in, sampled
    host token ids out. Wall clock around the whole run, synchronised on both sides."""
    import numpy as np
    import torch
    from infer_b200.engine.generation import GenerationEngine
    from infer_b200.engine.scheduler import Request, SampleParams, Scheduler, SchedulerConfig
    ge = GenerationEngine(eng)
    rng = np.random.default_rng(seed)
    V = eng.spec.vocab_size
    warm = Scheduler(ge, SchedulerConfig(eos_id=-1, max_batch_tokens=chunk, overlap=True))
    for r in range(2):
        warm.submit(Request(("warm", r), rng.integers(0, V, 3 * chunk // 2 + r).tolist(), 8, 0, SampleParams()))
    warm.run_until_idle()
    lengths = rng.integers(len_lo, len_hi + 1, n_requests)
    sch = Scheduler(ge, SchedulerConfig(eos_id=-1, max_batch_tokens=chunk, overlap=True))
    for r, n in enumerate(lengths):
        sch.submit(Request(r, rng.integers(0, V, int(n)).tolist(), max_new, 0, SampleParams()))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    sch.run_until_idle()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    eng.check_status()
    generated = sum(len(c.tokens) for c in sch.completed)
    lat = sorted(c.finished_ms for c in sch.completed)
    ttft = sorted(c.first_token_ms for c in sch.completed)
    return {"requests": n_requests, "prompt_tokens": int(lengths.sum()), "generated_tokens": generated,
            "wall_s": round(wall, 3), "generated_tok_s": round(generated / wall, 1),
            "total_tok_s": round((int(lengths.sum()) + generated) / wall, 1), "steps": sch.steps,
            "ms_per_step": round(wall * 1e3 / max(1, sch.steps), 3), "preemptions": sch.preemptions,
            "request_p50_ms": round(lat[len(lat) // 2], 1), "ttft_p50_ms": round(ttft[len(ttft) // 2], 1),
            "chunk": chunk, "prompt_lengths": [int(len_lo), int(len_hi)], "max_new": max_new}


def prefill_flops(cfg, n_layers, T):
    H, nh, nkv, hd, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                            cfg["hidden_size"] // cfg["num_attention_heads"], cfg["intermediate_size"], cfg["vocab_size"])
    lin = 2 * T * (H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * I)
    attn = 2 * 2 * nh * hd * T * (T + 1) / 2
    return n_layers * (lin + attn) + 2 * H * V          # logits at the last place only


def time_e2e(eng, batch, context, steps, warmup):
    """Decode through the scheduler of the Python entry point, as LLM.generate drives it: requests with prompts of
    `context` random host token ids are submitted and prefilled; then K scheduler steps are timed. Every step packs
    that step's integers into pinned host memory and copies them to the device, launches the step, samples on the
    device and copies the sampled ids to pinned host memory, where the scheduler reads them (one step late: the
    next step is launched first and takes its input tokens from the device)."""
    import numpy as np
    import torch
    from infer_b200.engine.generation import GenerationEngine
    from infer_b200.engine.scheduler import Request, SampleParams, Scheduler, SchedulerConfig
    ge = GenerationEngine(eng)
    got = []
    sch = Scheduler(ge, SchedulerConfig(eos_id=-1, max_batch_tokens=2048, overlap=True,
                                        on_token=lambda rid, tok: got.append(tok)))
    rng = np.random.default_rng(1)
    # requests whose prompts end early decode while the others' prompts still run: room for those tokens too
    prompt_steps = -(-batch * context // 2048) + batch
    for r in range(batch):
        sch.submit(Request(r, rng.integers(0, eng.spec.vocab_size, context).tolist(), warmup + steps + 8 + prompt_steps, 0, SampleParams()))
    while sch.queue or any(not a.decoding for a in sch.active.values()):
        sch.step()
    for _ in range(warmup):
        sch.step()
    torch.cuda.synchronize()
    n0 = len(got)
    t0 = time.perf_counter()
    for _ in range(steps):
        sch.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    n_tokens = batch * steps                 # tokens generated on the device in the timed steps
    assert len(got) - n0 >= batch * (steps - 1), "the scheduler did not hand the tokens to the host"
    h2d = eng.last_h2d_bytes                 # the one packed buffer: step integers and sampling inputs
    for rid in list(sch.active):
        sch.cancel(rid)
    sch.run_until_idle()
    release_all(eng)
    return n_tokens / dt, h2d, 4 * batch


def reference_arm(args):
    """The unmodified reference (built out of tree for sm_100 under baseline/_ref, see baseline/reference_arm.py)
    through its own serving bench, main_serve_bench: as many requests as slots, contexts of `context` tokens (a
    shared prefix plus 8 tokens each), CUDA graphs, continuous batching. The durations of its scheduler's decode
    steps come from its own event log; W of them are dropped and the next K taken. Its scheduler step copies the
    step's token ids to the device and reads the sampled ids back every step, so `value` and `e2e` are the same
    number: the reference has no device-only timing on this path. It refuses more than 32 rows in a step, so there
    is no batch-64 point."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ra
    n_layers = args.layers or CONFIG["num_hidden_layers"]
    cfg = dict(CONFIG, num_hidden_layers=n_layers)
    name = f"qwen2.5-{args.sizes}-random-{n_layers}l"
    try:
        binary = ra.build()
        ra.prepare_model(cfg, name)
        clocks = ClockSampler()
        clocks.start()
        need = args.warmup + args.steps
        main_run = ra.run_serve_bench(binary, name, args.batch, args.context, max_new=2 * need + 16)
        clk = clocks.stop()
        durs = main_run["step_ms"][args.warmup:args.warmup + args.steps]
        if len(durs) < args.steps:
            raise ra.Unavailable(f"only {len(durs)} timed decode steps, {args.steps} wanted")
        ms_step = sum(durs) / len(durs)
        points = {}
        if not args.no_points:
            one = ra.run_serve_bench(binary, name, 1, args.context, max_new=2 * need + 16)
            d1 = one["step_ms"][args.warmup:args.warmup + args.steps]
            points["decode_b1"] = round(1e3 * len(d1) / sum(d1), 1)
    except ra.Unavailable as e:
        print(json.dumps({"impl": "reference", "unavailable": str(e)}))
        return 0
    value = args.batch * 1e3 / ms_step
    pk = peaks()
    hd = cfg["hidden_size"] // cfg["num_attention_heads"]
    # what the reference's step has to read: bfloat16 weights once, and its float32 cache of the live requests
    w_bytes = 2 * (n_layers * (cfg["hidden_size"] * (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * hd
                               + cfg["num_attention_heads"] * hd * cfg["hidden_size"] + 3 * cfg["hidden_size"] * cfg["intermediate_size"])
                   + cfg["vocab_size"] * cfg["hidden_size"])
    kv_bytes = args.batch * (args.context + args.warmup + args.steps // 2) * n_layers * 2 * cfg["num_key_value_heads"] * hd * 4
    achieved = (w_bytes + kv_bytes) / (ms_step * 1e-3) / 1e9
    out = {"impl": "reference", "metric": f"decode tok/s at batch {args.batch}, {args.context}-token contexts (Qwen2.5-{args.sizes.upper()} sizes)",
           "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak",
           "vs_baseline": round(value / PUBLISHED_TOK_S[args.batch], 2) if args.sizes == "1.5b" and args.batch in PUBLISHED_TOK_S else None,
           "baseline": PUBLISHED_NOTE, "dtype": "bf16 weights, fp32 activations and cache (the reference's only mode)",
           "data": "synthetic: random weights N(0,0.02), random token ids",
           "config": {"model": f"Qwen2.5-{args.sizes.upper()} sizes", "layers": n_layers, "layers_of_model": CONFIG["num_hidden_layers"],
                      "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                      "head_dim": hd, "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                      "global_batch": args.batch, "seq_len": args.context, "page_size": 16,
                      "tied_head": bool(cfg["tie_word_embeddings"]), "parallelism": "single GPU",
                      "l2": "inputs larger than L2", "how": "main_serve_bench n=slots prefix=context-8 graphs=1, step durations from its event log"},
           "clocks": clk, "gpu_launches": None,
           "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None},
           "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                        "frac": round(achieved / pk["hbm_gbs"], 4)},
           "points": points,
           "prefill": {"value": round(main_run["prompt_tokens"] * 1e3 / max(main_run["prompt_ms"], 1e-9), 1),
                       "tokens": main_run["prompt_tokens"], "ms": round(main_run["prompt_ms"], 3),
                       "frac": round(prefill_flops(cfg, n_layers, main_run["prompt_tokens"]) / (max(main_run["prompt_ms"], 1e-9) * 1e-3)
                                     / (pk["bf16_tflops"] * 1e12), 4)}}
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all of them)")
    ap.add_argument("--sizes", default="1.5b", choices=sorted(SIZES), help="layer sizes: Qwen2.5-1.5B (the default), 7B or 14B")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--points", default="1,64", help="batch sizes of the further decode points (default 1,64)")
    ap.add_argument("--workload", default="decode", choices=["decode", "serve"],
                    help="serve: 64 requests with prompts of 128..4096 tokens and 128 new tokens each under continuous "
                         "batching with prompt portions of 512 (the 7B measurement workload); prints its own line")
    ap.add_argument("--requests", type=int, default=64, help="serve: number of requests")
    ap.add_argument("--chunk", type=int, default=512, help="serve: token budget of a step")
    ap.add_argument("--mode", default="all", choices=["all", "decode", "prefill"],
                    help="decode / prefill: run only that part and print a short line (for profiling small cases)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    global CONFIG
    CONFIG = SIZES[args.sizes]
    if args.impl == "reference":
        return reference_arm(args)
    import torch
    from infer_b200 import ops
    pk = peaks()
    n_layers = args.layers or CONFIG["num_hidden_layers"]
    total_steps = args.steps + args.warmup
    cfg = CONFIG
    if args.workload == "serve":
        lo, hi, max_new = 128, 4096, 128
        # the pool holds every request at once (the 7B sizes take 57 KB per position: 15 GB for 64 requests)
        eng = build_engine(n_layers, args.requests, hi, max_new + 64)
        rec = serve_workload(eng, args.requests, lo, hi, max_new, args.chunk)
        rec.update(workload="serve", model=f"Qwen2.5-{args.sizes.upper()} sizes", layers=n_layers,
                   layers_of_model=CONFIG["num_hidden_layers"], slots=args.requests, dtype="bf16")
        print(json.dumps(rec))
        return 0
    point_batches = [] if args.no_points else [int(b) for b in args.points.split(",") if b]
    eng = build_engine(n_layers, max([args.batch] + point_batches), args.context, 2 * total_steps + 64)

    if args.mode == "decode":
        ms_step, launches = time_decode(eng, args.batch, args.context, args.steps, args.warmup, ops.kernel_launches)
        print(json.dumps({"mode": "decode", "batch": args.batch, "ms_per_step": round(ms_step, 4), "gpu_launches": launches}))
        return 0
    if args.mode == "prefill":
        ms_p = time_prefill(eng, 2048, max(1, args.steps), args.warmup)
        print(json.dumps({"mode": "prefill", "tokens": 2048, "ms": round(ms_p, 3)}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    ms_step, launches = time_decode(eng, args.batch, args.context, args.steps, args.warmup, ops.kernel_launches)
    clk = clocks.stop()
    value = args.batch * 1e3 / ms_step
    ctx_mid = args.context + args.warmup + args.steps // 2
    nbytes, wbytes, kv_per_tok = decode_bytes(eng, args.batch, ctx_mid)
    achieved = nbytes / (ms_step * 1e-3) / 1e9
    e2e_value, h2d, d2h = time_e2e(eng, args.batch, args.context, args.steps, args.warmup)

    name = f"Qwen2.5-{args.sizes.upper()} sizes"
    out = {"metric": f"decode tok/s at batch {args.batch}, {args.context}-token contexts ({name})", "value": round(value, 1),
           "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
           "higher_is_better": True, "scaling": "weak",
           "vs_baseline": round(value / PUBLISHED_TOK_S[args.batch], 2) if args.sizes == "1.5b" and args.batch in PUBLISHED_TOK_S else None,
           "baseline": PUBLISHED_NOTE, "dtype": "bf16",
           "data": "synthetic: random weights N(0,0.02), random cache contents, fixed token ids",
           "config": {"model": name, "layers": n_layers, "layers_of_model": CONFIG["num_hidden_layers"],
                      "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                      "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                      "global_batch": args.batch, "seq_len": args.context, "page_size": 16,
                      "tied_head": bool(cfg["tie_word_embeddings"]), "parallelism": "single GPU",
                      "l2": f"inputs larger than L2 ({wbytes / 1e9:.1f} GB weights per step)",
                      "peaks": pk["source"]},
           "clocks": clk, "gpu_launches": launches,
           "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
           "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                        "frac": round(achieved / pk["hbm_gbs"], 4)}}
    if not args.no_points:
        points = {}
        fracs = {}
        for b in point_batches:
            n_b = max(16, args.steps // 2)
            ms_b, _ = time_decode(eng, b, args.context, n_b, args.warmup, ops.kernel_launches)
            points[f"decode_b{b}"] = round(b * 1e3 / ms_b, 1)
            fracs[f"decode_b{b}"] = round(decode_bytes(eng, b, args.context + args.warmup + n_b // 2)[0] / (ms_b * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        out["points"] = points
        out["points_roofline_frac"] = fracs
        T = 2048
        ms_p = time_prefill(eng, T, 5, 3)
        fl = prefill_flops(cfg, n_layers, T)
        out["prefill"] = {"value": round(T * 1e3 / ms_p, 1), "tokens": T, "ms": round(ms_p, 3),
                          "frac": round(fl / (ms_p * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
