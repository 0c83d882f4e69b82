"""Generation demo in the manner of the reference's main_generate (src/main_generate.cpp:7-15,41-47).

    bin/generate [prompt=0] [n_new=16] [device=gpu] [gemm=mine|plain] [cache=on|off] [attn=split|plain]
                 [step=fused|unfused] [--model DIR | --random SPEC [--weights-seed S]] [--dtype bfloat16|float32]
                 [--prompt-ids 1,2,3] [--prompt-len N] [--temp T] [--top-k K] [--top-p P] [--seed S] [--max N]
                 [--max-seq N] [--kv-blocks N] [--chunk N]

Positional arguments keep the reference's order and meaning: ``prompt`` is the index of a built-in prompt (the
reference reads golden token ids by index; here prompt i is a seeded list of 5 + 7*i random ids, or the ids given
with --prompt-ids), ``n_new`` the tokens to generate, ``device`` must be gpu (there is no CPU path), ``gemm=plain``
/ ``attn=plain`` / ``step=unfused`` switch the fast matrix, attention and fused kernels off in favour of the plain
ones (the reference's mine / naive choice), ``cache=off`` recomputes the whole sequence for every token (the
reference's no-cache baseline). The model folder comes from --model or the environment variable LLM_MODEL
(src/model_select.h:20-28). --temp/--top-k/--top-p/--seed/--max are the reference's chat options
(src/main_chat.cpp:61-71); --max overrides n_new. --random builds a model with seeded random weights instead of
reading one: SPEC is a preset (tiny-a, tiny-b, qwen2.5-1.5b, qwen2.5-7b, qwen2.5-14b), a config.json, or an inline
JSON object of config.json keys. --max-seq is the per-sequence cap, --kv-blocks the size of the page pool in pages of
16 positions (default: max-seq positions, kernels/batch_gpu.cu:92-95), --chunk the most prompt tokens one step takes.
Prints the ids, the prefill time and decode tokens/s.
"""
from __future__ import annotations

import argparse
import os
import sys
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="generate", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("positional", nargs="*", help="prompt n_new device gemm cache attn step (see above)")
    ap.add_argument("--model", default=os.environ.get("LLM_MODEL"))
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--prompt-ids", default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--temp", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", "--sample-seed", dest="seed", type=int, default=0, help="seed of the sampling noise")
    ap.add_argument("--max", type=int, default=None)
    ap.add_argument("--max-seq", type=int, default=4096)
    ap.add_argument("--random", default=None, metavar="SPEC", help="random weights: a preset, a config.json or a JSON object")
    ap.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights (--random)")
    ap.add_argument("--kv-blocks", type=int, default=0, help="pages of 16 positions in the cache pool (0: max-seq positions)")
    ap.add_argument("--chunk", type=int, default=512, help="most prompt tokens a step takes")
    args = ap.parse_args(argv)
    names = ["prompt", "n_new", "device", "gemm", "cache", "attn", "step"]
    opt = {"prompt": "0", "n_new": "16", "device": "gpu", "gemm": "mine", "cache": "on", "attn": "split", "step": "fused"}
    for i, v in enumerate(args.positional):
        if "=" in v:
            k, v = v.split("=", 1)
            if k not in opt:
                ap.error(f"unknown option {k}")
            opt[k] = v
        elif i < len(names):
            opt[names[i]] = v
        else:
            ap.error("too many positional arguments")
    if args.random:
        args.model = None
    elif not args.model:
        ap.error("no model: give --model DIR, --random SPEC, or set LLM_MODEL")
    if opt["device"] != "gpu":
        print("generate: device=cpu is not available: this engine has no CPU path", file=sys.stderr)
        return 2
    n_new = args.max if args.max is not None else int(opt["n_new"])

    import numpy as np
    from infer_b200.engine.generation import LLM
    from infer_b200.engine import StepEntry
    kernels = {}
    if opt["gemm"] in ("plain", "naive"):
        kernels["linear"] = "plain"
    if opt["attn"] in ("plain", "naive"):
        kernels["attention"] = "plain"
    if opt["step"] == "unfused":
        kernels.update({"rope": "plain", "swiglu": "plain", "norm": "plain"})
    spec = weights = None
    if args.random:
        import torch
        from infer_b200.config import parse_config
        from infer_b200.models import load_preset
        from infer_b200.weights import expected_tensors, random_weights
        arch, typed = parse_config(load_preset(args.random))
        spec = arch.to_spec(typed)
        # the values of write_random_model (drawn on the CPU from (seed, tensor name)); models beyond two billion
        # parameters are drawn on the device instead, which is faster and gives another stream of numbers
        n_params = sum(int(torch.Size(shape).numel()) for shape, *_ in expected_tensors(spec).values())
        weights = random_weights(spec, args.weights_seed, torch.bfloat16, device="cuda" if n_params > 2e9 else "cpu")
        args.max_seq = min(args.max_seq, spec.max_positions)
        args.model = f"random:{args.random} (weights seed {args.weights_seed})"
    llm = LLM(None if spec is not None else args.model, dtype=args.dtype, slots=1, max_seq=args.max_seq, kernels=kernels,
              spec=spec, weights=weights, kv_blocks=args.kv_blocks, max_batch_tokens=max(1, args.chunk))
    del weights
    V = llm.engine.spec.vocab_size
    if args.prompt_ids:
        ids = [int(t) for t in args.prompt_ids.split(",")]
    else:
        pi = int(opt["prompt"])
        n = args.prompt_len or 5 + 7 * pi
        ids = np.random.default_rng(pi).integers(0, V, n).tolist()
    print(f"model {args.model}")
    print(f"prompt {opt['prompt']} ({len(ids)} tokens), device=gpu gemm={opt['gemm']} cache={opt['cache']} "
          f"attn={opt['attn']} step={opt['step']} dtype={args.dtype}:")
    import torch
    if opt["cache"] == "off":
        eng, out = llm.engine, []
        t0 = time.perf_counter()
        seq = list(ids)
        t_first = None
        for i in range(n_new):
            eng.add_request("r")
            logits = eng.step([StepEntry("r", seq, [len(seq) - 1])])
            tok = int(llm.batch_engine.sampler.sample(
                logits, [type("P", (), dict(temperature=args.temp, seed=args.seed, top_k=args.top_k, top_p=args.top_p))()],
                [len(seq) - 1]).item())
            eng.end_request("r")
            if t_first is None:
                t_first = time.perf_counter() - t0
            out.append(tok)
            seq.append(tok)
        total = time.perf_counter() - t0
    else:
        stamps = []
        t0 = time.perf_counter()
        out = llm.generate([ids], max_new=n_new, temperature=args.temp, seed=args.seed, top_k=args.top_k,
                           top_p=args.top_p, on_token=lambda rid, tok: stamps.append(time.perf_counter()))[0]
        total = time.perf_counter() - t0
        t_first = (stamps[0] - t0) if stamps else total
    print("ids:", " ".join(str(t) for t in out))
    rest = max(1e-9, total - t_first)
    print(f"prefill {t_first:.4f} s, decode {max(0, len(out) - 1) / rest:.1f} tok/s ({len(out)} tokens, {total:.3f} s)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
