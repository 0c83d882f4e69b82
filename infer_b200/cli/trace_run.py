"""Trace replay: feeds given token ids through a model step by step and writes logits. Samples nothing.

It drives the framework's own model, step function, cache manager and kernels: the ones generation uses.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--format f32|npy|both]

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch.  ``end`` names requests that are finished after the step; their
pages and slot go back.  For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits at
the wanted places, in the order of the entries and of ``want``, little-endian float32 [wanted, vocab].
With ``--format npy`` (or ``both``) the same rows are written as ``<out>/<step>.npy``, a NumPy array file of
float32 [wanted, vocab] (the reference's tools exchange arrays in that format, src/npy.h).
After every step a line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

PAGE_SIZE = 16
ROUND_TO = 64          # each live request's token count is rounded up to this many when sizing the pool
MAX_LIVE = 4


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each request rounded up to 64)")
    ap.add_argument("--max-requests", type=int, default=MAX_LIVE, help="live requests at a time (default 4)")
    ap.add_argument("--format", default="f32", choices=["f32", "npy", "both"],
                    help="logit files: raw little-endian float32 (<step>.f32), NumPy (<step>.npy), or both")
    args = ap.parse_args(argv)

    print("[trace_run] loading the framework (kernels are compiled at first use) ...", file=sys.stderr, flush=True)
    import numpy as np
    import torch
    from infer_b200.engine import Engine, StepEntry

    os.makedirs(args.out, exist_ok=True)
    engine = Engine.from_folder(args.model, dtype=args.dtype, device="cuda:0", max_tokens=args.max_tokens,
                                max_requests=args.max_requests, page_size=PAGE_SIZE,
                                max_seq_len=args.max_tokens)
    print(f"[trace_run] ready: {engine.spec.architecture}, dtype {args.dtype}, "
          f"{engine.cache.pages_total()} pages of {PAGE_SIZE}", file=sys.stderr, flush=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            if not engine.has_request(e["id"]):
                engine.add_request(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e.get("want", [])))
        logits = engine.step(entries)
        if logits.shape[0] > 0:
            arr = logits.to("cpu", torch.float32).numpy().astype("<f4", copy=False)
            if args.format in ("f32", "both"):
                arr.tofile(os.path.join(args.out, f"{step}.f32"))
            if args.format in ("npy", "both"):
                np.save(os.path.join(args.out, f"{step}.npy"), arr)
        else:
            torch.cuda.synchronize()
        engine.check_status()
        for rid in rec.get("end", []):
            if engine.has_request(rid):
                engine.end_request(rid)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
