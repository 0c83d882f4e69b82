"""The reference arm of bench.py: builds RyanXiaoo/infer UNMODIFIED, out of tree, and runs its own serving bench.

The reference is a C++20/CUDA CMake project without Python packaging, and its CMakeLists.txt sets the CUDA
architecture to sm_120 with a plain ``set()`` that a command-line cache entry cannot override.  So the sources are
compiled file by file exactly as its two library targets list them (``engine_core``: src/*.cpp; ``engine_gpu``:
kernels/**/*.cu, CMakeLists.txt:19-31,124-141) with the same language standard and ``--default-stream per-thread``,
only the architecture flag differs (sm_100), and ``src/main_serve_bench.cpp`` is linked against them.  Nothing of
the reference is edited or copied into this repository: objects and the binary live under ``baseline/_ref/build``.

The run is the reference's stock path: ``main_serve_bench`` (src/main_serve_bench.cpp:84-140) with ``n = slots``
requests that share a prefix of ``context - 8`` tokens (``prefix=``), CUDA graphs on, continuous batching.  Its own
scheduler event log (``events=``, one JSON object per event) gives the duration of every scheduler step; the
steps in which every slot decodes and nothing is admitted are the decode steps.  The model folder (random weights
of the benchmark configuration, bfloat16 safetensors) and the five ``promptN_bf16.npz`` files it reads are written
by this module into ``baseline/_ref/root``, the ``MODEL_ROOT`` the binary is compiled with.
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys
import time
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
BUILD_DIR = os.path.join(REF_DIR, "build")
ROOT_DIR = os.path.join(REF_DIR, "root")           # MODEL_ROOT of the binary: models/<name>/, tests/golden/<name>/, bench/
SOURCES_INSTALLED = os.path.join(REF_DIR, "src")   # the install step's copy of the three source trees, unedited
SOURCES_ORIGIN = os.environ.get("INFER_REFERENCE_SRC", "/root/reference")

CORE = ["loader", "model_config", "npy", "model", "forward", "session", "tokenizer", "sampler", "scheduler",
        "block_pool", "serve", "quant"]
GPU = ["model_gpu", "session_gpu", "ops/embedding", "ops/rmsnorm", "ops/linear", "ops/rope", "ops/attention",
       "ops/elementwise", "ops/cache", "ops/batch", "ops/spec", "ops/gemm", "ops/quant", "batch_gpu", "spec_engine"]


class Unavailable(RuntimeError):
    """The reference cannot be built or run here; the message is one line for bench.py's record."""


def _say(msg: str) -> None:
    print(f"[reference] {msg}", file=sys.stderr, flush=True)


def _run(cmd, what):
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        tail = " | ".join(p.stdout.strip().splitlines()[-3:])
        raise Unavailable(f"{what} failed: {tail}"[:400])


def _cuda_home() -> str:
    for c in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if c and os.path.isfile(os.path.join(c, "bin", "nvcc")):
            return c
    nvcc = shutil.which("nvcc")
    if nvcc:
        return os.path.dirname(os.path.dirname(os.path.realpath(nvcc)))
    raise Unavailable("nvcc not found, the reference's CUDA sources cannot be compiled")


def install() -> str:
    """The offline install: places the reference's src/, kernels/ and third_party/ trees, unedited, under
    ``baseline/_ref/src`` (git-ignored), so that a machine without the original checkout can still link the bench
    against its own path, and builds everything. Returns the binary's path."""
    if os.path.isdir(os.path.join(SOURCES_ORIGIN, "src")) and not os.path.isdir(os.path.join(SOURCES_INSTALLED, "src")):
        for tree in ("src", "kernels", "third_party"):
            shutil.copytree(os.path.join(SOURCES_ORIGIN, tree), os.path.join(SOURCES_INSTALLED, tree))
    return build()


def build() -> str:
    """Compiles what is missing and links main_serve_bench; returns the binary's path."""
    global SOURCES
    SOURCES = next((s for s in (SOURCES_INSTALLED, SOURCES_ORIGIN) if os.path.isdir(os.path.join(s, "src"))), None)
    if SOURCES is None:
        raise Unavailable(f"the reference's sources are neither at {SOURCES_INSTALLED} nor at {SOURCES_ORIGIN}")
    os.makedirs(BUILD_DIR, exist_ok=True)
    cuda = _cuda_home()
    inc = ["-I", os.path.join(SOURCES, "third_party")]
    jobs = []
    for f in CORE:
        out = os.path.join(BUILD_DIR, f"core_{f}.o")
        if not os.path.isfile(out):
            jobs.append((["g++", "-std=c++20", "-O2"] + inc + ["-c", os.path.join(SOURCES, "src", f + ".cpp"), "-o", out], f))
    for f in GPU:
        out = os.path.join(BUILD_DIR, f"gpu_{os.path.basename(f)}.o")
        if not os.path.isfile(out):
            jobs.append(([os.path.join(cuda, "bin", "nvcc"), "-std=c++20", "-O3", "-gencode", "arch=compute_100,code=sm_100",
                          "--default-stream", "per-thread"] + inc + ["-c", os.path.join(SOURCES, "kernels", f + ".cu"), "-o", out], f))
    if jobs:
        _say(f"compiling {len(jobs)} reference sources for sm_100 ...")
        with ThreadPoolExecutor(max_workers=8) as pool:
            list(pool.map(lambda j: _run(j[0], f"compiling {j[1]}"), jobs))
    binary = os.path.join(BUILD_DIR, "main_serve_bench")
    if not os.path.isfile(binary) or _root_stamp() != ROOT_DIR:
        main_o = os.path.join(BUILD_DIR, "main_serve_bench.o")
        _run(["g++", "-std=c++20", "-O2"] + inc + ["-I", os.path.join(cuda, "include"), f'-DMODEL_ROOT="{ROOT_DIR}"',
              "-c", os.path.join(SOURCES, "src", "main_serve_bench.cpp"), "-o", main_o], "compiling main_serve_bench")
        objs = [os.path.join(BUILD_DIR, f"core_{f}.o") for f in CORE] + \
               [os.path.join(BUILD_DIR, f"gpu_{os.path.basename(f)}.o") for f in GPU]
        _run(["g++", "-o", binary, main_o] + objs + ["-L", os.path.join(cuda, "lib64"), "-lcudart", "-lcublas", "-lpthread"],
             "linking main_serve_bench")
        with open(os.path.join(BUILD_DIR, "model_root.txt"), "w") as f:
            f.write(ROOT_DIR)
    return binary


def _root_stamp() -> str:
    try:
        with open(os.path.join(BUILD_DIR, "model_root.txt")) as f:
            return f.read().strip()
    except OSError:
        return ""


def prepare_model(config: dict, name: str, seed: int = 0) -> str:
    """Random weights of ``config`` as a bfloat16 safetensors folder, and the five prompt files the bench reads."""
    import numpy as np
    import torch
    sys.path.insert(0, os.path.dirname(HERE))
    from infer_b200.config import parse_config
    from infer_b200.weights import random_weights
    from infer_b200.weights.safetensors_io import write_safetensors
    import infer_b200.models  # noqa: F401
    folder = os.path.join(ROOT_DIR, "models", name)
    os.makedirs(folder, exist_ok=True)
    os.makedirs(os.path.join(ROOT_DIR, "bench"), exist_ok=True)
    arch, typed = parse_config(config)
    spec = arch.to_spec(typed)
    if not os.path.isfile(os.path.join(folder, "model.safetensors")):
        _say(f"writing random weights for {name} ...")
        device = "cuda" if torch.cuda.is_available() else "cpu"
        W = {k: v.cpu() for k, v in random_weights(spec, seed, torch.bfloat16, device=device).items()}
        write_safetensors(os.path.join(folder, "model.safetensors"), W, metadata={"format": "pt"})
        del W
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(arch.to_dict(typed), torch_dtype="bfloat16"), f)
    golden = os.path.join(ROOT_DIR, "tests", "golden", name)
    os.makedirs(golden, exist_ok=True)
    rng = np.random.default_rng(1)
    for i in range(5):
        np.savez(os.path.join(golden, f"prompt{i}_bf16.npz"),
                 token_ids=rng.integers(0, spec.vocab_size, 8).astype(np.int64))
    return folder


def run_serve_bench(binary: str, name: str, slots: int, context: int, max_new: int, timeout: float = 900.0):
    """One run at ``slots`` concurrent sequences with contexts of ``context`` tokens. Returns a dict with the
    durations (ms, wall clock of the reference's scheduler) of the decode steps in which every slot is live, in
    order, and the longest admission (the first request's whole prompt; later ones reuse its cached prefix)."""
    events = os.path.join(ROOT_DIR, "bench", f"events_{name}_{slots}.jsonl")
    if os.path.exists(events):
        os.remove(events)
    env = dict(os.environ, LLM_MODEL=name)
    for k in ("LLM_QUANT", "LLM_DRAFT", "LLM_DRAFT_QUANT"):
        env.pop(k, None)
    # every request generates between max_new/2 and 3*max_new/2 tokens (src/main_serve_bench.cpp:137)
    max_seq = context + 2 * max_new + 32
    cmd = [binary, f"n={slots}", f"slots={slots}", f"max_new={max_new}", f"max_seq={max_seq}", f"prefix={context - 8}",
           "prefix_cache=1", "modes=continuous", "graphs=1", "attn=split", "gemm=mine", f"events={events}", "tag=b200"]
    t0 = time.time()
    try:
        p = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout,
                           cwd=ROOT_DIR)
    except subprocess.TimeoutExpired:
        raise Unavailable(f"main_serve_bench did not finish within {timeout:.0f} s at slots={slots}") from None
    if p.returncode != 0:
        tail = " | ".join(p.stdout.strip().splitlines()[-3:])
        raise Unavailable(f"main_serve_bench exited with {p.returncode}: {tail}"[:400])
    steps, admits = [], []
    with open(events) as f:
        for line in f:
            e = json.loads(line)
            if e["kind"] == "step":
                steps.append(e)
            elif e["kind"] == "admit":
                admits.append(e)
    last_admit = max((e["step"] for e in admits), default=0)
    full = [e["dur_ms"] for e in steps if e["step"] > last_admit and e["batch"] == slots]
    if len(full) < 8:
        raise Unavailable(f"the reference's event log has only {len(full)} full decode steps at slots={slots}")
    prompt_ms = max((e["dur_ms"] for e in admits), default=0.0)
    return {"slots": slots, "step_ms": full, "prompt_ms": prompt_ms, "prompt_tokens": context,
            "wall_s": time.time() - t0, "stdout": p.stdout}
