"""The command lines as a user runs them, as subprocesses on a model folder that the test writes: bin/generate (the
reference's main_generate, src/main_generate.cpp:7-15,41-47), bin/serve_bench (main_serve_bench,
src/main_serve_bench.cpp:15-27) and the kernel timing tool. Greedy ids in float32 equal the plain implementation's."""
import json
import os
import re
import subprocess
import sys

import pytest
import torch

import helpers as H
import plain_model as pm

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SEED = 13


def _run(args, timeout=600):
    env = dict(os.environ)
    env.pop("LLM_MODEL", None)
    proc = subprocess.run([sys.executable] + args, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert proc.returncode == 0, (proc.stdout[-1500:], proc.stderr[-1500:])
    return proc.stdout


def _ids(stdout):
    line = next(l for l in stdout.splitlines() if l.startswith("ids:"))
    return [int(t) for t in line.split()[1:]]


@pytest.fixture(scope="module")
def model_b(tmp_path_factory):
    from infer_b200.weights import write_random_model
    folder = tmp_path_factory.mktemp("cli") / "model_b"
    write_random_model(str(folder), H.TINY["b"], SEED, torch.bfloat16)
    return str(folder)


def test_generate_on_a_model_folder_equals_the_plain_implementation(model_b):
    cfg = H.TINY["b"]
    prompt = H.random_ids(cfg, 21, 1)
    W = H.as_compute(H.make_weights(cfg, SEED, torch.bfloat16), torch.float32)
    want = pm.greedy_decode(cfg, W, prompt, 10)
    gen = os.path.join(ROOT, "bin", "generate")
    ids = ",".join(map(str, prompt))
    out = _run([gen, "0", "10", "--model", model_b, "--dtype", "float32", "--prompt-ids", ids, "--max-seq", "64"])
    assert _ids(out) == want
    assert re.search(r"prefill [0-9.]+ s, decode [0-9.]+ tok/s", out)
    # the prompt in portions of 5 tokens, a pool of 3 pages (48 positions for 31): the same ids
    out = _run([gen, "0", "10", "--model", model_b, "--dtype", "float32", "--prompt-ids", ids, "--max-seq", "64",
                "--chunk", "5", "--kv-blocks", "3"])
    assert _ids(out) == want
    # the reference's switches: plain kernels, and recomputing the whole sequence for every token
    out = _run([gen, "0", "10", "gpu", "plain", "off", "plain", "unfused", "--model", model_b, "--dtype", "float32",
                "--prompt-ids", ids, "--max-seq", "64"])
    assert _ids(out) == want
    # the model folder from the environment, as the reference's tools take it (src/model_select.h:20-28)
    env = dict(os.environ, LLM_MODEL=model_b)
    proc = subprocess.run([sys.executable, gen, "n_new=4", "--dtype", "float32", "--prompt-ids", ids, "--max-seq", "64"],
                          capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0 and _ids(proc.stdout) == want[:4]


def test_generate_with_random_weights_from_a_preset():
    from infer_b200.config import parse_config
    from infer_b200.models import load_preset
    from infer_b200.weights import random_weights
    cfg = load_preset("tiny-a")
    arch, typed = parse_config(cfg)
    W = H.as_compute(random_weights(arch.to_spec(typed), 4, torch.bfloat16), torch.float32)
    prompt = H.random_ids(cfg, 9, 2)
    want = pm.greedy_decode(cfg, W, prompt, 8)
    gen = os.path.join(ROOT, "bin", "generate")
    ids = ",".join(map(str, prompt))
    out = _run([gen, "--random", "tiny-a", "--weights-seed", "4", "--dtype", "float32", "--prompt-ids", ids, "--max", "8"])
    assert _ids(out) == want
    # seeded sampling: the same seed gives the same ids, another seed others; bfloat16 runs through the fast kernels
    a = _ids(_run([gen, "--random", "tiny-a", "--weights-seed", "4", "--prompt-ids", ids, "--max", "12", "--temp", "0.9", "--seed", "5"]))
    b = _ids(_run([gen, "--random", "tiny-a", "--weights-seed", "4", "--prompt-ids", ids, "--max", "12", "--temp", "0.9", "--sample-seed", "5"]))
    c = _ids(_run([gen, "--random", "tiny-a", "--weights-seed", "4", "--prompt-ids", ids, "--max", "12", "--temp", "0.9", "--seed", "6"]))
    assert a == b and a != c and len(a) == 12
    # device=cpu is refused, as this engine has no CPU path
    proc = subprocess.run([sys.executable, gen, "0", "4", "cpu", "--random", "tiny-a"], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 2 and "no CPU path" in proc.stderr


def test_serve_bench_runs_continuous_and_static(model_b, tmp_path):
    events = tmp_path / "events.jsonl"
    out = _run([os.path.join(ROOT, "bin", "serve_bench"), "--model", model_b, "n=6", "slots=1,3", "max_new=6", "max_seq=64",
                "prompt_len=9", "chunk=16", f"events={events}", "tag=test"])
    recs = [json.loads(l) for l in out.splitlines() if l.startswith("{")]
    assert [(r["slots"], r["mode"]) for r in recs] == [(1, "continuous"), (1, "static"), (3, "continuous"), (3, "static")]
    want_tokens = sum(max(1, 6 // 2 + (i * 7) % 7) for i in range(6))
    assert all(r["tokens"] == want_tokens and r["tok_s"] > 0 and r["tag"] == "test" for r in recs)
    kinds = {json.loads(l)["kind"] for l in events.read_text().splitlines()}
    assert {"admit", "step", "retire"} <= kinds
    # a pool too small for all slots at once: requests are preempted and still all finish
    out = _run([os.path.join(ROOT, "bin", "serve_bench"), "random=tiny-b", "n=5", "slots=3", "max_new=20", "max_seq=64",
                "prompt_len=12", "kv_blocks=5", "modes=continuous", "dtype=float32"])
    rec = [json.loads(l) for l in out.splitlines() if l.startswith("{")][0]
    assert rec["pages"] == 5 and rec["preemptions"] > 0 and rec["tokens"] == sum(max(1, 10 + (i * 7) % 21) for i in range(5))


def test_kernel_bench_times_a_kernel():
    out = _run(["-m", "infer_b200.cli.kernel_bench", "linear", "--M", "8", "--N", "512", "--K", "256", "--reps", "3"])
    rec = json.loads(out.strip().splitlines()[-1])
    assert rec["what"] == "linear" and rec["us_median"] > 0 and "error" not in rec
    out = _run(["-m", "infer_b200.cli.kernel_bench", "attention", "--batch", "2", "--context", "100", "--heads", "4", "--kv-heads", "2",
                "--head-dim", "64", "--fused", "--reps", "3"])
    assert json.loads(out.strip().splitlines()[-1])["us_median"] > 0
