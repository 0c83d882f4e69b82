"""bin/trace_run as a user runs it: a model folder, steps on standard input, logits in files."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SEED = 9


def _replay(tmp_path, name, dtype, steps, max_tokens, fmt=None):
    from infer_b200.weights import write_random_model
    model = tmp_path / "model"
    write_random_model(str(model), H.TINY[name], SEED, H.STORED_DTYPE[name])
    out = tmp_path / f"out_{dtype}"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(model), "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(max_tokens)] + (["--format", fmt] if fmt else []),
                          input=H.trace_to_jsonl(steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    V = H.TINY[name]["vocab_size"]
    got, pos = {}, {}
    for i, st in enumerate(steps):
        n_want = sum(len(w) for _, _, w in st["entries"])
        path = out / f"{i}.f32"
        if n_want == 0:
            assert not path.exists()
            for rid, toks, _ in st["entries"]:
                pos[rid] = pos.get(rid, 0) + len(toks)
            continue
        arr = np.fromfile(path, dtype="<f4").reshape(n_want, V)
        if fmt == "both":
            saved = np.load(out / f"{i}.npy")
            assert saved.dtype == np.float32 and saved.shape == (n_want, V) and np.array_equal(saved, arr)
        r = 0
        for rid, toks, want in st["entries"]:
            for w in want:
                got.setdefault(rid, {})[pos.get(rid, 0) + w] = arr[r]
                r += 1
            pos[rid] = pos.get(rid, 0) + len(toks)
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_trace_through_the_program(tmp_path, dtype):
    name = "b"
    cfg = H.TINY[name]
    lengths = [70, 40, 100, 33, 64, 50]
    ids = {f"r{i}": H.random_ids(cfg, n, 600 + i) for i, n in enumerate(lengths)}
    reqs = {rid: (t, max(2, len(t) - 32)) for rid, t in ids.items()}
    steps = H.trace_mixed(reqs, 320, seed=3)
    # leave some places unasked, and one step with nothing wanted
    steps[0]["entries"] = [(r, t, []) for r, t, w in steps[0]["entries"]]
    got = _replay(tmp_path, name, dtype, steps, 320)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    for rid, t in ids.items():
        ref = H.oracle(cfg, SEED, H.STORED_DTYPE[name], tdt, t)
        rows = sorted(got[rid])
        g = np.stack([got[rid][p] for p in rows])
        if dtype == "float32":
            H.check_f32(g, ref[rows], rid)
        else:
            H.check_bf16(g, ref[rows], H.oracle(cfg, SEED, H.STORED_DTYPE[name], tdt, t, torch.bfloat16)[rows], rid)


def test_whole_and_tail_agree_through_the_program(tmp_path):
    name = "c"
    ids = {"x": H.random_ids(H.TINY[name], 90, 700)}
    a = _replay(tmp_path, name, "float32", H.trace_whole(ids), 128)["x"]
    b = _replay(tmp_path, name, "float32", H.trace_tail(ids, 32), 128, fmt="both")["x"]
    ref = H.oracle(H.TINY[name], SEED, H.STORED_DTYPE[name], torch.float32, ids["x"])
    for p in b:
        assert np.array_equal(a[p], b[p])
        H.check_f32(b[p][None], ref[p][None], f"position {p}")
