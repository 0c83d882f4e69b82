"""The C handle API (infer_b200/csrc/capi.cpp): through its exported symbols from Python (ctypes), and from a C++ host
program that holds no Python object, against the plain implementation."""
import os
import subprocess
import sys
import sysconfig

import numpy as np
import pytest
import torch

import helpers as H
import plain_model as pm

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SEED = 21


def test_an_engine_that_cannot_be_made_gives_a_message():
    """Needs no GPU: a missing folder (or, without a GPU, the engine's own refusal) comes back as an error string."""
    from infer_b200.capi import CEngine, CEngineError
    from infer_b200.csrc.build import BuildError
    try:
        with pytest.raises(CEngineError) as e:
            CEngine(model_dir="/nonexistent/model/folder", dtype="float32")
    except BuildError as err:
        pytest.skip(f"the library cannot be compiled here: {str(err)[:80]}")
    assert "ib_engine_create" in str(e.value) and ("config.json" in str(e.value) or "CUDA" in str(e.value))


@pytest.mark.gpu
def test_steps_and_generation_through_the_c_symbols(tmp_path):
    from infer_b200.capi import CEngine, CEngineError
    from infer_b200.weights import write_random_model
    cfg = H.TINY["b"]
    folder = tmp_path / "model"
    write_random_model(str(folder), cfg, SEED, torch.bfloat16)
    W = H.as_compute(H.make_weights(cfg, SEED, torch.bfloat16), torch.float32)
    eng = CEngine(model_dir=str(folder), dtype="float32", slots=3, max_seq=64, kv_blocks=4, chunk=8)
    assert eng.vocab_size == cfg["vocab_size"]
    prompts = [H.random_ids(cfg, n, 50 + n) for n in (5, 19)]
    assert eng.generate(prompts, max_new=6) == [pm.greedy_decode(cfg, W, p, 6) for p in prompts]
    # steps by hand: a portion, then the rest beside another request's portion; logits against the plain model
    a, b = H.random_ids(cfg, 30, 1), H.random_ids(cfg, 20, 2)
    eng.add_request(1), eng.add_request(2)
    assert eng.step([(1, a[:17], [0, 16])]) == 2
    first = eng.logits()
    assert eng.step([(1, a[17:], [12]), (2, b[:9], [])]) == 1
    second = eng.logits()
    ref = pm.forward(cfg, W, a).numpy()
    H.check_f32(np.concatenate([first, second]), ref[[0, 16, 29]], "steps through the C API")
    # 4 pages in the pool: request 1 holds 2, request 2 one; a third request's 40 tokens do not fit, a short one does
    eng.add_request(3)
    with pytest.raises(CEngineError, match="pages"):
        eng.step([(3, H.random_ids(cfg, 40, 3), [39])])
    rows, ran = eng.step([(3, H.random_ids(cfg, 40, 3), [39]), (2, b[9:12], [2])], partial=True)
    assert (rows, ran) == (1, [False, True])
    H.check_f32(eng.logits(), pm.forward(cfg, W, b[:12]).numpy()[[11]], "partial step")
    with pytest.raises(CEngineError, match="not admitted"):
        eng.step([(77, [1], [0])])
    for r in (1, 2, 3):
        eng.end_request(r)
    eng.close()


@pytest.mark.gpu
def test_a_host_program_without_python_objects(tmp_path):
    from infer_b200.config import parse_config
    from infer_b200.csrc.build import compile_module
    from infer_b200.models import load_preset
    from infer_b200.weights import random_weights
    lib = compile_module("capi")
    exe = tmp_path / "capi_host"
    ver = sysconfig.get_config_var("LDVERSION") or sysconfig.get_python_version()
    libdir = sysconfig.get_config_var("LIBDIR")
    cmd = ["g++", "-O1", "-o", str(exe), os.path.join(ROOT, "tests", "capi_host.cpp"), f"-L{libdir}", "-Wl,--no-as-needed", f"-lpython{ver}", "-ldl",
           f"-Wl,-rpath,{libdir}"]
    built = subprocess.run(cmd, capture_output=True, text=True)
    if built.returncode != 0:
        pytest.skip(f"no libpython to link a host program against: {built.stderr[-200:]}")
    # the host program's interpreter must find this package and the packages of this interpreter (torch, numpy)
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT] + [p for p in sys.path if p]))
    proc = subprocess.run([str(exe), lib, "tiny-a"], capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, (proc.stdout[-1000:], proc.stderr[-2000:])
    cfg = load_preset("tiny-a")
    arch, typed = parse_config(cfg)
    W = H.as_compute(random_weights(arch.to_spec(typed), 4, torch.bfloat16), torch.float32)
    prompt = [3, 200, 17, 42, 9, 9, 101]
    lines = dict(l.split(" ", 1) for l in proc.stdout.strip().splitlines())
    assert [int(t) for t in lines["generated"].split()] == pm.greedy_decode(cfg, W, prompt, 8)
    ref = pm.forward(cfg, W, prompt).numpy()
    assert [int(t) for t in lines["argmax"].split()] == [int(ref[0].argmax()), int(ref[6].argmax())]
    assert "not admitted" in lines["error"]
