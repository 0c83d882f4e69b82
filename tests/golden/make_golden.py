"""Makes tests/golden/*.npy: logits and greedy tokens of the reference engine's OWN CPU forward pass
(RyanXiaoo/infer src/forward.cpp, compiled here out of tree with g++, nothing copied) on two tiny random
models of the architecture.  The plain implementation (tests/plain_model.py) is compared with these files.

Run once:  python tests/golden/make_golden.py <path to a checkout of RyanXiaoo/infer>

The reference reads bfloat16 tensors only (it never checks a tensor's dtype, src/model.cpp:18-29), so the
models are written in bfloat16; tests regenerate the same weights from the same seeds.
The reference requires head_dim == hidden_size / num_attention_heads and knows no sliding window, so the
golden models have neither.
"""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from infer_b200.weights import write_random_model  # noqa: E402  (only writes the random checkpoint)
import infer_b200.parts, infer_b200.models  # noqa: E402,F401

DRIVER = r"""
#include "forward.h"
#include "model.h"
#include <cstdio>
#include <cstdlib>
#include <vector>
int main(int argc, char** argv) {
    llm::Model model;
    model.load(argv[1]);
    std::vector<int64_t> ids;
    for (int i = 4; i < argc; i++) ids.push_back(std::atoll(argv[i]));
    std::vector<float> logits = llm::forward(model, ids, nullptr, false);
    FILE* f = std::fopen(argv[2], "wb");
    std::fwrite(logits.data(), sizeof(float), logits.size(), f);
    std::fclose(f);
    std::vector<int64_t> out = llm::greedy_decode(model, ids, std::atoi(argv[3]));
    for (int64_t t : out) std::printf("%lld ", (long long)t);
    std::printf("\n");
    return 0;
}
"""

CONFIGS = {
    "tiny_a": dict(architectures=["Qwen2ForCausalLM"], hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                   num_key_value_heads=2, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
                   rms_norm_eps=1e-6, max_position_embeddings=128, tie_word_embeddings=True),
    "tiny_b": dict(architectures=["Qwen2ForCausalLM"], hidden_size=96, num_hidden_layers=3, num_attention_heads=3,
                   num_key_value_heads=1, intermediate_size=224, vocab_size=320, rope_theta=1000000.0,
                   rms_norm_eps=1e-5, max_position_embeddings=256, tie_word_embeddings=False),
}
SEEDS = {"tiny_a": 11, "tiny_b": 12}
PROMPT_LEN = {"tiny_a": 33, "tiny_b": 40}
N_NEW = 8


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to a checkout of RyanXiaoo/infer>")
    ref = sys.argv[1]
    work = tempfile.mkdtemp(prefix="golden_")
    with open(os.path.join(work, "driver.cpp"), "w") as f:
        f.write(DRIVER)
    exe = os.path.join(work, "driver")
    srcs = [os.path.join(ref, "src", n) for n in ("forward.cpp", "model.cpp", "model_config.cpp", "loader.cpp")]
    subprocess.check_call(["g++", "-std=c++20", "-O2", "-I", os.path.join(ref, "src"), "-I", os.path.join(ref, "third_party"),
                           os.path.join(work, "driver.cpp")] + srcs + ["-o", exe])
    meta = {}
    for name, cfg in CONFIGS.items():
        folder = os.path.join(work, name)
        write_random_model(folder, cfg, SEEDS[name], torch.bfloat16)
        rng = np.random.default_rng(SEEDS[name])
        ids = rng.integers(0, cfg["vocab_size"], PROMPT_LEN[name]).tolist()
        raw = os.path.join(work, name + ".f32")
        out = subprocess.check_output([exe, folder, raw, str(N_NEW)] + [str(i) for i in ids], text=True)
        logits = np.fromfile(raw, dtype="<f4").reshape(len(ids), cfg["vocab_size"])
        np.save(os.path.join(HERE, name + "_logits.npy"), logits)
        meta[name] = {"config": cfg, "seed": SEEDS[name], "ids": ids, "greedy": [int(t) for t in out.split()]}
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(meta, f, indent=1)
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()
