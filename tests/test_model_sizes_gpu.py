"""The layer sizes of the real models (Qwen2.5-1.5B / 7B / 14B: widths 1536 / 3584 / 5120, none a power of two,
28 / 40 heads in groups of 7 / 5, intermediate 8960 / 18944 / 13824), with one or two layers and a small vocabulary
so that the plain implementation stays fast: the kernels meet the K and N they serve in production, in float32 and in
bfloat16, for a prompt taken whole, then decoded one by one beside a second request."""
import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu
SEED = 3

SIZES = {
    "1.5b": dict(architectures=["Qwen2ForCausalLM"], hidden_size=1536, num_hidden_layers=2, num_attention_heads=12,
                 num_key_value_heads=2, intermediate_size=8960, vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-6,
                 max_position_embeddings=4096, tie_word_embeddings=True, use_sliding_window=False),
    "7b": dict(architectures=["Qwen2ForCausalLM"], hidden_size=3584, num_hidden_layers=1, num_attention_heads=28,
               num_key_value_heads=4, intermediate_size=18944, vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-6,
               max_position_embeddings=4096, tie_word_embeddings=False, use_sliding_window=False),
    "14b": dict(architectures=["Qwen2ForCausalLM"], hidden_size=5120, num_hidden_layers=1, num_attention_heads=40,
                num_key_value_heads=8, intermediate_size=13824, vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-5,
                max_position_embeddings=4096, tie_word_embeddings=False, use_sliding_window=False),
}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", list(SIZES))
def test_real_layer_sizes(name, dtype):
    from infer_b200.engine import Engine
    cfg = SIZES[name]
    W = H.make_weights(cfg, SEED, torch.bfloat16)
    eng = Engine(H.spec_of(cfg), W, dtype=dtype, max_tokens=512, max_requests=4)
    reqs = {"p": H.random_ids(cfg, 83, 1), "q": H.random_ids(cfg, 30, 2)}
    # p: 70 tokens at once (a tensor-core product of more than 64 rows), q: 20 tokens (one of fewer), then both decode
    # side by side (the streaming product with two rows), p alone at the end (one row)
    steps = [{"entries": [("p", reqs["p"][:70], [0, 69])], "end": []},
             {"entries": [("q", reqs["q"][:20], [19])], "end": []}]
    for i in range(10):
        steps.append({"entries": [("p", [reqs["p"][70 + i]], [0]), ("q", [reqs["q"][20 + i]], [0])],
                      "end": ["q"] if i == 9 else []})
    for i in range(80, 83):
        steps.append({"entries": [("p", [reqs["p"][i]], [0])], "end": ["p"] if i == 82 else []})
    got = H.run_trace(eng, steps)
    for rid, ids in reqs.items():
        ref = H.oracle(cfg, SEED, torch.bfloat16, dtype, ids)
        rows = sorted(got[rid])
        g = np.stack([got[rid][p] for p in rows])
        if dtype == torch.float32:
            H.check_f32(g, ref[rows], f"{name}/{rid}")
        else:
            refr = H.oracle(cfg, SEED, torch.bfloat16, dtype, ids, torch.bfloat16)
            H.check_bf16(g, ref[rows], refr[rows], f"{name}/{rid}")
    assert eng.cache.pages_in_use() == [0] * len(eng.cache.groups)
