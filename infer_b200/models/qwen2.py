"""Qwen2 / Qwen2.5 dense decoder: typed configuration and its translation into a ModelSpec.

The architecture, as the reference engine runs it (kernels/batch_gpu.cu:180-234,
src/forward.cpp:170-258): token table -> L x [RMSNorm -> grouped-query attention with bias on
Q/K/V, none on O, half-split rotary positions -> residual; RMSNorm -> SwiGLU feed-forward ->
residual] -> RMSNorm -> output matrix (its own, or the token table when tied).

Keys follow the architecture's own config.json.  The reference reads a subset of them
(src/model_config.cpp:18-45) and silently ignores the rest; here every key that changes the
computation is either honoured or refused with an error.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Dict, Mapping, Optional

from ..config.registry import Architecture, ConfigError, register_architecture
from ..config.specs import LayerCall, LayerSpec, ModelSpec, PartSpec

NAME = "Qwen2ForCausalLM"


@dataclass(frozen=True)
class Qwen2Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    vocab_size: int
    rope_theta: float
    rms_norm_eps: float
    max_position_embeddings: int
    head_dim: int                      # default hidden_size // num_attention_heads
    tie_word_embeddings: bool = False  # reference default (src/model_config.cpp:30)
    attention_bias: bool = True        # Q/K/V bias; default true for this architecture (model_config.cpp:41-42)
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"


_REQUIRED_INT = ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                 "intermediate_size", "vocab_size", "max_position_embeddings")
_REQUIRED_NUM = ("rope_theta", "rms_norm_eps")


def _need(raw: Mapping[str, Any], key: str, types, what: str):
    if key not in raw:
        raise ConfigError(f"config.json is missing required key {key!r}")
    v = raw[key]
    if isinstance(v, bool) or not isinstance(v, types):
        raise ConfigError(f"config.json key {key!r} must be {what}, got {v!r}")
    return v


def parse(raw: Mapping[str, Any]) -> Qwen2Config:
    vals: Dict[str, Any] = {}
    for k in _REQUIRED_INT:
        vals[k] = _need(raw, k, int, "an integer")
        if vals[k] <= 0:
            raise ConfigError(f"config.json key {k!r} must be positive, got {vals[k]}")
    for k in _REQUIRED_NUM:
        vals[k] = float(_need(raw, k, (int, float), "a number"))
        if vals[k] <= 0:
            raise ConfigError(f"config.json key {k!r} must be positive, got {vals[k]}")
    nh, nkv, H = vals["num_attention_heads"], vals["num_key_value_heads"], vals["hidden_size"]
    if nh % nkv != 0:
        raise ConfigError(f"num_attention_heads ({nh}) must be a multiple of num_key_value_heads ({nkv})")
    if raw.get("head_dim") is not None:
        vals["head_dim"] = _need(raw, "head_dim", int, "an integer")
    else:
        if H % nh != 0:
            raise ConfigError(f"hidden_size ({H}) is not a multiple of num_attention_heads ({nh}) and no head_dim is given")
        vals["head_dim"] = H // nh
    if vals["head_dim"] <= 0 or vals["head_dim"] % 2 != 0:
        raise ConfigError(f"head_dim must be positive and even for rotary positions, got {vals['head_dim']}")
    for k, default in (("tie_word_embeddings", False), ("attention_bias", True), ("use_sliding_window", False)):
        v = raw.get(k, default)
        if not isinstance(v, bool):
            raise ConfigError(f"config.json key {k!r} must be true or false, got {v!r}")
        vals[k] = v
    vals["hidden_act"] = raw.get("hidden_act", "silu")
    if vals["hidden_act"] != "silu":
        raise ConfigError(f"hidden_act {vals['hidden_act']!r} is not supported (this architecture's feed-forward uses 'silu')")
    if raw.get("rope_scaling") not in (None, {}):
        raise ConfigError("rope_scaling is not supported (the key must be absent or null)")
    for k in ("sliding_window", "max_window_layers", "eos_token_id", "bos_token_id"):
        v = raw.get(k)
        if isinstance(v, (list, tuple)) and k == "eos_token_id" and v:
            v = v[0]
        if v is not None and (isinstance(v, bool) or not isinstance(v, int)):
            raise ConfigError(f"config.json key {k!r} must be an integer or null, got {v!r}")
        vals[k] = v
    if vals["use_sliding_window"]:
        if not vals["sliding_window"] or vals["sliding_window"] <= 0:
            raise ConfigError("use_sliding_window is true but sliding_window is not a positive integer")
        if vals["max_window_layers"] is None:
            vals["max_window_layers"] = 0
        if vals["max_window_layers"] < 0:
            raise ConfigError("max_window_layers must not be negative")
    vals["torch_dtype"] = str(raw.get("torch_dtype", raw.get("dtype", "bfloat16")))
    return Qwen2Config(**vals)


def to_dict(cfg: Qwen2Config) -> Dict[str, Any]:
    d = asdict(cfg)
    d["architectures"] = [NAME]
    d["model_type"] = "qwen2"
    return d


def layer_window(cfg: Qwen2Config, layer: int) -> Optional[int]:
    """Layers below ``max_window_layers`` see every key; the others see the last ``sliding_window``."""
    if cfg.use_sliding_window and layer >= int(cfg.max_window_layers or 0):
        return int(cfg.sliding_window)
    return None


def to_spec(cfg: Qwen2Config) -> ModelSpec:
    rotary = PartSpec("rotary_half", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                      "max_positions": cfg.max_position_embeddings})
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = PartSpec("attention", {
            "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "qkv_bias": cfg.attention_bias, "window": layer_window(cfg, i),
            "softmax_scale": None, "position": rotary,
        }, p + "self_attn.")
        ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size,
                                  "intermediate_size": cfg.intermediate_size}, p + "mlp.")
        n1 = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, p + "input_layernorm.")
        n2 = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, p + "post_attention_layernorm.")
        layers.append(LayerSpec.standard("prenorm", mixer, ffn, n1, n2))
    spec = ModelSpec(
        architecture=NAME, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings, layers=tuple(layers),
        schedule=tuple(LayerCall(i, i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, "model.norm."),
        embedding=PartSpec("token_table", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "scale": None},
                           "model.embed_tokens."),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                      "tied": cfg.tie_word_embeddings}, "lm_head."),
        eos_token_id=cfg.eos_token_id)
    spec.validate()
    return spec


ARCHITECTURE = register_architecture(Architecture(NAME, parse, to_spec, to_dict))
