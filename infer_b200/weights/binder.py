"""Binds checkpoint tensors to a ModelSpec by tensor name, and makes seeded random checkpoints.

Which tensors a model has follows from its spec alone: the parameters that each part class
declares (``Part.param_shapes``) under the part's prefix, for the embedding, the head (none when
it is tied), the final norm and every part of every layer.  The reference resolves the same names one by
one and stops at the first problem (src/model.cpp:13-29,54-76); here every problem of a
checkpoint is collected into one error.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict, Mapping, Tuple

import torch

from ..config.registry import parse_config
from ..config.specs import ModelSpec, PartSpec
from ..parts.base import part_class
from .safetensors_io import open_checkpoint, write_safetensors


class WeightsError(ValueError):
    """Lists every missing tensor, unexpected tensor and wrong shape of a checkpoint."""

    def __init__(self, where: str, missing, unexpected, wrong_shape):
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        lines = [f"checkpoint {where} does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape for {name}: the configuration expects {list(want)}, the file has {list(got)}")
        super().__init__("\n".join(lines))


def _part_entries(family: str, spec: PartSpec):
    """(full tensor name, shape, part class, part spec, local name) of one part, nested parts included."""
    cls = part_class(family, spec.kind)
    for local, shape in cls.param_shapes(spec).items():
        yield spec.prefix + local, tuple(shape), cls, spec, local


def expected_tensors(spec: ModelSpec) -> Dict[str, Tuple[Tuple[int, ...], type, PartSpec, str]]:
    """Full tensor name -> (shape, owning part class, its spec, local name), over every part the spec lists."""
    out: Dict[str, Tuple] = {}
    for family, ps in spec.part_specs():
        for name, shape, cls, pspec, local in _part_entries(family, ps):
            if name in out and out[name][0] != shape:
                raise ValueError(f"two parts declare tensor {name} with different shapes")
            out[name] = (shape, cls, pspec, local)
    return out


def load_weights(model_dir: str, spec: ModelSpec) -> Dict[str, torch.Tensor]:
    """Every tensor the spec expects, by name, in its stored precision (see safetensors_io)."""
    want = expected_tensors(spec)
    files = open_checkpoint(model_dir)
    try:
        have = {}
        for f in files:
            for n in f.names():
                have.setdefault(n, f)
        missing = [n for n in sorted(want) if n not in have]
        unexpected = [n for n in sorted(have) if n not in want]
        wrong = [(n, want[n][0], have[n].shape(n)) for n in sorted(want)
                 if n in have and tuple(have[n].shape(n)) != tuple(want[n][0])]
        if missing or unexpected or wrong:
            raise WeightsError(model_dir, missing, unexpected, wrong)
        return {n: have[n].get(n) for n in want}
    finally:
        for f in files:
            f.close()


def check_weights(weights: Mapping[str, torch.Tensor], spec: ModelSpec, where: str = "(in memory)") -> None:
    want = expected_tensors(spec)
    missing = [n for n in sorted(want) if n not in weights]
    unexpected = [n for n in sorted(weights) if n not in want]
    wrong = [(n, want[n][0], tuple(weights[n].shape)) for n in sorted(want)
             if n in weights and tuple(weights[n].shape) != tuple(want[n][0])]
    if missing or unexpected or wrong:
        raise WeightsError(where, missing, unexpected, wrong)


def random_weights(spec: ModelSpec, seed: int, dtype: torch.dtype = torch.bfloat16,
                   device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Seeded random parameters: each tensor's values depend on (seed, tensor name) only, so the
    order of generation and the presence of other tensors do not matter.  Matrices, biases and
    tables are N(0, 0.02); a part class may choose otherwise (norm weights are 1 + N(0, 0.1)).
    Values are drawn in float32 and rounded to ``dtype``.  With ``device='cuda'`` the values are
    drawn on the device (a different stream of numbers than on the CPU)."""
    out = {}
    for name, (shape, cls, ps, local) in expected_tensors(spec).items():
        gen = torch.Generator(device=device)
        gen.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF)
        out[name] = cls.init_params(ps, local, shape, gen).to(dtype)
    return out


def write_random_model(folder: str, config: Mapping, seed: int, dtype: torch.dtype = torch.bfloat16) -> ModelSpec:
    """Writes ``config.json`` and ``model.safetensors`` for the architecture that ``config`` names."""
    arch, typed = parse_config(config)
    spec = arch.to_spec(typed)
    os.makedirs(folder, exist_ok=True)
    cfg = dict(arch.to_dict(typed))
    cfg["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}.get(dtype, str(dtype))
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=1, sort_keys=True)
    write_safetensors(os.path.join(folder, "model.safetensors"), random_weights(spec, seed, dtype),
                      metadata={"format": "pt", "seed": str(seed)})
    return spec
