"""What every part needs to know about where and how it runs: device, compute dtype, kernel choice.

``dtype`` is the compute dtype of the whole model: ``torch.bfloat16`` is the serving path
(bfloat16 matrices, activations and cache; float32 residual stream, norms, softmax, rotation and
logits), ``torch.float32`` is the true 32-bit path (every tensor float32, plain FFMA kernels only).

``kernels`` chooses, per operation, between the fast kernel ("auto": the fast kernel where it
accepts the shape, else the plain one) and the plain kernel ("plain").  Tests use it to check one
fast kernel after the other inside the whole model.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict

import torch

OPERATIONS = ("linear", "attention", "norm", "rope", "swiglu", "embedding")


@dataclass
class Runtime:
    dtype: torch.dtype = torch.bfloat16
    device: torch.device = field(default_factory=lambda: torch.device("cuda", 0))
    kernels: Dict[str, str] = field(default_factory=dict)
    max_seq_len: int = 0          # longest sequence the engine will hold (sizes position tables); 0 = the model's limit

    def __post_init__(self):
        if self.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype must be bfloat16 or float32, not {self.dtype}")
        self.device = torch.device(self.device)
        if self.device.type != "cuda":
            raise RuntimeError("infer_b200 runs on a CUDA device only; there is no CPU path")
        for k, v in self.kernels.items():
            if k not in OPERATIONS or v not in ("auto", "plain"):
                raise ValueError(f"kernels[{k!r}]={v!r}: operations are {OPERATIONS}, choices 'auto' or 'plain'")

    def fast(self, op: str) -> bool:
        """True if the fast kernel of this operation may be used."""
        return self.dtype == torch.bfloat16 and self.kernels.get(op, "auto") == "auto"


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
             "f32": torch.float32}
    try:
        return table[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}") from None
