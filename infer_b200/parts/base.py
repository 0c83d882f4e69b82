"""Interfaces of the parts a layer is made of, and the registries that map a spec's ``kind`` to a class.

A part is built from its own ``PartSpec`` alone: it knows its sizes and constants, the local
names and shapes of its parameters, and what it needs from the cache manager.  It does not know
which architecture, which layer index or which model it is in.

To add a part: subclass the matching interface below, decorate it with
``@register_mixer("name")`` (or the feed-forward / norm / position / block / embedding / head
variant), and let an architecture's ``to_spec`` name that kind.  No framework file changes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional, Tuple

import torch

from ..config.specs import PartSpec


# ----------------------------------------------------------------------------- cache needs

@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every position (or of the last ``window`` positions) in pages."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None     # None: all positions stay; n: only the last n are ever read


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size state per request, zeroed when the request is admitted.

    shapes maps a state tensor's name to (shape without the slot dimension, torch dtype)."""
    shapes: Mapping[str, Tuple[Tuple[int, ...], torch.dtype]]


# ----------------------------------------------------------------------------- interfaces

class Part:
    """Common surface of every part."""

    def __init__(self, spec: PartSpec, runtime: "Runtime"):
        self.spec = spec
        self.rt = runtime

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[int, ...]]:
        """Local parameter name -> shape, as the checkpoint stores them under ``spec.prefix``."""
        return {}

    @classmethod
    def init_params(cls, spec: PartSpec, name: str, shape: Tuple[int, ...], gen: torch.Generator) -> torch.Tensor:
        """Random value for one parameter (float32, on the generator's device): matrices and
        biases N(0, 0.02).  Parts whose parameters want another distribution override this."""
        return torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device) * 0.02

    # False: the part's forward() cannot be captured into a CUDA graph (it reads device memory on the host, allocates
    # outside the stream's pool, or launches by data). The engine then runs every step of the model eagerly.
    graph_safe = True

    def load(self, params: Mapping[str, torch.Tensor]) -> None:
        """Receives the part's parameters (CPU tensors in their stored dtype) and moves what it
        needs to the device, in the layout its kernels want."""


class DeferredNorm:
    """The float32 rows ``h`` with a norm that has not been applied yet. A part that declares
    ``accepts_deferred_norm`` may receive this instead of the normalised tensor and hand it to a kernel that
    normalises on the fly; ``materialize()`` applies the norm the ordinary way."""

    def __init__(self, norm: "Norm", h: torch.Tensor):
        self.norm, self.h = norm, h
        self._value = None

    @property
    def shape(self):
        return self.h.shape

    def materialize(self) -> torch.Tensor:
        if self._value is None:
            self._value = self.norm.forward(self.h)
        return self._value


class Norm(Part):
    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """x [rows, size] float32 (the residual stream) -> normalised rows in the compute dtype."""
        raise NotImplementedError


class PositionEncoding(Part):
    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        """Encodes positions into q [T, heads, head_dim] and k [T, kv_heads, head_dim] in place.
        positions: int32 [T], absolute."""
        raise NotImplementedError

    def rotary_tables(self):
        """(cos, sin) float32 [max_positions, head_dim/2] if this encoding is a half-split rotation
        that a mixer's fused kernel may apply itself; None otherwise."""
        return None


class Mixer(Part):
    accepts_deferred_norm = False    # True: forward() may get a DeferredNorm as x

    def cache_need(self):
        """PagedKVNeed, StateNeed or None."""
        return None

    def forward(self, x: torch.Tensor, step: "StepContext", cache: Any, residual: torch.Tensor,
                write_cache: bool = True) -> torch.Tensor:
        """x: normalised rows [T, hidden] in the compute dtype; residual: float32 [T, hidden].
        Returns residual + mixer(x) as float32 [T, hidden] (it may overwrite ``residual``).
        ``cache`` is what the cache manager made for this part's need: a ``PagedKVView``,
        a dict of state tensors [slots, ...], or None."""
        raise NotImplementedError


class FeedForward(Part):
    accepts_deferred_norm = False

    def forward(self, x: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        """Returns residual + feed_forward(x), float32 [T, hidden] (may overwrite ``residual``)."""
        raise NotImplementedError


class Embedding(Part):
    """Token ids -> float32 rows of the residual stream."""

    def forward(self, step: "StepContext") -> torch.Tensor:
        """float32 [T, hidden] for ``step.token_ids`` (an id of -1 stands for the request's last sampled token, kept
        on the device in ``step.feedback[step.seg_slot[step.token_seg[t]]]``)."""
        raise NotImplementedError

    def table(self) -> Optional[torch.Tensor]:
        """The [vocab, hidden] matrix on the device, for a head that is tied to it; None if there is none."""
        return None


class Head(Part):
    """Normalised rows -> float32 logits [rows, vocab]."""

    def tie(self, embedding: Embedding) -> None:
        """Called once after loading, with the model's embedding part; a tied head takes its matrix from there."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """An arrangement of parts into a layer. ``parts`` maps the slot names of the layer's spec to the built and
    loaded parts, in the spec's order; each is also an attribute of the block under its slot name. A block class
    defines which slots it wants and how ``forward`` runs them."""

    def __init__(self, **parts: Part):
        self.parts: Dict[str, Part] = dict(parts)
        for slot, part in parts.items():
            setattr(self, slot, part)

    def cache_need(self):
        """What the layer needs from the cache manager per run-order entry: the need of its one part that has one."""
        needs = [n for n in (p.cache_need() for p in self.parts.values() if hasattr(p, "cache_need")) if n is not None]
        if len(needs) > 1:
            raise ValueError("a block with more than one stateful part must define cache_need() itself")
        return needs[0] if needs else None

    def forward(self, h: torch.Tensor, step: "StepContext", cache: Any, write_cache: bool) -> torch.Tensor:
        raise NotImplementedError


# ----------------------------------------------------------------------------- registries

_REGISTRIES: Dict[str, Dict[str, type]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {},
                                           "embedding": {}, "head": {}}


def _register(family: str, name: str) -> Callable[[type], type]:
    def deco(cls: type) -> type:
        if name in _REGISTRIES[family] and _REGISTRIES[family][name] is not cls:
            raise ValueError(f"{family} kind {name!r} is already registered")
        _REGISTRIES[family][name] = cls
        return cls
    return deco


def register_mixer(name: str): return _register("mixer", name)
def register_feed_forward(name: str): return _register("feed_forward", name)
def register_norm(name: str): return _register("norm", name)
def register_position(name: str): return _register("position", name)
def register_block(name: str): return _register("block", name)
def register_embedding(name: str): return _register("embedding", name)
def register_head(name: str): return _register("head", name)


def unregister(family: str, name: str) -> None:
    _REGISTRIES[family].pop(name, None)


def part_class(family: str, kind: str) -> type:
    try:
        return _REGISTRIES[family][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[family])) or "(none)"
        raise KeyError(f"no {family} part of kind {kind!r} is registered; known: {known}") from None


def build_part(family: str, spec: PartSpec, runtime: "Runtime") -> Part:
    return part_class(family, spec.kind)(spec, runtime)
