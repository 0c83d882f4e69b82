"""Architecture-neutral descriptions of a model: parts, layers, and the order they run in.

A registered architecture turns its own ``config.json`` keys into these specs; everything
below the registry (weights binder, cache manager, parts, engine) reads only the specs and
never the architecture's name.  A spec is plain data: a ``kind`` that selects a registered
part class, the sizes and constants of that part, and the tensor-name prefix under which the
checkpoint stores the part's parameters.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Iterator, Mapping, Optional, Sequence, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer (a mixer, a feed-forward, a norm, or a position encoding).

    kind    name under which the part class is registered (``parts.registry``)
    params  the part's sizes and constants; the part's constructor validates them
    prefix  checkpoint tensor-name prefix of the part's parameters (``""`` if it has none)
    """
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


# The families a part can belong to; each has its own registry of kinds (``parts.base``).
FAMILIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement (``block`` kind) and the parts it arranges.

    parts maps a slot name, which the block class defines, to (family, PartSpec), in the order in which the block
    runs them. The framework does not know the slot names: it builds, loads and binds whatever the mapping holds,
    and hands the built parts to the block class by slot name. A block with a third norm, without a feed-forward,
    or with two mixers is another block class and another mapping, not another framework."""
    block: str
    parts: Mapping[str, Tuple[str, PartSpec]]

    def __post_init__(self):
        for slot, fp in self.parts.items():
            if not (isinstance(fp, tuple) and len(fp) == 2 and fp[0] in FAMILIES and isinstance(fp[1], PartSpec)):
                raise ValueError(f"layer slot {slot!r} must map to (family, PartSpec), got {fp!r}")

    @classmethod
    def standard(cls, block: str, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec,
                 feed_forward_norm: PartSpec) -> "LayerSpec":
        """The usual four slots: a norm before the mixer, the mixer, a norm before the feed-forward, the feed-forward."""
        return cls(block, {"mixer_norm": ("norm", mixer_norm), "mixer": ("mixer", mixer),
                           "feed_forward_norm": ("norm", feed_forward_norm), "feed_forward": ("feed_forward", feed_forward)})

    def part(self, slot: str) -> PartSpec:
        return self.parts[slot][1]


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    layer        index into ``ModelSpec.layers`` (a layer may be named more than once)
    cache        index of the cache/state entry this call uses; two calls that name the same
                 cache share it
    write_cache  False lets the call read a cache that another call filled in this step
    """
    layer: int
    cache: int
    write_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    """Everything the framework needs to know to build, load and run a model."""
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: Sequence[LayerSpec]
    schedule: Sequence[LayerCall]
    final_norm: PartSpec
    embedding: PartSpec              # family "embedding": token ids -> float32 rows of the residual stream
    head: PartSpec                   # family "head": normalised rows -> float32 logits; may be tied to the embedding
    eos_token_id: Optional[int] = None

    def part_specs(self) -> Iterator[Tuple[str, PartSpec]]:
        """Every (family, PartSpec) of the model: embedding, head, final norm, then the layers' parts in order."""
        yield "embedding", self.embedding
        yield "head", self.head
        yield "norm", self.final_norm
        for layer in self.layers:
            yield from layer.parts.values()

    def validate(self) -> None:
        if self.hidden_size <= 0 or self.vocab_size <= 0 or self.max_positions <= 0:
            raise ValueError("hidden_size, vocab_size and max_positions must be positive")
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        written = set()
        for i, call in enumerate(self.schedule):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"schedule[{i}] names layer {call.layer}, but there are {len(self.layers)}")
            if call.cache < 0:
                raise ValueError(f"schedule[{i}] has a negative cache index")
            if call.write_cache:
                if call.cache in written:
                    raise ValueError(f"schedule[{i}]: cache {call.cache} is written by two calls")
                written.add(call.cache)
            elif call.cache not in written:
                raise ValueError(f"schedule[{i}] reads cache {call.cache} before any call wrote it")

    @property
    def num_caches(self) -> int:
        return 1 + max(c.cache for c in self.schedule)
