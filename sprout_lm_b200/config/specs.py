"""Architecture-neutral description of a model: which parts, with which constants, in which order.

An architecture's typed configuration (for instance ``Qwen2Config``) turns the
keys of its ``config.json`` into a ``ModelSpec``.  Everything below the
registry (parts, cache manager, step function, scheduler) reads only these
specs, never a ``config.json`` key and never a model's name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


class ConfigError(ValueError):
    """A config.json that this framework refuses, with the reason."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: ``kind`` names a registered part class, ``params`` are its constants."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def get(self, key: str, default=None):
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement (``block``) and the parts it arranges.

    ``prefix`` is the layer's prefix in checkpoint tensor names.
    """
    block: str
    prefix: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: tuple[PartSpec, ...]


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers``.  ``cache`` indexes the model's
    cache slots: the slot the layer's mixer reads, and writes when
    ``writes_cache``.  A layer may appear more than once in the order, and a
    call with ``writes_cache=False`` reads the cache that an earlier call
    filled (another layer's cache).
    """
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    order: tuple[LayerCall, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: tuple[int, ...]
    ignorable_tensors: tuple[str, ...] = ()

    def __post_init__(self):
        for call in self.order:
            if not 0 <= call.layer < len(self.layers):
                raise ConfigError(f"run order names layer {call.layer}, the model has {len(self.layers)}")
        slots = sorted({c.cache for c in self.order})
        if slots != list(range(len(slots))):
            raise ConfigError("cache slots of the run order must be 0..n-1 without gaps")
        written = set()
        for call in self.order:
            if call.writes_cache:
                written.add(call.cache)
            elif call.cache not in written:
                raise ConfigError(f"layer call reads cache slot {call.cache} before any call writes it")

    @property
    def cache_slots(self) -> int:
        return len({c.cache for c in self.order})
