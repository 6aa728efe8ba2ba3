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

    ``prefix`` is the layer's prefix in checkpoint tensor names; ``options`` are constants of the
    arrangement itself (a post_norm block's ``alpha``).
    """
    block: str
    prefix: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: tuple[PartSpec, ...]
    options: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers``.  ``cache`` indexes the model's
    cache slots: the slot the layer's mixer reads, and writes when
    ``writes_cache``.  A layer may appear more than once in the order, and a
    call with ``writes_cache=False`` reads the cache that an earlier call
    filled (another layer's cache).  ``state`` names the per-request state
    that the call's mixer carries: None is the layer's own (entry ``layer``);
    a layer that runs several times with a state per run gives its further
    calls entries from ``len(layers)`` on.
    """
    layer: int
    cache: int
    writes_cache: bool = True
    state: int | None = None


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
    stream: PartSpec | None = None       # what goes from one layer call to the next (None: the call's result)

    def __post_init__(self):
        for call in self.order:
            if not 0 <= call.layer < len(self.layers):
                raise ConfigError(f"run order names layer {call.layer}, the model has {len(self.layers)}")
        slots = sorted({c.cache for c in self.order})
        if slots != list(range(len(slots))):
            raise ConfigError("cache slots of the run order must be 0..n-1 without gaps")
        entries = sorted({c.layer if c.state is None else c.state for c in self.order})
        if entries and (entries[0] < 0 or entries[-1] >= len(self.layers) + len(self.order)):
            raise ConfigError("a layer call names a state entry out of range")
        written = set()
        for call in self.order:
            if call.writes_cache:
                written.add(call.cache)
            elif call.cache not in written:
                raise ConfigError(f"layer call reads cache slot {call.cache} before any call writes it")

    @property
    def cache_slots(self) -> int:
        return len({c.cache for c in self.order})
