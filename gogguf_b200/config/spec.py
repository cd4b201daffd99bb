"""Model description as data.

A model is described by a `ModelSpec`: a list of `BlockSpec` (each names its
mixer, feed-forward, norms and their sizes), a *schedule* (the order in which
blocks run; an entry may name a block twice or let a block read the cache that
an earlier entry wrote), the embedding / final norm / head description, and the
tensor-name prefixes under which every part finds its weights.

Nothing in here knows about a particular architecture.  An architecture's
typed configuration (for instance `Qwen3Config`) turns its own `config.json`
keys into a `ModelSpec`; the parts are then built from the spec by kind name
through the registries in `gogguf_b200.parts.registry`.

The reference keeps the same facts in one struct per architecture
(pkg/model/qwen3/config.go:10-21) and hard-wires the block structure into its
forward function (pkg/model/qwen3/model.go:198-288); here the structure itself
is data so that another architecture only adds a config class.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a block: a kind name (registry key) and its parameters.

    `prefix` is prepended to the part's local tensor names (for instance
    ``model.layers.3.self_attn.`` + ``q_proj.weight``).
    """

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]


@dataclass(frozen=True)
class BlockSpec:
    """One layer: arrangement (how the parts are wired) plus its parts."""

    arrangement: str  # registry key of the block arrangement, e.g. "pre_norm"
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a block.

    `block` indexes `ModelSpec.blocks`.  `cache_of` is None when this execution
    owns a cache (or state) of its own; otherwise it is the index of an earlier
    schedule entry whose cache this execution reads instead of writing one.
    """

    block: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    blocks: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0:
            raise ValueError("model spec: vocab_size and hidden_size must be positive")
        if not self.blocks:
            raise ValueError("model spec: no blocks")
        if not self.schedule:
            raise ValueError("model spec: empty schedule")
        for i, e in enumerate(self.schedule):
            if not (0 <= e.block < len(self.blocks)):
                raise ValueError(f"model spec: schedule[{i}] names block {e.block}, "
                                 f"but there are {len(self.blocks)} blocks")
            if e.cache_of is not None:
                if not (0 <= e.cache_of < i):
                    raise ValueError(f"model spec: schedule[{i}].cache_of={e.cache_of} must name an earlier entry")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"model spec: schedule[{i}].cache_of={e.cache_of} must name an entry "
                                     "that owns its cache")


def default_schedule(n_blocks: int) -> Tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(block=i) for i in range(n_blocks))
