"""Model description as data.

A model is described by a `ModelSpec`: a list of `BlockSpec` (each names its
arrangement and, by role, its parts - mixer, feed-forward, norms - with their sizes), a *schedule* (the order in which
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
from types import MappingProxyType
from typing import Any, Dict, List, Mapping, Optional, Tuple


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


@dataclass(frozen=True, init=False)
class BlockSpec:
    """One layer: an arrangement (how the parts are wired) and its parts by *role*.

    Which roles a block has is the arrangement's business: the arrangement class declares
    ``roles = {role: family}`` (family: "mixer", "feed_forward" or "norm", the registry the part's kind
    is looked up in), and the model builder builds exactly those.  The pre-norm arrangement of this
    library has the roles mixer, feed_forward, mixer_norm and feed_forward_norm; an arrangement with
    norms after its parts as well, with one norm shared by parallel parts, or without a feed-forward
    declares other roles and needs no change here or in the builder.

    ``BlockSpec("pre_norm", mixer=..., feed_forward=..., mixer_norm=..., feed_forward_norm=...)`` and
    ``BlockSpec("pre_norm", parts={...})`` are the same thing; ``block.mixer`` reads role "mixer".
    """

    arrangement: str  # registry key of the block arrangement, e.g. "pre_norm"
    parts: Mapping[str, PartSpec]

    def __init__(self, arrangement: str, parts: Optional[Mapping[str, PartSpec]] = None, **roles: PartSpec):
        merged = dict(parts or {})
        for role, ps in roles.items():
            if role in merged:
                raise ValueError(f"block spec: role {role!r} is given twice")
            merged[role] = ps
        for role, ps in merged.items():
            if not isinstance(ps, PartSpec):
                raise TypeError(f"block spec: role {role!r} must be a PartSpec, got {type(ps).__name__}")
        object.__setattr__(self, "arrangement", arrangement)
        object.__setattr__(self, "parts", MappingProxyType(merged))

    def __getattr__(self, role: str) -> PartSpec:
        # only reached when normal lookup fails: a role read as an attribute
        parts = object.__getattribute__(self, "__dict__").get("parts")
        if parts is not None and role in parts:
            return parts[role]
        raise AttributeError(f"block spec has no role {role!r}; its roles are {sorted(parts or ())}")

    def with_part(self, role: str, part: Optional[PartSpec]) -> "BlockSpec":
        """A copy with one role replaced, added, or (part None) taken out."""
        merged = dict(self.parts)
        if part is None:
            merged.pop(role, None)
        else:
            merged[role] = part
        return BlockSpec(self.arrangement, merged)

    def with_arrangement(self, arrangement: str) -> "BlockSpec":
        return BlockSpec(arrangement, dict(self.parts))


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
