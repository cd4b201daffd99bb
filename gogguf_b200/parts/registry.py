"""Registries of part kinds: mixers, feed-forwards, norms, position encodings, block arrangements,
embeddings and heads.  A `PartSpec.kind` is looked up here; a new kind is added by decorating its
class, in this package or in user code, without touching the engine.

Interfaces (duck-typed; see `gogguf_b200.parts.base` for the step context they receive):

* every part:   ``tensors(spec) -> {local_name: TensorDecl}`` (classmethod) and
                ``__init__(spec, weights, runtime)`` with `weights` keyed by local names.
* mixer:        ``cache_request(spec) -> KVRequest | StateRequest | None`` (classmethod),
                ``prepare(ctx)`` once per step, and
                ``forward(h, residual, ctx, cache, writes_cache)``: reads the normed activations
                `h[T, hidden]` (compute dtype) and ADDS its output into `residual[T, hidden]` (float32).
* feed-forward: ``forward(h, residual, ctx)``, same contract.
* norm:         ``forward(x, out, rows=None)``: `x` float32 rows -> `out` in the compute dtype.
* position:     built by the mixer that uses it from ``spec["position"]``; ``tables(ctx)``.
* arrangement:  class attribute ``roles = {role: family}`` (family "mixer", "feed_forward" or "norm"; optional
                ``optional_roles``), ``__init__(block_spec, parts, runtime)`` with `parts` the built parts by role,
                an attribute ``parts`` holding them, and ``forward(x, ctx, cache, writes_cache)``.
* any part may set ``capturable = False`` if its `forward` reads back to the host or allocates; a model with
  such a part is stepped eagerly instead of through captured CUDA graphs.
"""
from __future__ import annotations

from typing import Callable, Dict, Type

MIXERS: Dict[str, Type] = {}
FEED_FORWARDS: Dict[str, Type] = {}
NORMS: Dict[str, Type] = {}
POSITIONS: Dict[str, Type] = {}
ARRANGEMENTS: Dict[str, Type] = {}
EMBEDDINGS: Dict[str, Type] = {}
HEADS: Dict[str, Type] = {}


def _register(table: Dict[str, Type], what: str) -> Callable[[str], Callable[[Type], Type]]:
    def by_kind(kind: str) -> Callable[[Type], Type]:
        def deco(cls: Type) -> Type:
            if kind in table and table[kind] is not cls:
                raise ValueError(f"{what} kind {kind!r} is already registered")
            table[kind] = cls
            return cls
        return deco
    return by_kind


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position = _register(POSITIONS, "position encoding")
register_arrangement = _register(ARRANGEMENTS, "block arrangement")
register_embedding = _register(EMBEDDINGS, "embedding")
register_head = _register(HEADS, "head")


def lookup(table: Dict[str, Type], kind: str, what: str) -> Type:
    try:
        return table[kind]
    except KeyError:
        raise KeyError(f"unknown {what} kind {kind!r}; registered: {sorted(table)}") from None
