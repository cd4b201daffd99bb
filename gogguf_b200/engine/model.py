"""A model: parts built from a `ModelSpec` and a set of tensors, ready to be stepped.

The reference builds one hard-wired struct per architecture (pkg/model/qwen3/model.go:30-69: parse
the config, copy the norm weights, resolve the head's name, make cache and scratch).  Here the
architecture only supplies the spec; this module asks every part which tensors it expects, checks
them against what was found, and wires the blocks in schedule order.
"""
from __future__ import annotations

import os
from typing import Dict, List, Mapping, Optional, Tuple

import torch

from ..cache.sequence_cache import Request, SequenceCache
from ..config.registry import load_config
from ..config.spec import BlockSpec, ModelSpec, PartSpec
from ..parts import registry as R
from ..parts.base import Runtime
from ..weights.loader import TensorDecl, check_tensors, load_tensors, random_tensors

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {name}")
        return name
    try:
        return DTYPES[str(name)]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {name!r}") from None


def _part_class(table, spec: PartSpec, what: str):
    return R.lookup(table, spec.kind, what)


_FAMILIES = {"mixer": (R.MIXERS, "mixer"), "feed_forward": (R.FEED_FORWARDS, "feed-forward"),
             "norm": (R.NORMS, "norm")}


def _block_parts(b: BlockSpec) -> List[Tuple[str, PartSpec, type]]:
    """(role, spec, class) of every part of a block, in the order of the arrangement's `roles`.

    The arrangement class says which roles a block of its kind has and which family (registry) each
    role's part comes from; the block spec must name exactly those (roles listed in the arrangement's
    `optional_roles` may be left out)."""
    acls = R.lookup(R.ARRANGEMENTS, b.arrangement, "block arrangement")
    roles = getattr(acls, "roles", None)
    if roles is None:
        raise TypeError(f"block arrangement {b.arrangement!r} declares no `roles` (role -> family)")
    optional = set(getattr(acls, "optional_roles", ()))
    missing = [r for r in roles if r not in b.parts and r not in optional]
    extra = [r for r in b.parts if r not in roles]
    if missing or extra:
        raise ValueError(f"block arrangement {b.arrangement!r} has the roles {sorted(roles)}"
                         + (f"; missing: {sorted(missing)}" if missing else "")
                         + (f"; not known to it: {sorted(extra)}" if extra else ""))
    out = []
    for role, family in roles.items():
        if role not in b.parts:
            continue
        if family not in _FAMILIES:
            raise ValueError(f"block arrangement {b.arrangement!r}: role {role!r} names the unknown family "
                             f"{family!r} (known: {sorted(_FAMILIES)})")
        table, what = _FAMILIES[family]
        out.append((role, b.parts[role], _part_class(table, b.parts[role], what)))
    return out


def _cache_part(b: BlockSpec) -> Optional[Tuple[PartSpec, type]]:
    """The part of a block that may ask for cache or state: its mixer-family role (at most one)."""
    acls = R.lookup(R.ARRANGEMENTS, b.arrangement, "block arrangement")
    mixers = [(ps, cls) for role, ps, cls in _block_parts(b) if acls.roles[role] == "mixer"]
    if len(mixers) > 1:
        raise ValueError(f"block arrangement {b.arrangement!r}: a block may hold one mixer, not {len(mixers)} "
                         "(a schedule entry owns one cache)")
    return mixers[0] if mixers else None


def expected_tensors(spec: ModelSpec) -> Dict[str, TensorDecl]:
    """Every tensor the model expects, by full name."""
    out: Dict[str, TensorDecl] = {}

    def add(ps: PartSpec, cls) -> None:
        for local, decl in cls.tensors(ps).items():
            name = ps.prefix + local
            if name in out and out[name] != decl:
                raise ValueError(f"tensor {name!r} is declared twice with different shapes")
            out[name] = decl

    add(spec.embedding, _part_class(R.EMBEDDINGS, spec.embedding, "embedding"))
    for b in spec.blocks:
        for _, ps, cls in _block_parts(b):
            add(ps, cls)
    add(spec.final_norm, _part_class(R.NORMS, spec.final_norm, "norm"))
    add(spec.head, _part_class(R.HEADS, spec.head, "head"))
    return out


def _local(tensors: Mapping[str, torch.Tensor], ps: PartSpec, cls, consume: bool = False) -> Dict[str, torch.Tensor]:
    """A part's tensors under their local names.  consume: take them out of `tensors` (a dict the caller gave up),
    so that a part which builds its own fused copies leaves no second copy of its weights behind while the
    remaining layers are built."""
    names = [local for local in cls.tensors(ps) if ps.prefix + local in tensors]
    if consume:
        return {local: tensors.pop(ps.prefix + local) for local in names}
    return {local: tensors[ps.prefix + local] for local in names}


class Model:
    """Embedding, blocks in schedule order, final norm, head."""

    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor], dtype="bfloat16",
                 device="cuda:0", fast: bool = True, config=None, fold_norms: Optional[bool] = None,
                 consume: bool = False):
        spec.validate()
        self.spec = spec
        self.config = config
        if fold_norms is None:      # GOGGUF_B200_FOLD_NORMS=0 keeps every norm a kernel of its own
            fold_norms = os.environ.get("GOGGUF_B200_FOLD_NORMS", "1") != "0"
        self.rt = Runtime(dtype=parse_dtype(dtype), device=torch.device(device), fast=fast, fold_norms=fold_norms)
        found = {n: (t.dtype, tuple(t.shape)) for n, t in tensors.items()}
        check_tensors(expected_tensors(spec), found, where="model tensors")
        rt = self.rt

        ecls = _part_class(R.EMBEDDINGS, spec.embedding, "embedding")
        consume = consume and isinstance(tensors, dict)
        self.embedding = ecls(spec.embedding, _local(tensors, spec.embedding, ecls, consume), rt)
        self.blocks = []
        self._cache_parts = []
        for b in spec.blocks:
            built = {role: cls(ps, _local(tensors, ps, cls, consume), rt) for role, ps, cls in _block_parts(b)}
            acls = R.lookup(R.ARRANGEMENTS, b.arrangement, "block arrangement")
            self.blocks.append(acls(b, built, rt))
            self._cache_parts.append(_cache_part(b))
        ncls = _part_class(R.NORMS, spec.final_norm, "norm")
        self.final_norm = ncls(spec.final_norm, _local(tensors, spec.final_norm, ncls, consume), rt)
        hcls = _part_class(R.HEADS, spec.head, "head")
        tied = getattr(self.embedding, "weight", None) if spec.head.get("tied_to") is not None else None
        if tied is not None and spec.head.prefix + "weight" in found:
            import warnings
            warnings.warn(f"the configuration ties the head to the embedding; the stored {spec.head.prefix}weight "
                          "is not used", stacklevel=2)
        self.head = hcls(spec.head, _local(tensors, spec.head, hcls, consume), rt, tied)

    # ------------------------------------------------------------------ constructors
    @classmethod
    def load(cls, folder: str, dtype="bfloat16", device="cuda:0", fast: bool = True,
             fold_norms: Optional[bool] = None) -> "Model":
        """From a model folder: config.json picks the architecture, model.safetensors gives the tensors."""
        cfg = load_config(folder)
        spec = cfg.to_spec()
        aliases = cfg.tensor_aliases() if hasattr(cfg, "tensor_aliases") else None
        tensors = load_tensors(folder, expected_tensors(spec), device=device, aliases=aliases,
                               compute_dtype=parse_dtype(dtype))
        return cls(spec, tensors, dtype=dtype, device=device, fast=fast, config=cfg, fold_norms=fold_norms, consume=True)

    @classmethod
    def random(cls, config, seed: int, dtype="bfloat16", device="cuda:0", fast: bool = True,
               std: Optional[float] = None, norm_std: float = 0.0, store_dtype=None,
               fold_norms: Optional[bool] = None) -> "Model":
        """Random weights made on the device, without a folder (for measurement)."""
        spec = config.to_spec()
        sd = parse_dtype(store_dtype) if store_dtype is not None else parse_dtype(dtype)
        tensors = random_tensors(expected_tensors(spec), seed,
                                 std if std is not None else getattr(config, "initializer_range", 0.02),
                                 norm_std, dtype=sd, device=device)
        return cls(spec, tensors, dtype=dtype, device=device, fast=fast, config=config, fold_norms=fold_norms,
                   consume=True)

    # ------------------------------------------------------------------ cache
    def cache_requests(self) -> List[Request]:
        out: List[Request] = []
        for e in self.spec.schedule:
            cp = self._cache_parts[e.block]
            out.append(cp[1].cache_request(cp[0]) if cp is not None else None)
        return out

    def parts(self):
        """Every built part of the model: embedding, the parts of every block, final norm, head."""
        yield self.embedding
        for b in self.blocks:
            yield from getattr(b, "parts", {}).values()
        yield self.final_norm
        yield self.head

    def new_cache(self, max_tokens: int, max_slots: Optional[int] = None) -> SequenceCache:
        return SequenceCache(self.cache_requests(), [e.cache_of for e in self.spec.schedule], max_tokens,
                             dtype=self.rt.dtype, device=self.rt.device, max_slots=max_slots)

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size


def write_random_model(config, seed: int, folder: str, dtype="bfloat16", std: Optional[float] = None,
                       norm_std: float = 0.02) -> None:
    """Random-weights mode: write a model folder (config.json, model.safetensors) from a
    configuration and a seed.  Matrices and the embedding are N(0, std), norm weights
    1 + N(0, norm_std); values are drawn in float32 and rounded to `dtype`."""
    from ..weights.loader import write_model_folder
    spec = config.to_spec()
    tensors = random_tensors(expected_tensors(spec), seed,
                             std if std is not None else getattr(config, "initializer_range", 0.02),
                             norm_std, dtype=parse_dtype(dtype), device="cpu")
    write_model_folder(folder, config.to_dict(), tensors)
