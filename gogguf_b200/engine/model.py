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


def _block_parts(b: BlockSpec) -> List[Tuple[PartSpec, type]]:
    return [
        (b.mixer, _part_class(R.MIXERS, b.mixer, "mixer")),
        (b.feed_forward, _part_class(R.FEED_FORWARDS, b.feed_forward, "feed-forward")),
        (b.mixer_norm, _part_class(R.NORMS, b.mixer_norm, "norm")),
        (b.feed_forward_norm, _part_class(R.NORMS, b.feed_forward_norm, "norm")),
    ]


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
        for ps, cls in _block_parts(b):
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
        self.mixer_classes = []
        for b in spec.blocks:
            built = [cls(ps, _local(tensors, ps, cls, consume), rt) for ps, cls in _block_parts(b)]
            acls = R.lookup(R.ARRANGEMENTS, b.arrangement, "block arrangement")
            self.blocks.append(acls(b, *built, rt))
            self.mixer_classes.append(_part_class(R.MIXERS, b.mixer, "mixer"))
        ncls = _part_class(R.NORMS, spec.final_norm, "norm")
        self.final_norm = ncls(spec.final_norm, _local(tensors, spec.final_norm, ncls, consume), rt)
        hcls = _part_class(R.HEADS, spec.head, "head")
        tied = getattr(self.embedding, "weight", None) if spec.head.get("tied_to") is not None else None
        self.head = hcls(spec.head, _local(tensors, spec.head, hcls, consume), rt, tied)

    # ------------------------------------------------------------------ constructors
    @classmethod
    def load(cls, folder: str, dtype="bfloat16", device="cuda:0", fast: bool = True,
             fold_norms: Optional[bool] = None) -> "Model":
        """From a model folder: config.json picks the architecture, model.safetensors gives the tensors."""
        cfg = load_config(folder)
        spec = cfg.to_spec()
        aliases = cfg.tensor_aliases() if hasattr(cfg, "tensor_aliases") else None
        tensors = load_tensors(folder, expected_tensors(spec), device=device, aliases=aliases)
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
            b = self.spec.blocks[e.block]
            out.append(self.mixer_classes[e.block].cache_request(b.mixer))
        return out

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
