"""Weights by tensor name: declaration, checking, loading, random generation.

Every part of a model declares the tensors it expects (`TensorDecl`), the
model collects them under their full names, and `check_tensors` compares that
set with what a folder holds.  All disagreements are reported in ONE
`WeightsError` that lists missing tensors, unexpected tensors and wrong
shapes, instead of the reference's first-failure errors
(pkg/format/reader.go:306-313 "tensor not found"; pkg/model/qwen3/norms.go:16-45
wraps it with the layer; pkg/model/qwen3/model.go:664-666 checks q/k-norm length).

Storage policy: a tensor stored in bfloat16 stays bfloat16, a tensor stored in
32-bit floating point stays 32-bit, and integer tables become int32.  float16
has no kernel of its own: under the 32-bit compute path it is widened to
float32, which holds every float16 value exactly, and only under the bfloat16
path is it rounded to bfloat16.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Optional, Tuple

import torch

from .safetensors_io import SafetensorsError, open_model_files, write_safetensors


class WeightsError(ValueError):
    """The tensors of a model folder do not fit the configuration."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)


@dataclass(frozen=True)
class TensorDecl:
    """What a part expects of one tensor.

    init: "normal" (N(0, std)), "ones_normal" (1 + N(0, norm_std)) or "zeros";
    used only by the random-weights mode.  optional: may be absent (for
    instance a separate head matrix of a model with tied embeddings).
    """

    shape: Tuple[int, ...]
    init: str = "normal"
    optional: bool = False
    integer: bool = False


def check_tensors(expected: Mapping[str, TensorDecl],
                  found: Mapping[str, Tuple[torch.dtype, Tuple[int, ...]]],
                  where: str = "weights") -> None:
    missing = [n for n, d in expected.items() if n not in found and not d.optional]
    unexpected = [n for n in found if n not in expected]
    wrong = []
    for n, d in expected.items():
        if n in found:
            _, shape = found[n]
            if tuple(shape) != tuple(d.shape):
                wrong.append((n, tuple(shape), tuple(d.shape)))
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where}: tensors do not fit the configuration"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): " + ", ".join(
            f"{n} has {list(s)} but {list(e)} is expected" for n, s, e in sorted(wrong)))
    raise WeightsError("\n".join(lines), missing=sorted(missing), unexpected=sorted(unexpected),
                       wrong_shape=sorted(wrong))


def _stored_to_kept(t: torch.Tensor, compute_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Storage policy of the loader (see module docstring)."""
    if t.dtype in (torch.bfloat16, torch.float32):
        return t
    if t.dtype == torch.float16:
        return t.to(torch.float32 if compute_dtype == torch.float32 else torch.bfloat16)
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.bool, torch.int32):
        return t.to(torch.int32)
    raise WeightsError(f"unsupported tensor dtype {t.dtype}")


def load_tensors(folder: str, expected: Mapping[str, TensorDecl], device: str | torch.device = "cpu",
                 aliases: Optional[Mapping[str, str]] = None,
                 compute_dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Read the expected tensors of a model folder onto `device`.

    `compute_dtype` decides only what a float16 tensor becomes (float32 under the 32-bit path).

    `aliases` maps an alternative stored name to the expected name (for
    instance the GGUF-style names of pkg/model/qwen3/tensors.go:19-34).
    """
    try:
        files = open_model_files(folder)
    except SafetensorsError as e:
        raise WeightsError(str(e)) from None
    try:
        found: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]] = {}
        source: Dict[str, Tuple[object, str]] = {}
        for f in files:
            for stored in f.names():
                name = aliases.get(stored, stored) if aliases else stored
                if name in found:
                    raise WeightsError(f"{folder}: tensor {name!r} is stored twice")
                found[name] = f.info(stored)
                source[name] = (f, stored)
        check_tensors(expected, found, where=folder)
        out: Dict[str, torch.Tensor] = {}
        for name in expected:
            if name not in source:
                continue
            f, stored = source[name]
            t = _stored_to_kept(f.tensor(stored), compute_dtype)
            out[name] = t.to(device, copy=True) if torch.device(device).type != "cpu" else t.clone()
        return out
    finally:
        for f in files:
            f.close()


def random_tensors(expected: Mapping[str, TensorDecl], seed: int, std: float, norm_std: float,
                   dtype: torch.dtype = torch.bfloat16, device: str | torch.device = "cpu",
                   ) -> Dict[str, torch.Tensor]:
    """Seeded random weights: matrices and tables N(0, std), norm weights 1 + N(0, norm_std).

    Tensors are drawn in sorted name order from one generator in float32 and
    then rounded to `dtype`, so that a seed names one model whatever dtype it
    is stored in.  Optional tensors are not generated.
    """
    dev = torch.device(device)
    g = torch.Generator(device=dev)
    g.manual_seed(int(seed))
    out: Dict[str, torch.Tensor] = {}
    for name in sorted(expected):
        d = expected[name]
        if d.optional:
            continue
        if d.integer:
            out[name] = torch.zeros(d.shape, dtype=torch.int32, device=dev)
            continue
        if d.init == "zeros":
            t = torch.zeros(d.shape, dtype=torch.float32, device=dev)
        else:
            t = torch.empty(d.shape, dtype=torch.float32, device=dev)
            # large tensors are filled in slabs to bound the float32 staging memory
            t.normal_(0.0, 1.0, generator=g)
            if d.init == "normal":
                t.mul_(std)
            elif d.init == "ones_normal":
                t.mul_(norm_std).add_(1.0)
            else:
                raise ValueError(f"tensor {name!r}: unknown init {d.init!r}")
        out[name] = t.to(dtype)
    return out


def write_model_folder(folder: str, config_dict: Mapping[str, object], tensors: Mapping[str, torch.Tensor]) -> None:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(config_dict), f, indent=2)
        f.write("\n")
    write_safetensors(os.path.join(folder, "model.safetensors"), dict(tensors),
                      metadata={"format": "pt"})
