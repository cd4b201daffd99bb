"""Hidden states per layer: collecting them from a step, writing and reading them, comparing two dumps.

The reference writes the embedding and the hidden state after every layer of its last token as
``GGUFLYR1`` + embd + n_layers + float32 data with a JSON file of root mean squares beside it
(pkg/debug/layers.go:12-163) and compares two such dumps layer by layer with the figures of
`DiffLogits` (pkg/debug/layers.go:165-181, pkg/debug/diff.go:17-48).  Here a dump holds one row per
wanted place of a step instead of one token, so its header carries the row count as well:

    "GGB2LYR1"  u32 hidden  u32 layers  u32 rows  float32[rows, hidden] (embedding)
                float32[layers, rows, hidden]                            (after each scheduled block)

all little-endian.  `LayerCollector` is the `LayerTaps` that fills one.
"""
from __future__ import annotations

import json
import math
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from .step import LayerTaps

MAGIC = b"GGB2LYR1"


@dataclass
class LayersDump:
    embed: np.ndarray                    # [rows, hidden] float32
    layers: np.ndarray                   # [n_layers, rows, hidden] float32

    @property
    def hidden(self) -> int:
        return int(self.embed.shape[1])

    @property
    def rows(self) -> int:
        return int(self.embed.shape[0])


class LayerCollector(LayerTaps):
    """Layer taps that keep what they are handed: the rows after the embedding and after every
    scheduled block, and (with `logits=True`) the head applied to each of them."""

    def __init__(self, logits: bool = False):
        self.embed: Optional[torch.Tensor] = None
        self.layers: List[torch.Tensor] = []
        self.layer_logits: List[torch.Tensor] = []
        self.final_logits: Optional[torch.Tensor] = None
        super().__init__(on_embed=self._embed, on_layer=self._layer,
                         on_layer_logits=self._layer_logits if logits else None, on_logits=self._logits)

    def _embed(self, rows: torch.Tensor) -> None:
        self.embed = rows

    def _layer(self, i: int, rows: torch.Tensor) -> None:
        self.layers.append(rows)

    def _layer_logits(self, i: int, logits: torch.Tensor) -> None:
        self.layer_logits.append(logits)

    def _logits(self, logits: torch.Tensor) -> None:
        self.final_logits = logits

    def dump(self) -> LayersDump:
        if self.embed is None:
            raise ValueError("nothing was tapped: the step wanted no rows")
        to_np = lambda t: t.detach().to("cpu", torch.float32).contiguous().numpy()    # noqa: E731
        return LayersDump(embed=to_np(self.embed), layers=np.stack([to_np(x) for x in self.layers]))


def write_layers(path: str, dump: LayersDump) -> None:
    n_layers, rows, hidden = dump.layers.shape
    if dump.embed.shape != (rows, hidden):
        raise ValueError(f"layers dump: embedding rows {dump.embed.shape} do not fit layers {dump.layers.shape}")
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<III", hidden, n_layers, rows))
        f.write(np.ascontiguousarray(dump.embed, dtype="<f4").tobytes())
        f.write(np.ascontiguousarray(dump.layers, dtype="<f4").tobytes())


def read_layers(path: str) -> LayersDump:
    with open(path, "rb") as f:
        magic = f.read(8)
        if magic != MAGIC:
            raise ValueError(f"{path}: not a layers dump (magic {magic!r}, expected {MAGIC!r})")
        hidden, n_layers, rows = struct.unpack("<III", f.read(12))
        data = np.frombuffer(f.read(), dtype="<f4").copy()
    want = (1 + n_layers) * rows * hidden
    if data.size != want:
        raise ValueError(f"{path}: holds {data.size} values, its header says {want}")
    data = data.reshape(1 + n_layers, rows, hidden)
    return LayersDump(embed=data[0], layers=data[1:])


def rms(x: np.ndarray) -> float:
    """Root mean square as the reference's dump metadata records it (pkg/debug/layers.go:183-194)."""
    x = np.asarray(x, dtype=np.float64)
    return float(math.sqrt(float((x * x).mean()))) if x.size else 0.0


def layers_meta(dump: LayersDump, **extra) -> Dict[str, object]:
    """The JSON that goes beside a dump (LayersMeta, pkg/debug/layers.go:14-27)."""
    meta: Dict[str, object] = dict(magic=MAGIC.decode(), embd=dump.hidden, num_layers=int(dump.layers.shape[0]),
                                   rows=dump.rows, embed_rms=rms(dump.embed),
                                   layer_rms=[rms(ly) for ly in dump.layers])
    meta.update(extra)
    return meta


def save_layers(prefix: str, dump: LayersDump, **extra) -> None:
    """`prefix`.bin and `prefix`.json (SaveLayersDump, pkg/debug/layers.go:116-146)."""
    write_layers(prefix + ".bin", dump)
    with open(prefix + ".json", "w", encoding="utf-8") as f:
        json.dump(layers_meta(dump, **extra), f, indent=2)
        f.write("\n")


@dataclass
class DiffStats:
    """DiffStats of pkg/debug/diff.go:6-14."""
    n: int = 0
    max_abs: float = 0.0
    mean_abs: float = 0.0
    rmse: float = 0.0
    max_abs_idx: int = -1
    over_tol: int = 0
    tol: float = 0.0


def diff_values(a: np.ndarray, b: np.ndarray, tol: float) -> DiffStats:
    """DiffLogits (pkg/debug/diff.go:17-48) over two arrays of equal size."""
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    n = min(a.size, b.size)
    st = DiffStats(n=n, tol=tol)
    if n == 0:
        return st
    d = np.abs(a[:n] - b[:n])
    st.max_abs_idx = int(d.argmax())
    st.max_abs = float(d[st.max_abs_idx])
    st.mean_abs = float(d.mean())
    st.rmse = float(math.sqrt(float((d * d).mean())))
    st.over_tol = int((d > tol).sum()) if tol > 0 else 0
    return st


@dataclass
class LayersDiff:
    embed: DiffStats
    layers: List[DiffStats] = field(default_factory=list)

    @property
    def worst_layer(self) -> int:
        return max(range(len(self.layers)), key=lambda i: self.layers[i].max_abs) if self.layers else -1

    @property
    def first_over(self) -> int:
        """The first layer with a value over the tolerance (-1: the embedding already, None: none)."""
        if self.embed.over_tol:
            return -1
        for i, st in enumerate(self.layers):
            if st.over_tol:
                return i
        return None


def diff_layers(a: LayersDump, b: LayersDump, tol: float) -> LayersDiff:
    """DiffLayers (pkg/debug/layers.go:165-181)."""
    if a.embed.shape != b.embed.shape:
        raise ValueError(f"layers dumps differ in shape: rows x hidden {a.embed.shape} and {b.embed.shape}")
    if a.layers.shape[0] != b.layers.shape[0]:
        raise ValueError(f"layers dumps differ in depth: {a.layers.shape[0]} and {b.layers.shape[0]} layers")
    return LayersDiff(embed=diff_values(a.embed, b.embed, tol),
                      layers=[diff_values(x, y, tol) for x, y in zip(a.layers, b.layers)])
