"""Reading and writing the safetensors container, by tensor name.

File layout: 8 bytes little-endian header length N, N bytes of JSON mapping
each tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}``
(offsets relative to the end of the header), then the raw little-endian data.

This plays the part of the reference's weight store (pkg/weights/store.go:33-81
looks tensors up by name in the parsed file, pkg/format/reader.go:306-313); the
container differs (a model folder instead of one GGUF file), the role does not.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One ``.safetensors`` file, memory mapped; tensors are views until copied."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + n
        self._data_len = size - self._data_start
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            try:
                dt = _DTYPES[e["dtype"]]
            except KeyError:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {e.get('dtype')!r}") from None
            shape = tuple(int(s) for s in e["shape"])
            b, en = (int(x) for x in e["data_offsets"])
            numel = 1
            for s in shape:
                numel *= s
            if en - b != numel * torch.empty((), dtype=dt).element_size():
                raise SafetensorsError(f"{path}: tensor {name!r}: byte range {en - b} does not match "
                                       f"shape {list(shape)} of {e['dtype']}")
            if b < 0 or en > self._data_len:
                raise SafetensorsError(f"{path}: tensor {name!r} reaches beyond the end of the file (truncated?)")
            self.entries[name] = (dt, shape, b, en)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self.entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dt, shape, _, _ = self.entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (read-only memory: copy before writing)."""
        dt, shape, b, e = self.entries[name]
        if e == b:
            return torch.empty(shape, dtype=dt)
        mv = memoryview(self._mm)[self._data_start + b:self._data_start + e]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # "buffer is not writable": it is only read
            t = torch.frombuffer(mv, dtype=dt)
        return t.reshape(shape)

    def close(self) -> None:
        # tensors that still view the map keep it alive through their memoryview
        try:
            if self._mm is not None:
                self._mm.close()
        except BufferError:
            pass
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of tensor {name!r}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)


def open_model_files(folder: str) -> List[SafetensorsFile]:
    """The safetensors files of a model folder: ``model.safetensors`` or the shards its index names."""
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.isfile(single):
        return [SafetensorsFile(single)]
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            idx = json.load(f)
        shards = sorted(set(idx.get("weight_map", {}).values()))
        if not shards:
            raise SafetensorsError(f"{index}: empty weight_map")
        return [SafetensorsFile(os.path.join(folder, s)) for s in shards]
    raise SafetensorsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json found")
