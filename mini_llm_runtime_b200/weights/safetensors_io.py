"""Reading and writing the safetensors container.

File layout: 8 bytes little-endian header length n, n bytes of JSON
`{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}`,
then the tensor bytes; offsets are relative to the end of the header.  The
reference reads GGUF through a parser of the same shape: map the file, bounds-check
every tensor against the file size, look tensors up by name
(src/minillm/gguf_model.cpp:106-136, :182-208).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch


class WeightFileError(ValueError):
    """A weight file that is damaged or of a kind that cannot be read."""


# safetensors dtype tag -> (bytes per element, torch dtype)
_DTYPES = {
    "F32": (4, torch.float32),
    "BF16": (2, torch.bfloat16),
    "F16": (2, torch.float16),
    "I32": (4, torch.int32),
    "I64": (8, torch.int64),
}
_TAG_OF = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16",
           torch.int32: "I32", torch.int64: "I64"}


class SafetensorsFile:
    """One mapped .safetensors file; `tensor(name)` is a CPU view into the map."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._file = open(path, "rb")
        except OSError as e:
            raise WeightFileError(f"cannot open {path}: {e.strerror}") from None
        size = os.fstat(self._file.fileno()).st_size
        if size < 8:
            raise WeightFileError(f"{path}: shorter than a safetensors header")
        (n,) = struct.unpack("<Q", self._file.read(8))
        if n > size - 8 or n > (1 << 30):
            raise WeightFileError(f"{path}: header length {n} exceeds the file")
        try:
            header = json.loads(self._file.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightFileError(f"{path}: header is not JSON: {e}") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + n
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        data_bytes = size - self._base
        for name, entry in header.items():
            try:
                tag, shape = entry["dtype"], tuple(int(s) for s in entry["shape"])
                begin, end = (int(x) for x in entry["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise WeightFileError(f"{path}: malformed header entry for {name!r}") from None
            if tag not in _DTYPES:
                raise WeightFileError(f"{path}: tensor {name!r} has unsupported dtype {tag}; supported: {sorted(_DTYPES)}")
            count = 1
            for s in shape:
                count *= s
            if begin < 0 or end < begin or end > data_bytes or end - begin != count * _DTYPES[tag][0]:
                raise WeightFileError(f"{path}: tensor {name!r} has byte range [{begin}, {end}) that does not fit its shape {shape} or the file")
            self._entries[name] = (tag, shape, begin, end)
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_COPY)

    def names(self) -> List[str]:
        return list(self._entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self._entries[name][0]][1]

    def tensor(self, name: str) -> torch.Tensor:
        tag, shape, begin, end = self._entries[name]
        tdtype = _DTYPES[tag][1]
        count = (end - begin) // _DTYPES[tag][0]
        if count == 0:
            return torch.empty(shape, dtype=tdtype)
        return torch.frombuffer(self._map, dtype=tdtype, count=count, offset=self._base + begin).reshape(shape)

    def close(self) -> None:
        # Tensors handed out keep the map alive; only the file handle is dropped.
        self._file.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    """Write tensors (any device) as one safetensors file, names in sorted order."""
    header = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TAG_OF:
            raise WeightFileError(f"tensor {name!r} has dtype {t.dtype}, which safetensors output here does not cover")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TAG_OF[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".partial"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.dtype is torch.bfloat16:
                t = t.view(torch.int16)
            f.write(t.numpy().tobytes())
    os.replace(tmp, path)


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """The weight files of a model folder: `model.safetensors`, or the shards that
    `model.safetensors.index.json` names."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(single):
        return [SafetensorsFile(single)]
    if os.path.exists(index):
        with open(index, "r", encoding="utf-8") as f:
            shards = sorted(set(json.load(f).get("weight_map", {}).values()))
        if not shards:
            raise WeightFileError(f"{index} names no shard")
        return [SafetensorsFile(os.path.join(model_dir, s)) for s in shards]
    raise WeightFileError(f"{model_dir} holds neither model.safetensors nor model.safetensors.index.json")
