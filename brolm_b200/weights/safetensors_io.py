"""Reader and writer of the safetensors container.

Layout: an unsigned 64-bit little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` with offsets
relative to the end of the header, then the payload
(the layout wlejon/brolm's test fixture writes, tests/test_gemma2.cpp:60-94).
Tensors are memory-mapped and handed out as torch tensors without a copy.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Iterable, Iterator

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One ``.safetensors`` file, mapped read-only."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"safetensors: cannot open '{path}'") from e
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"safetensors: '{path}' is shorter than its length field")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if 8 + hlen > size:
            raise SafetensorsError(f"safetensors: '{path}' header length {hlen} exceeds the file")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"safetensors: '{path}' has a malformed header: {e}") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"safetensors: '{path}' header is not an object")
        header.pop("__metadata__", None)
        self._base = 8 + hlen
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        self.entries: dict[str, tuple[torch.dtype, tuple[int, ...], int, int]] = {}
        payload = size - self._base
        for name, info in header.items():
            try:
                dtype = _DTYPES[info["dtype"]]
                shape = tuple(int(s) for s in info["shape"])
                begin, end = (int(x) for x in info["data_offsets"])
            except (KeyError, TypeError, ValueError) as e:
                raise SafetensorsError(
                    f"safetensors: '{path}' entry '{name}' is malformed or of an unsupported dtype") from e
            numel = 1
            for s in shape:
                numel *= s
            if begin < 0 or end < begin or end > payload:
                raise SafetensorsError(f"safetensors: '{path}' entry '{name}' lies outside the file (truncated?)")
            if end - begin != numel * dtype.itemsize:
                raise SafetensorsError(
                    f"safetensors: '{path}' entry '{name}' has {end - begin} bytes for shape {list(shape)}")
            self.entries[name] = (dtype, shape, begin, end)

    def names(self) -> list[str]:
        return list(self.entries)

    def __contains__(self, name: str) -> bool:
        return name in self.entries

    def shape(self, name: str) -> tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self.entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, begin, end = self.entries[name]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)      # the map is read-only; nothing here writes to it
            flat = torch.frombuffer(self._map, dtype=dtype, count=(end - begin) // dtype.itemsize,
                                    offset=self._base + begin)
        return flat.reshape(shape)


def write_safetensors(path: str, tensors: Iterable[tuple[str, torch.Tensor]] | dict) -> None:
    """Write tensors in the order given.  Tensors are taken one at a time, so
    a generator keeps only one of them in memory."""
    if isinstance(tensors, dict):
        tensors = tensors.items()
    tmp = path + ".payload.tmp"
    header: dict[str, dict] = {}
    offset = 0
    with open(tmp, "wb") as out:
        for name, t in tensors:
            if name in header:
                raise SafetensorsError(f"safetensors: duplicate tensor name '{name}'")
            if t.dtype not in _NAMES:
                raise SafetensorsError(f"safetensors: dtype {t.dtype} of '{name}' cannot be stored")
            t = t.detach().to("cpu").contiguous()
            raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
            header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                            "data_offsets": [offset, offset + len(raw)]}
            out.write(raw)
            offset += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as out, open(tmp, "rb") as payload:
        out.write(struct.pack("<Q", len(text)))
        out.write(text)
        while True:
            chunk = payload.read(1 << 24)
            if not chunk:
                break
            out.write(chunk)
    os.remove(tmp)


def open_model_shards(folder: str) -> list[SafetensorsFile]:
    """The shards of a model folder: those ``model.safetensors.index.json``
    lists, else every ``*.safetensors`` in name order."""
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index, "r", encoding="utf-8") as fh:
            files = sorted(set(json.load(fh).get("weight_map", {}).values()))
    else:
        try:
            files = sorted(f for f in os.listdir(folder) if f.endswith(".safetensors"))
        except OSError as e:
            raise SafetensorsError(f"weights: cannot list '{folder}'") from e
    if not files:
        raise SafetensorsError(f"weights: no safetensors shards in '{folder}'")
    return [SafetensorsFile(os.path.join(folder, f)) for f in files]


def iter_tensors(shards: list[SafetensorsFile]) -> Iterator[tuple[str, SafetensorsFile]]:
    """Every (name, shard); the first shard that holds a name wins
    (include/brolm/detail/weights.h:259-264)."""
    seen: set[str] = set()
    for shard in shards:
        for name in shard.names():
            if name not in seen:
                seen.add(name)
                yield name, shard
