"""Reading and writing safetensors files without a third-party reader.

Layout: 8 bytes little-endian header length, a JSON header
{name: {dtype, shape, data_offsets: [begin, end]}}, then the raw tensor
bytes. Every tensor is checked to lie inside the file, as the GGUF reader of
MythEclipse/llm checks its tensors (apps/engine/src/gguf.rs:158-165).
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

from ..errors import FormatError

DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
NAMES = {v: k for k, v in DTYPES.items()}
_MAX_HEADER = 100 << 20


class SafetensorsFile:
    """A memory-mapped safetensors file; `tensor(name)` is a view of the map."""

    def __init__(self, path):
        self.path = Path(path)
        if not self.path.is_file():
            raise FormatError(f"{self.path}: no such file")
        size = self.path.stat().st_size
        if size < 8:
            raise FormatError(f"{self.path}: too short to be a safetensors file")
        self._handle = open(self.path, "rb")
        self._map = mmap.mmap(self._handle.fileno(), 0, access=mmap.ACCESS_READ)
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if header_len > min(size - 8, _MAX_HEADER):
            raise FormatError(f"{self.path}: header length {header_len} exceeds the file")
        try:
            header = json.loads(self._map[8:8 + header_len].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise FormatError(f"{self.path}: header is not JSON ({error})") from None
        if not isinstance(header, dict):
            raise FormatError(f"{self.path}: header is not an object")
        self.metadata = header.pop("__metadata__", None) or {}
        self._data_start = 8 + header_len
        self.entries = {}
        for name, entry in header.items():
            try:
                dtype = entry["dtype"]
                shape = tuple(int(d) for d in entry["shape"])
                begin, end = (int(v) for v in entry["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise FormatError(f"{self.path}: malformed entry for '{name}'") from None
            if dtype not in DTYPES:
                raise FormatError(f"{self.path}: '{name}' has unknown dtype {dtype}")
            count = 1
            for d in shape:
                count *= d
            width = torch.empty((), dtype=DTYPES[dtype]).element_size()
            if begin < 0 or end < begin or self._data_start + end > size:
                raise FormatError(f"{self.path}: '{name}' lies outside the file")
            if end - begin != count * width:
                raise FormatError(f"{self.path}: '{name}' holds {end - begin} bytes, "
                                  f"its shape {list(shape)} needs {count * width}")
            self.entries[name] = (dtype, shape, begin, end)

    def names(self):
        return list(self.entries)

    def shape(self, name):
        return self.entries[name][1]

    def dtype(self, name):
        return DTYPES[self.entries[name][0]]

    def tensor(self, name) -> torch.Tensor:
        dtype, shape, begin, end = self.entries[name]
        if end == begin:
            return torch.empty(shape, dtype=DTYPES[dtype])
        view = memoryview(self._map)[self._data_start + begin:self._data_start + end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")       # the map is read-only; tensors are only read
            flat = torch.frombuffer(view, dtype=DTYPES[dtype])
        return flat.reshape(shape)


def write_safetensors(path, tensors: dict, metadata: dict | None = None) -> None:
    """Write CPU tensors under their names, data 8-byte aligned."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in NAMES:
            raise FormatError(f"cannot store dtype {t.dtype} of '{name}'")
        size = t.numel() * t.element_size()
        header[name] = {"dtype": NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + size]}
        offset += size
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as out:
        out.write(struct.pack("<Q", len(blob)))
        out.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            out.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def open_checkpoint(folder) -> dict:
    """name -> (SafetensorsFile, name) for model.safetensors, or for the shards
    that model.safetensors.index.json lists."""
    folder = Path(folder)
    single = folder / "model.safetensors"
    index = folder / "model.safetensors.index.json"
    out = {}
    if single.is_file():
        f = SafetensorsFile(single)
        for name in f.names():
            out[name] = f
        return out
    if index.is_file():
        try:
            weight_map = json.loads(index.read_text())["weight_map"]
        except (json.JSONDecodeError, KeyError, TypeError):
            raise FormatError(f"{index}: no weight_map") from None
        files = {}
        for name, shard in weight_map.items():
            if shard not in files:
                files[shard] = SafetensorsFile(folder / shard)
            if name not in files[shard].entries:
                raise FormatError(f"{index}: '{name}' is not in {shard}")
            out[name] = files[shard]
        return out
    raise FormatError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")
