"""Reading and writing safetensors files without a third-party reader.

Layout: 8 bytes little-endian header length, a JSON header
{name: {dtype, shape, data_offsets: [begin, end]}}, then the raw tensor
bytes. The reader is the native host library's (`csrc/host/safetensors.cpp`):
it maps the file, reads the header with its own JSON reader and checks every
tensor to lie inside the file, as the GGUF reader of MythEclipse/llm checks its
tensors (apps/engine/src/gguf.rs:158-165). Tensors are views of that map.
"""
from __future__ import annotations

import ctypes
import json
import struct
import warnings
from ctypes import POINTER, byref, c_char_p, c_int, c_longlong, c_void_p
from pathlib import Path

import torch

from .. import native
from ..errors import FormatError

DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
NAMES = {v: k for k, v in DTYPES.items()}


class SafetensorsFile:
    """A memory-mapped safetensors file; `tensor(name)` is a view of the map
    (the map stays until the last such tensor is gone)."""

    def __init__(self, path):
        self.path = Path(path)
        lib = native.lib()
        handle = c_void_p()
        native.check(lib.llmh_safetensors_open(str(self.path).encode(), byref(handle)))
        self._handle = handle
        self.entries = {}                      # name -> (dtype name, shape, address, bytes)
        name, dtype, rank = c_char_p(), c_char_p(), c_int()
        shape, address, nbytes = POINTER(c_longlong)(), c_void_p(), c_longlong()
        for i in range(lib.llmh_safetensors_count(handle)):
            native.check(lib.llmh_safetensors_entry(handle, i, byref(name), byref(dtype), byref(rank),
                                                    byref(shape), byref(address), byref(nbytes)))
            self.entries[name.value.decode("utf-8")] = (
                dtype.value.decode(), tuple(shape[d] for d in range(rank.value)), address.value, nbytes.value)
        self.metadata = {}
        key, value = c_char_p(), c_char_p()
        for i in range(lib.llmh_safetensors_metadata_count(handle)):
            native.check(lib.llmh_safetensors_metadata_item(handle, i, byref(key), byref(value)))
            self.metadata[key.value.decode("utf-8")] = value.value.decode("utf-8")

    def __del__(self):
        handle = getattr(self, "_handle", None)
        if handle:
            native.lib().llmh_safetensors_close(handle)
            self._handle = None

    def names(self):
        return list(self.entries)

    def shape(self, name):
        return self.entries[name][1]

    def dtype(self, name):
        return DTYPES[self.entries[name][0]]

    def tensor(self, name) -> torch.Tensor:
        dtype, shape, address, nbytes = self.entries[name]
        if nbytes == 0:
            return torch.empty(shape, dtype=DTYPES[dtype])
        view = (ctypes.c_ubyte * nbytes).from_address(address)
        view._file = self                          # the tensor's storage keeps `view`, and so the map, alive
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
            weight_map = native.read_json(index.read_bytes(), str(index))["weight_map"]
            weight_map.items()
        except (KeyError, TypeError, AttributeError):
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
