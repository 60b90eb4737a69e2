"""Random weights from a configuration and a seed.

Follows the tiny-model writer of MythEclipse/llm (scripts/make_tiny_moe.py:
93-119: seeded normal matrices, norm gains 1 + N(0, 0.02)) for the model
folder layout this library reads: config.json and model.safetensors.
"""
from __future__ import annotations

import ctypes
import zlib
from pathlib import Path

import torch

from .safetensors_io import write_safetensors


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of one tensor: every element is a function of (key, index)."""
    return (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode("utf-8"))) & 0xFFFFFFFFFFFFFFFF


def normal_(out: torch.Tensor, key: int, mean: float, deviation: float) -> torch.Tensor:
    """Fill `out` (contiguous float32 or bfloat16, on the CPU or on a CUDA device) with
    mean + deviation * N(0, 1), element i drawn from (key, i) by the counter-based generator of
    csrc/random_normal.h. The host library and the device kernel give the same bits."""
    if out.dtype not in (torch.float32, torch.bfloat16) or not out.is_contiguous():
        raise ValueError("normal_: a contiguous float32 or bfloat16 tensor is needed")
    code = 0 if out.dtype == torch.float32 else 1
    if out.is_cuda:
        from .. import ops
        with torch.cuda.device(out.device):
            ops.random_normal_(out, key, mean, deviation)
    else:
        from .. import native
        native.check(native.lib().llmh_random_normal(
            ctypes.c_void_p(out.data_ptr()), code, ctypes.c_longlong(out.numel()),
            ctypes.c_ulonglong(key), ctypes.c_float(mean), ctypes.c_float(deviation)))
    return out


def random_tensors(expected: dict, seed: int, dtype=torch.bfloat16, std: float = 0.02,
                   gain_noise: float = 0.02, device="cpu") -> dict:
    """One tensor per declared parameter. Each value depends only on (seed, the tensor's
    name, its index in the tensor), not on the order, on the other tensors or on the
    device that makes it: a model made on the GPU and one written to a folder on the CPU
    from the same seed are the same model. Matrices and biases are N(0, std); gains are
    1 + N(0, gain_noise). Values are drawn in 32-bit and rounded once to `dtype`."""
    out = {}
    for name in sorted(expected):
        spec = expected[name]
        if spec.role == "table":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
            continue
        tensor = torch.empty(spec.shape, dtype=dtype, device=device)
        if spec.role == "gain":
            normal_(tensor, tensor_key(seed, name), 1.0, gain_noise)
        else:
            normal_(tensor, tensor_key(seed, name), 0.0, std)
        out[name] = tensor
    return out


def write_random_model(folder, config, seed: int, dtype=torch.bfloat16, std: float = 0.02,
                       gain_noise: float = 0.02) -> Path:
    """Write `folder`/config.json and `folder`/model.safetensors for `config`
    (any registered configuration object) with random weights."""
    from ..engine.model import declared_parameters
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    expected = declared_parameters(config.model_spec())
    tensors = random_tensors(expected, seed, dtype, std, gain_noise)
    raw = config.to_dict()
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}.get(dtype, str(dtype))
    import json
    (folder / "config.json").write_text(json.dumps(raw, indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", tensors,
                      {"format": "pt", "seed": seed, "std": std})
    return folder
