"""Random weights from a configuration and a seed.

Follows the tiny-model writer of MythEclipse/llm (scripts/make_tiny_moe.py:
93-119: seeded normal matrices, norm gains 1 + N(0, 0.02)) for the model
folder layout this library reads: config.json and model.safetensors.
"""
from __future__ import annotations

import zlib
from pathlib import Path

import torch

from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode("utf-8"))) & 0x7FFFFFFFFFFFFFFF


def random_tensors(expected: dict, seed: int, dtype=torch.bfloat16, std: float = 0.02,
                   gain_noise: float = 0.02, device="cpu") -> dict:
    """One tensor per declared parameter. Each tensor's values depend only on
    (seed, its name, its shape), not on the order or on the other tensors.
    Matrices and biases are N(0, std); gains are 1 + N(0, gain_noise)."""
    out = {}
    for name in sorted(expected):
        spec = expected[name]
        gen = torch.Generator(device=device)
        gen.manual_seed(_tensor_seed(seed, name))
        if spec.role == "table":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
            continue
        noise = torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)
        if spec.role == "gain":
            value = 1.0 + gain_noise * noise
        else:
            value = std * noise
        out[name] = value.to(dtype)
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
