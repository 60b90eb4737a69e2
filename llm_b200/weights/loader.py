"""Binding a checkpoint's tensors to a model's declared parameters by name."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..errors import WeightError
from .safetensors_io import open_checkpoint


@dataclass(frozen=True)
class ParamSpec:
    """What a part expects under one tensor name.

    role: 'matrix' (an operand of a matrix product, held in the run dtype),
    'gain' (a norm's weight), 'bias', 'table' (integers, held as int32).
    Gains and biases are held in 32-bit whatever the file stores.
    """
    shape: tuple
    role: str = "matrix"


def storage_dtype(file_dtype: torch.dtype) -> torch.dtype:
    """bfloat16 stays bfloat16, 32-bit stays 32-bit, float16 widens to 32-bit
    (exactly), float64 narrows to 32-bit, integers become int32."""
    if file_dtype == torch.bfloat16:
        return torch.bfloat16
    if file_dtype.is_floating_point:
        return torch.float32
    return torch.int32


def check_names(expected: dict, found: dict, where: str = "") -> None:
    """Raise one WeightError listing every missing and unexpected name and
    every wrong shape. `found` maps name -> shape (tuple)."""
    missing = [n for n in expected if n not in found]
    unexpected = [n for n in found if n not in expected]
    mismatched = [(n, list(found[n]), list(expected[n].shape))
                  for n in expected if n in found and tuple(found[n]) != tuple(expected[n].shape)]
    if missing or unexpected or mismatched:
        raise WeightError(missing, unexpected, mismatched, where)


def load_checkpoint(folder, expected: dict) -> dict:
    """Read every expected tensor of the checkpoint in `folder` (CPU, in its
    storage dtype). The names and shapes are checked first, all at once."""
    files = open_checkpoint(folder)
    check_names(expected, {name: f.shape(name) for name, f in files.items()}, str(folder))
    out = {}
    for name in expected:
        f = files[name]
        out[name] = f.tensor(name).to(storage_dtype(f.dtype(name)))
    return out
