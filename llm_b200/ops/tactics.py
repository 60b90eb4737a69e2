"""Which kernel variant serves which shape.

One table per kernel family. A row names a variant, a rank, a guard that
states every assumption the kernel makes, and the evidence for its rank; the
highest-ranked row whose guard holds is chosen, and every refusal keeps its
reason (`explain`). The scheme is the tactics table of MythEclipse/llm
(apps/engine/src/tactics.rs:99-109 rows, :353-396 selection with recorded
fallback reasons); the rows are this library's own kernels. The tables, the
guards and the selection live in the native host library
(`csrc/host/tactics.cpp`), next to the kernels they describe; this module is
their Python face.
"""
from __future__ import annotations

import ctypes
import hashlib
from ctypes import byref, c_char_p, c_int
from dataclasses import dataclass

import torch

from .. import native

_FAMILY = {"linear": 0, "attention": 1}


@dataclass(frozen=True)
class Tactic:
    name: str
    rank: int
    evidence: str


def rows(family: str) -> list:
    """The rows of a family's table as they stand in the native library."""
    lib, out = native.lib(), []
    name, rank, evidence = c_char_p(), c_int(), c_char_p()
    for i in range(lib.llmh_tactics_rows(_FAMILY[family])):
        native.check(lib.llmh_tactics_row(_FAMILY[family], i, byref(name), byref(rank), byref(evidence)))
        out.append(Tactic(name.value.decode(), rank.value, evidence.value.decode()))
    return out


_chosen: dict = {}       # arguments of a choice -> the variant's name, until a variant is switched
generation = 0           # grows whenever a variant is switched on or off (recorded passes are then stale)


def disable(name: str) -> None:
    """Take a variant out of the choice (tests use it to reach a fallback)."""
    global generation
    native.lib().llmh_tactics_set_disabled(name.encode(), 1)
    _chosen.clear()
    generation += 1


def enable(name: str) -> None:
    global generation
    native.lib().llmh_tactics_set_disabled(name.encode(), 0)
    _chosen.clear()
    generation += 1


def is_disabled(name: str) -> bool:
    key = ("disabled", name)
    answer = _chosen.get(key)
    if answer is None:
        answer = _chosen[key] = bool(native.lib().llmh_tactics_is_disabled(name.encode()))
    return answer


def _choose(family: str, m=0, n=0, k=0, lda=0, decode=False, n_heads=1, n_kv_heads=1, head_dim=0,
            window=0, packed=False, aligned=True, in_dtype=None, out_dtype=None, dtype=None):
    bf16 = (in_dtype if in_dtype is not None else dtype) == torch.bfloat16
    shape = (c_int * 12)(int(m), int(n), int(k), int(lda), int(bool(decode)), int(n_heads), int(n_kv_heads),
                         int(head_dim), int(window), int(bool(packed)), int(bf16), int(bool(aligned)))
    name, reasons = ctypes.create_string_buffer(64), ctypes.create_string_buffer(2048)
    native.check(native.lib().llmh_tactics_choose(_FAMILY[family], shape, name, 64, reasons, 2048))
    return name.value.decode(), reasons.value.decode()


def choose_linear(m, n, k, in_dtype, out_dtype, lda, aligned=True) -> str:
    key = ("linear", m, n, k, in_dtype, out_dtype, lda, aligned)
    name = _chosen.get(key)
    if name is None:
        if len(_chosen) > 8192:
            _chosen.clear()
        name = _chosen[key] = _choose("linear", m=m, n=n, k=k, in_dtype=in_dtype, out_dtype=out_dtype,
                                      lda=lda, aligned=aligned)[0]
    return name


def choose_attention(decode, dtype, n_heads, n_kv_heads, head_dim, window, packed=False,
                     aligned=True) -> str:
    key = ("attention", decode, dtype, n_heads, n_kv_heads, head_dim, window, packed, aligned)
    name = _chosen.get(key)
    if name is None:
        name = _chosen[key] = _choose("attention", decode=decode, dtype=dtype, n_heads=n_heads,
                                      n_kv_heads=n_kv_heads, head_dim=head_dim, window=window,
                                      packed=packed, aligned=aligned)[0]
    return name


def explain(family: str, **shape) -> str:
    """The chosen variant and why each higher-ranked one was refused."""
    name, reasons = _choose(family, **shape)
    return f"{family}: {name}" + ("\n" + reasons.rstrip("\n") if reasons else "")


def plan_identity(shapes) -> str:
    """A hash of which variant every (family, shape) of `shapes` gets, in the manner of the kernel
    plan's identity in MythEclipse/llm (apps/engine/src/tactics.rs:298-303): it changes exactly when
    a selection changes. `shapes`: iterable of (family, dict of the chooser's arguments)."""
    h = hashlib.sha256()
    for family, shape in shapes:
        name = _choose(family, **shape)[0]
        h.update(f"{family}:{sorted((k, str(v)) for k, v in shape.items())}->{name};".encode())
    return h.hexdigest()[:16]
