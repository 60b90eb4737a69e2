"""Which kernel variant serves which shape.

One table per kernel family. A row names a variant, a rank, a guard that
states every assumption the kernel makes, and the evidence for its rank; the
highest-ranked row whose guard holds is chosen, and every refusal keeps its
reason (`explain`). The scheme is the tactics table of MythEclipse/llm
(apps/engine/src/tactics.rs:99-109 rows, :353-396 selection with recorded
fallback reasons); the rows are this library's own kernels.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch


@dataclass(frozen=True)
class Tactic:
    name: str
    rank: int
    guard: Callable          # (**shape) -> None if it can run, else the reason it cannot
    evidence: str


def _always(**_):
    return None


LINEAR = [
    Tactic("gemm_simt", 0, _always,
           "CUDA-core product with a fixed summation order; any shape and stride; the only "
           "variant of the 32-bit path"),
]

ATTENTION = [
    Tactic("attention_generic", 0, _always,
           "one block per (token, head), 32-bit arithmetic, any head size up to 256, any group, "
           "window and ring; the only variant of the 32-bit path"),
]

_disabled: set = set()


def disable(name: str) -> None:
    """Take a variant out of the choice (tests use it to reach a fallback)."""
    _disabled.add(name)


def enable(name: str) -> None:
    _disabled.discard(name)


def _choose(table, **shape):
    best, reasons = None, []
    for row in sorted(table, key=lambda r: -r.rank):
        reason = "disabled" if row.name in _disabled else row.guard(**shape)
        if reason is None:
            best = row
            break
        reasons.append((row.name, reason))
    if best is None:
        raise RuntimeError(f"no kernel accepts {shape}: {reasons}")
    return best.name, reasons


def choose_linear(m, n, k, in_dtype, out_dtype, lda) -> str:
    return _choose(LINEAR, m=m, n=n, k=k, in_dtype=in_dtype, out_dtype=out_dtype, lda=lda)[0]


def choose_attention(decode, dtype, n_heads, n_kv_heads, head_dim, window) -> str:
    return _choose(ATTENTION, decode=decode, dtype=dtype, n_heads=n_heads, n_kv_heads=n_kv_heads,
                   head_dim=head_dim, window=window)[0]


def explain(family: str, **shape) -> str:
    """The chosen variant and why each higher-ranked one was refused."""
    table = {"linear": LINEAR, "attention": ATTENTION}[family]
    name, reasons = _choose(table, **shape)
    lines = [f"{family}: {name}"]
    lines += [f"  not {n}: {why}" for n, why in reasons]
    return "\n".join(lines)
