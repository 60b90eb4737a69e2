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


def _skinny_guard(m, n, k, in_dtype, out_dtype, lda, aligned=True, **_):
    if in_dtype != torch.bfloat16:
        return "bfloat16 operands only"
    if m > 64:
        return f"{m} rows exceed 64"
    if k % 8 or lda % 8:
        return f"K {k} or the row stride {lda} is no multiple of 8 elements (16-byte loads)"
    if not aligned:
        return "an operand does not start on a 16-byte boundary"
    return None


def _tc_guard(m, n, k, in_dtype, out_dtype, lda, aligned=True, **_):
    if in_dtype != torch.bfloat16:
        return "bfloat16 operands only"
    if k % 8 or lda % 8:
        return (f"K {k} or the row stride {lda} is no multiple of 8 elements: a TMA row stride "
                "must be a multiple of 16 bytes")
    if not aligned:
        return "an operand does not start on a 16-byte boundary (TMA base address)"
    return None


LINEAR = [
    Tactic("gemm_tc", 30, _tc_guard,
           "tcgen05.mma with the accumulator in tensor memory, operands by TMA; weights on the "
           "128-row side and split K for up to 64 tokens, tokens on it above (pairs of SMs on "
           "256 x 256 tiles from 512 tokens). Measured on a B200 at 4096 x 14336 layer sizes: "
           "about 1,200 TFLOP/s at 2,048 tokens, 5.4 to 6.0 TB/s of weights at 8 tokens"),
    Tactic("gemm_skinny", 20, _skinny_guard,
           "decode product for up to 64 rows: W streamed once with 128-bit loads into "
           "mma.sync fragments, K split over warps with an ordered last-arriver sum; within "
           "a few percent of gemm_tc at 8 rows, behind it from 16"),
    Tactic("gemm_simt", 0, _always,
           "CUDA-core product with a fixed summation order; any shape and stride; the only "
           "variant of the 32-bit path"),
]

def _decode_guard(decode, dtype, n_heads, n_kv_heads, head_dim, window, **_):
    if not decode:
        return "serves steps in which every sequence brings one token"
    if dtype != torch.bfloat16:
        return "bfloat16 caches only"
    if window:
        return "no window"
    if n_heads // n_kv_heads > 8:
        return f"group of {n_heads // n_kv_heads} query heads exceeds 8"
    if head_dim not in (32, 64, 96, 128):
        return f"head_dim {head_dim} (served: 32, 64, 96, 128)"
    return None


def _prefill_guard(decode, dtype, n_heads, n_kv_heads, head_dim, window, packed=False, **_):
    if not packed:
        return "needs the packed batch description (cu_seqlens and seq_lens)"
    if dtype != torch.bfloat16:
        return "bfloat16 caches only"
    if window:
        return "no window"
    if head_dim not in (32, 64, 96, 128):
        return f"head_dim {head_dim} (served: 32, 64, 96, 128)"
    return None


def _prefill_tc_guard(decode, dtype, n_heads, n_kv_heads, head_dim, window, packed=False,
                      aligned=True, **_):
    reason = _prefill_guard(decode, dtype, n_heads, n_kv_heads, head_dim, window, packed)
    if reason:
        return reason
    if head_dim not in (64, 128):
        return f"head_dim {head_dim} (served: 64, 128)"
    if not aligned:
        return "the projection's rows are not 16-byte aligned (TMA)"
    return None


ATTENTION = [
    Tactic("attention_prefill_tc", 15, _prefill_tc_guard,
           "flash attention with both products on tcgen05 (accumulators in tensor memory, K and V "
           "pages by TMA), one thread per query row for the softmax, two blocks an SM; head sizes "
           "64 and 128. Measured with 32/8 heads of 128: 79 us at 2,048 tokens, 730 us at 8,192 "
           "(436 and 753 TFLOP/s of causal work); with heads of 64: 71 and 668 us"),
    Tactic("attention_prefill", 10, _prefill_guard,
           "flash attention over the paged cache for steps with several new tokens a sequence: "
           "64-query tiles, mma.sync, online softmax, heaviest tile first; head sizes in steps of "
           "16 up to 256. Measured: 170 us at 2,048 tokens with 32/8 heads of 128, 90 us with "
           "heads of 64"),
    Tactic("attention_decode", 20, _decode_guard,
           "split-KV decode attention: pages through shared memory with cp.async, the query "
           "heads of a group as rows of mma.sync tiles, partials merged by a second kernel. "
           "Measured: 46 us for 8 sequences of 8,192 keys with 8 kv heads of 128 (5.8 TB/s)"),
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


def choose_linear(m, n, k, in_dtype, out_dtype, lda, aligned=True) -> str:
    return _choose(LINEAR, m=m, n=n, k=k, in_dtype=in_dtype, out_dtype=out_dtype, lda=lda,
                   aligned=aligned)[0]


def choose_attention(decode, dtype, n_heads, n_kv_heads, head_dim, window, packed=False,
                     aligned=True) -> str:
    return _choose(ATTENTION, decode=decode, dtype=dtype, n_heads=n_heads, n_kv_heads=n_kv_heads,
                   head_dim=head_dim, window=window, packed=packed, aligned=aligned)[0]


def explain(family: str, **shape) -> str:
    """The chosen variant and why each higher-ranked one was refused."""
    table = {"linear": LINEAR, "attention": ATTENTION}[family]
    name, reasons = _choose(table, **shape)
    lines = [f"{family}: {name}"]
    lines += [f"  not {n}: {why}" for n, why in reasons]
    return "\n".join(lines)


def plan_identity(shapes) -> str:
    """A hash of which variant every (family, shape) of `shapes` gets, in the manner of the kernel
    plan's identity in MythEclipse/llm (apps/engine/src/tactics.rs:298-303): it changes exactly when
    a selection changes. `shapes`: iterable of (family, dict of the chooser's arguments)."""
    import hashlib
    h = hashlib.sha256()
    for family, shape in shapes:
        table = LINEAR if family == "linear" else ATTENTION
        name = _choose(table, **shape)[0]
        h.update(f"{family}:{sorted((k, str(v)) for k, v in shape.items())}->{name};".encode())
    return h.hexdigest()[:16]
