"""Planning the scratch buffers of a step into one arena.

The planner follows MythEclipse/llm's workspace (apps/engine/src/workspace.rs):
every activation of a pass is a request {name, size, first_use, last_use} over
numbered phases (workspace.rs:24-43), requests are placed in order of first use
at the lowest aligned offset that overlaps no buffer that is live at the same
time, where writing in the phase another buffer is last read counts as overlap
(workspace.rs:63-106), and the layout has an identity hash (workspace.rs:135-146).
Its value is less the memory saved than fixed addresses: a captured decode step
points into the arena, and no allocation happens inside a step.

Here the requests are not one fixed list: every part declares the buffers of
its own forward pass with phases of its own, and the block lines them up. All
layers share one plan, so the arena is as large as one layer needs.
"""
from __future__ import annotations

import hashlib
from ctypes import byref, c_char_p, c_longlong
from dataclasses import dataclass

import torch

from .. import native

ALIGNMENT = 256          # bytes; TMA wants 16, 256 keeps every buffer on its own cache lines


@dataclass(frozen=True)
class BufferRequest:
    name: str
    shape: tuple
    dtype: torch.dtype
    first_use: int          # phase in which the buffer is first written
    last_use: int           # last phase in which it is read

    @property
    def nbytes(self) -> int:
        n = torch.empty((), dtype=self.dtype).element_size()
        for d in self.shape:
            n *= d
        return n

    def shifted(self, by: int, prefix: str = "") -> "BufferRequest":
        return BufferRequest(prefix + self.name, self.shape, self.dtype, self.first_use + by,
                             self.last_use + by)


@dataclass(frozen=True)
class Placement:
    request: BufferRequest
    offset: int


class Plan:
    def __init__(self, placements: list, total: int):
        self.placements = {p.request.name: p for p in placements}
        self.total = total

    def identity(self) -> str:
        h = hashlib.sha256()
        for name in sorted(self.placements):
            p = self.placements[name]
            h.update(f"{name}:{p.offset}:{p.request.nbytes}:{p.request.first_use}:{p.request.last_use};".encode())
        return h.hexdigest()[:16]

    def check(self) -> None:
        """No two buffers that are live in a common phase share a byte; all are aligned."""
        items = list(self.placements.values())
        for p in items:
            if p.offset % ALIGNMENT:
                raise AssertionError(f"{p.request.name} is not aligned")
            if p.offset + p.request.nbytes > self.total:
                raise AssertionError(f"{p.request.name} leaves the arena")
        for i, a in enumerate(items):
            for b in items[i + 1:]:
                if _live_together(a.request, b.request) and _bytes_overlap(a, b):
                    raise AssertionError(f"{a.request.name} and {b.request.name} overlap while both live")


def _live_together(a: BufferRequest, b: BufferRequest) -> bool:
    return a.first_use <= b.last_use and b.first_use <= a.last_use


def _bytes_overlap(a: Placement, b: Placement) -> bool:
    return a.offset < b.offset + b.request.nbytes and b.offset < a.offset + a.request.nbytes


def plan(requests) -> Plan:
    """Greedy first fit in order of (first use, name), done by the native host library
    (`csrc/host/planner.cpp`); `Plan.check` verifies a layout independently."""
    requests = list(requests)
    n = len(requests)
    offsets, total = (c_longlong * n)(), c_longlong()
    code = native.lib().llmh_plan_place(
        n, (c_char_p * n)(*[r.name.encode() for r in requests]),
        native.ints((r.nbytes for r in requests), c_longlong), native.ints(r.first_use for r in requests),
        native.ints(r.last_use for r in requests), ALIGNMENT, offsets, byref(total))
    if code != native.OK:
        raise ValueError(native.lib().llmh_last_error().decode("utf-8", "replace"))
    return Plan([Placement(r, offsets[i]) for i, r in enumerate(requests)], total.value)


class Workspace:
    """The arena of an engine. `for_tokens(n)` plans (once per token count) and
    returns named views; an arena that was outgrown stays alive, because a
    captured step may still point into it."""

    def __init__(self, device, requests_for_tokens):
        self.device = torch.device(device)
        self.requests_for_tokens = requests_for_tokens      # n_tokens -> list of BufferRequest
        self.plans: dict = {}
        self.arena = None
        self._retired: list = []
        self._views: dict = {}                              # n_tokens -> Views of the current arena

    def plan_for(self, n_tokens: int) -> Plan:
        if n_tokens not in self.plans:
            if len(self.plans) > 64:
                self.plans.clear()
                self._views.clear()
            self.plans[n_tokens] = plan(self.requests_for_tokens(n_tokens))
        return self.plans[n_tokens]

    def for_tokens(self, n_tokens: int) -> "Views":
        p = self.plan_for(n_tokens)
        if self.arena is None or self.arena.numel() < p.total:
            if self.arena is not None:
                self._retired.append(self.arena)
            self.arena = torch.empty(max(p.total, 1), dtype=torch.uint8, device=self.device)
            self._views.clear()
        views = self._views.get(n_tokens)
        if views is None:
            views = self._views[n_tokens] = Views(p, self.arena)
        views.prefix = ""
        return views

    def bytes(self) -> int:
        return 0 if self.arena is None else self.arena.numel()


class Views:
    """Named tensors inside the arena for the steps of one token count (made once, then reused:
    every step of that size gets the same addresses)."""

    def __init__(self, plan_: Plan, arena: torch.Tensor):
        self.plan = plan_
        self.arena = arena
        self.prefix = ""
        self._tensors: dict = {}

    def get(self, name: str, shape=None, dtype=None):
        """The planned buffer `name` (of the current layer prefix), or None if no part declared
        it. With `shape` (and `dtype`) the front of the buffer is returned in that form: blocks
        of one model may ask for different sizes under one name; the plan holds the largest.
        A shape that does not fit into the planned buffer is refused."""
        full = self.prefix + name
        key = full if shape is None else (full, tuple(shape), dtype)
        try:
            return self._tensors[key]
        except KeyError:
            pass
        placement = self.plan.placements.get(full)
        if placement is None:
            tensor = None
        else:
            r = placement.request
            flat = self.arena[placement.offset:placement.offset + r.nbytes]
            if shape is None:
                tensor = flat.view(r.dtype).view(r.shape)
            else:
                want = BufferRequest(full, tuple(shape), dtype or r.dtype, r.first_use, r.last_use)
                if want.nbytes > r.nbytes:
                    raise ValueError(f"scratch buffer '{full}' was planned with {r.nbytes} bytes "
                                     f"({r.shape}, {r.dtype}); {tuple(shape)} {want.dtype} needs "
                                     f"{want.nbytes}")
                tensor = flat[:want.nbytes].view(want.dtype).view(want.shape)
        self._tensors[key] = tensor
        return tensor
