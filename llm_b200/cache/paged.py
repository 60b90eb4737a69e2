"""The cache: a slot per sequence, pages of keys and values per group of
layers, and fixed-size per-sequence state.

MythEclipse/llm keeps one cache per session (apps/engine/src/model.rs:351-436:
a key and a value buffer per attention layer, a layer -> cache index table with
None for layers that keep no keys, one length) and a separate fixed-size state
per recurrent layer that is zeroed on reset (model.rs:443-483). Here one cache
serves a batch:

* a *slot* is one live sequence with its own length;
* layers are put in *groups* by what they need: `full` (every earlier key) or
  `window` (the last w keys, kept in a ring of pages). Each group has its own
  page pool [layers, 2, pages, kv heads, 64, head_dim] and, per slot, its own
  list of pages: logical page i of a sequence is `pages[i % ring]`;
* `state` tensors [slots, ...] hold what a mixer keeps per sequence at a fixed
  size; a slot's rows are zeroed when the slot is taken.

Slots and pages are given back by `release` and reused.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..errors import CacheFull, ContextFull, LlmError
from .allocator import FreeList

PAGE = 64


def round_up(n: int, unit: int = PAGE) -> int:
    return (n + unit - 1) // unit * unit


@dataclass(frozen=True)
class KvRequest:
    """What one cache-owning run of a layer asks of the cache."""
    n_kv_heads: int
    head_dim: int
    window: int = 0            # 0: keep every position

    @property
    def group_key(self):
        return ("window" if self.window else "full", self.n_kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class StateRequest:
    """Fixed-size per-sequence state: one tensor [slots, *shape] of `dtype`."""
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class Group:
    kind: str
    n_kv_heads: int
    head_dim: int
    window: int
    entries: list = field(default_factory=list)     # schedule positions that own storage here
    ring_pages: int = 0                               # logical pages per sequence
    pool: FreeList | None = None
    storage: torch.Tensor | None = None               # [entries, 2, pages, Hkv, PAGE, D]
    slot_pages: dict = field(default_factory=dict)    # slot -> list of physical pages
    host_table: torch.Tensor | None = None            # int32 [slots, ring_pages], mirrors slot_pages


class PagedCache:
    """See the module text. `requests[i]` is the KvRequest of schedule entry i
    (None if that run keeps no keys of its own); `states[i]` its StateRequest or
    None. `max_tokens` bounds the tokens held by all live sequences together,
    each rounded up to a multiple of 64; `max_seq_len` bounds one sequence;
    `step_tokens` bounds the new tokens of one sequence in one step (it sizes
    the ring of window groups)."""

    def __init__(self, requests, states, max_tokens: int, max_seq_len: int, max_slots: int,
                 dtype, device, step_tokens: int | None = None):
        self.max_tokens = round_up(max(max_tokens, PAGE))
        self.max_seq_len = max_seq_len
        self.max_slots = max_slots
        self.dtype = dtype
        self.device = torch.device(device)
        self.step_tokens = step_tokens or max_seq_len
        self.slots = FreeList(max_slots, "slot")
        self.lengths = [0] * max_slots
        self.groups: list[Group] = []
        self.entry_group: list = []          # schedule entry -> (group index, index in group) or None
        by_key = {}
        for entry, request in enumerate(requests):
            if request is None:
                self.entry_group.append(None)
                continue
            key = request.group_key
            if key not in by_key:
                by_key[key] = len(self.groups)
                self.groups.append(Group(key[0], request.n_kv_heads, request.head_dim, request.window))
            g = by_key[key]
            self.entry_group.append((g, len(self.groups[g].entries)))
            self.groups[g].entries.append(entry)
        total_pages = self.max_tokens // PAGE
        seq_pages = round_up(max_seq_len) // PAGE
        for group in self.groups:
            if group.kind == "window":
                # a step writes up to step_tokens new positions before attention runs, and
                # the oldest query of the step still needs the window before it
                group.ring_pages = min(seq_pages, (group.window + self.step_tokens - 2) // PAGE + 2)
                n_pages = min(total_pages, max_slots * group.ring_pages)
            else:
                group.ring_pages = seq_pages
                n_pages = total_pages
            group.pool = FreeList(n_pages, f"page of the {group.kind} group")
            group.host_table = torch.zeros((max_slots, group.ring_pages), dtype=torch.int32)
            group.storage = torch.zeros(
                (len(group.entries), 2, n_pages, group.n_kv_heads, PAGE, group.head_dim),
                dtype=dtype, device=self.device)
        self.states = []
        for request in states:
            if request is None:
                self.states.append(None)
            else:
                self.states.append(torch.zeros((max_slots, *request.shape), dtype=request.dtype,
                                               device=self.device))

    # ------------------------------------------------------------------ slots

    def acquire(self) -> int:
        """Take a free slot: length 0, no pages, state zeroed."""
        slot = self.slots.take()
        self.lengths[slot] = 0
        for group in self.groups:
            group.slot_pages[slot] = []
            group.host_table[slot].zero_()
        for state in self.states:
            if state is not None:
                state[slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        """Give the slot and all of its pages back."""
        if not (0 <= slot < self.max_slots) or not self.slots.is_held(slot):
            raise LlmError(f"slot {slot} is not held")
        for group in self.groups:
            for page in group.slot_pages.pop(slot):
                group.pool.give_back(page)
        self.lengths[slot] = 0
        self.slots.give_back(slot)

    def reserve(self, slot: int, new_length: int) -> None:
        """Make sure the slot has pages for positions < new_length. Raises
        ContextFull or CacheFull before anything is changed."""
        if not self.slots.is_held(slot):
            raise LlmError(f"slot {slot} is not held")
        if new_length > self.max_seq_len:
            raise ContextFull(new_length, self.max_seq_len)
        needs = []
        for group in self.groups:
            want = min(round_up(new_length) // PAGE, group.ring_pages)
            extra = want - len(group.slot_pages[slot])
            if extra > group.pool.n_free:
                raise CacheFull(f"the {group.kind} group has {group.pool.n_free} free pages, "
                                f"slot {slot} needs {extra} more for {new_length} positions")
            needs.append(extra)
        for group, extra in zip(self.groups, needs):
            for _ in range(max(extra, 0)):
                page = group.pool.take()
                group.host_table[slot, len(group.slot_pages[slot])] = page
                group.slot_pages[slot].append(page)

    def reserve_many(self, wanted) -> None:
        """`reserve` for several (slot, new_length) pairs: all of them or none."""
        needs = [0] * len(self.groups)
        for slot, new_length in wanted:
            if not self.slots.is_held(slot):
                raise LlmError(f"slot {slot} is not held")
            if new_length > self.max_seq_len:
                raise ContextFull(new_length, self.max_seq_len)
            for g, group in enumerate(self.groups):
                want = min(round_up(new_length) // PAGE, group.ring_pages)
                needs[g] += max(want - len(group.slot_pages[slot]), 0)
        for g, group in enumerate(self.groups):
            if needs[g] > group.pool.n_free:
                raise CacheFull(f"the {group.kind} group has {group.pool.n_free} free pages, "
                                f"this step needs {needs[g]}")
        for slot, new_length in wanted:
            self.reserve(slot, new_length)

    def can_hold(self, lengths) -> bool:
        """Whether new sequences of these final lengths fit beside what is held."""
        if len(lengths) > self.slots.n_free or any(n > self.max_seq_len for n in lengths):
            return False
        for group in self.groups:
            pages = sum(min(round_up(n) // PAGE, group.ring_pages) for n in lengths)
            if pages > group.pool.n_free:
                return False
        return True

    def set_length(self, slot: int, length: int) -> None:
        self.lengths[slot] = length

    def length(self, slot: int) -> int:
        return self.lengths[slot]

    # ------------------------------------------------------------------ views for a step

    def table_width(self, group_index: int) -> int:
        return self.groups[group_index].ring_pages

    def block_table_rows(self, group_index: int, slots) -> torch.Tensor:
        """int32 [len(slots), width] on the host: one row of physical pages per
        slot, 0 where the slot has no page yet."""
        return self.groups[group_index].host_table[torch.as_tensor(slots, dtype=torch.long)]

    def layer_view(self, entry: int):
        """(group index, keys, values) of the schedule entry that owns storage:
        keys and values are [pages, Hkv, 64, D]."""
        where = self.entry_group[entry]
        if where is None:
            return None
        g, i = where
        storage = self.groups[g].storage
        return g, storage[i, 0], storage[i, 1]

    def state_view(self, entry: int):
        return self.states[entry]

    def held_tokens(self) -> int:
        """Tokens held now, each sequence rounded up to whole pages."""
        return sum(round_up(self.lengths[s]) for s in range(self.max_slots) if self.slots.is_held(s))

    def bytes(self) -> int:
        total = sum(g.storage.numel() * g.storage.element_size() for g in self.groups)
        total += sum(s.numel() * s.element_size() for s in self.states if s is not None)
        return total

    def check(self) -> None:
        """No slot or page lost, held twice, or shared between two slots."""
        self.slots.check()
        for group in self.groups:
            group.pool.check()
            owners = {}
            for slot, pages in group.slot_pages.items():
                if not self.slots.is_held(slot):
                    raise LlmError(f"freed slot {slot} still lists pages")
                for page in pages:
                    if page in owners:
                        raise LlmError(f"page {page} is held by slots {owners[page]} and {slot}")
                    if not group.pool.is_held(page):
                        raise LlmError(f"slot {slot} lists page {page} that is on the free list")
                    owners[page] = slot
            if len(owners) != group.pool.n_held:
                raise LlmError(f"{group.pool.n_held - len(owners)} pages are held by no slot")
