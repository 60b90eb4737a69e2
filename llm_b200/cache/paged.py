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
  page pool [layers, 2, pages, kv heads, 64, head_dim] (or, for a mixer whose
  values are wider or narrower than its keys, one tensor for the keys and one
  for the values) and, per slot, its own list of pages: logical page i of a
  sequence is `pages[i % ring]`;
* `state` tensors [slots, ...] hold what a mixer keeps per sequence at a fixed
  size; a slot's rows are zeroed when the slot is taken.

Slots and pages are given back by `release` and reused. Which page holds what is
decided by the native host library (`csrc/host/cache.cpp`); this class owns the
tensors and hands out views of them.
"""
from __future__ import annotations

from ctypes import byref, c_int, c_longlong, c_void_p
from dataclasses import dataclass, field

import torch

from .. import native
from .allocator import FreeList

PAGE = native.plan_constant("page")      # positions per cache page (csrc/plan.h)


def round_up(n: int, unit: int = PAGE) -> int:
    return (n + unit - 1) // unit * unit


@dataclass(frozen=True)
class KvRequest:
    """What one cache-owning run of a layer asks of the cache."""
    n_kv_heads: int
    head_dim: int
    window: int = 0            # 0: keep every position
    value_dim: int | None = None   # width of a value, where it differs from a key's (None: head_dim)

    @property
    def group_key(self):
        return ("window" if self.window else "full", self.n_kv_heads, self.head_dim, self.window,
                self.value_dim or self.head_dim)


@dataclass(frozen=True)
class StateRequest:
    """Fixed-size per-sequence state: one tensor [slots, *shape] of `dtype`."""
    shape: tuple
    dtype: torch.dtype = torch.float32


class _SlotPages:
    """slot -> list of the slot's physical pages in one group (read from the native cache)."""

    def __init__(self, cache, group_index: int):
        self._cache, self._group = cache, group_index

    def __getitem__(self, slot: int) -> list:
        width = self._cache.groups[self._group].ring_pages
        pages, count = (c_int * width)(), c_int()
        native.check(native.lib().llmh_cache_slot_pages(self._cache._handle, self._group, int(slot), pages,
                                                        width, byref(count)))
        return list(pages[:count.value])

    def _held(self):
        return [s for s in range(self._cache.max_slots) if self._cache.slots.is_held(s)]

    def items(self):
        return [(s, self[s]) for s in self._held()]

    def values(self):
        return [self[s] for s in self._held()]


@dataclass
class Group:
    kind: str
    n_kv_heads: int
    head_dim: int
    window: int
    value_dim: int = 0                                # width of a value (== head_dim unless a mixer asks otherwise)
    entries: list = field(default_factory=list)     # schedule positions that own storage here
    ring_pages: int = 0                               # logical pages per sequence
    pool: FreeList | None = None
    storage: torch.Tensor | None = None               # [entries, 2, pages, Hkv, PAGE, D] (keys and values alike)
    keys: torch.Tensor | None = None                  # [entries, pages, Hkv, PAGE, D] and
    values: torch.Tensor | None = None                # [entries, pages, Hkv, PAGE, value_dim] where they differ
    slot_pages: _SlotPages | None = None              # slot -> list of physical pages


class PagedCache:
    """See the module text. `requests[i]` is the KvRequest of schedule entry i
    (None if that run keeps no keys of its own); `states[i]` its StateRequest or
    None. `max_tokens` bounds the tokens held by all live sequences together,
    each rounded up to a multiple of 64; `max_seq_len` bounds one sequence;
    `step_tokens` bounds the new tokens of one sequence in one step (it sizes
    the ring of window groups)."""

    def __init__(self, requests, states, max_tokens: int, max_seq_len: int, max_slots: int,
                 dtype, device, step_tokens: int | None = None):
        self.max_seq_len = max_seq_len
        self.max_slots = max_slots
        self.dtype = dtype
        self.device = torch.device(device)
        self.step_tokens = step_tokens or max_seq_len
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
                self.groups.append(Group(key[0], request.n_kv_heads, request.head_dim, request.window,
                                         request.value_dim or request.head_dim))
            g = by_key[key]
            self.entry_group.append((g, len(self.groups[g].entries)))
            self.groups[g].entries.append(entry)
        lib = native.lib()
        handle = c_void_p()
        native.check(lib.llmh_cache_create(c_longlong(int(max_tokens)), int(max_seq_len), int(max_slots),
                                           int(self.step_tokens), len(self.groups),
                                           native.ints(g.window for g in self.groups), byref(handle)))
        self._handle = handle
        self.max_tokens = lib.llmh_cache_max_tokens(handle)
        self.slots = FreeList(max_slots, "slot", _borrowed=lib.llmh_cache_list(handle, -1), _owner=self)
        for g, group in enumerate(self.groups):
            ring, n_pages = c_int(), c_int()
            lib.llmh_cache_group_info(handle, g, byref(ring), byref(n_pages))
            group.ring_pages = ring.value
            group.pool = FreeList(n_pages.value, f"page of the {group.kind} group",
                                  _borrowed=lib.llmh_cache_list(handle, g), _owner=self)
            group.slot_pages = _SlotPages(self, g)
            if group.value_dim == group.head_dim:
                group.storage = torch.zeros(
                    (len(group.entries), 2, n_pages.value, group.n_kv_heads, PAGE, group.head_dim),
                    dtype=dtype, device=self.device)
            else:
                shape = (len(group.entries), n_pages.value, group.n_kv_heads, PAGE)
                group.keys = torch.zeros(shape + (group.head_dim,), dtype=dtype, device=self.device)
                group.values = torch.zeros(shape + (group.value_dim,), dtype=dtype, device=self.device)
        self.states = []
        for request in states:
            if request is None:
                self.states.append(None)
            else:
                self.states.append(torch.zeros((max_slots, *request.shape), dtype=request.dtype,
                                               device=self.device))

    def __del__(self):
        handle = getattr(self, "_handle", None)
        if handle:
            native.lib().llmh_cache_destroy(handle)
            self._handle = None

    # ------------------------------------------------------------------ slots

    def acquire(self) -> int:
        """Take a free slot: length 0, no pages, state zeroed."""
        slot = c_int()
        native.check(native.lib().llmh_cache_acquire(self._handle, byref(slot)))
        for state in self.states:
            if state is not None:
                state[slot.value].zero_()
        return slot.value

    def release(self, slot: int) -> None:
        """Give the slot and all of its pages back."""
        native.check(native.lib().llmh_cache_release(self._handle, int(slot)))

    def reserve(self, slot: int, new_length: int) -> None:
        """Make sure the slot has pages for positions < new_length. Raises
        ContextFull or CacheFull before anything is changed."""
        native.check(native.lib().llmh_cache_reserve(self._handle, int(slot), c_longlong(int(new_length))))

    def reserve_many(self, wanted) -> None:
        """`reserve` for several (slot, new_length) pairs: all of them or none."""
        wanted = list(wanted)
        native.check(native.lib().llmh_cache_reserve_many(
            self._handle, len(wanted), native.ints(s for s, _ in wanted),
            native.ints((n for _, n in wanted), c_longlong)))

    def can_hold(self, lengths) -> bool:
        """Whether new sequences of these final lengths fit beside what is held."""
        lengths = list(lengths)
        return bool(native.lib().llmh_cache_can_hold(self._handle, len(lengths), native.ints(lengths, c_longlong)))

    def set_length(self, slot: int, length: int) -> None:
        native.check(native.lib().llmh_cache_set_length(self._handle, int(slot), int(length)))

    def length(self, slot: int) -> int:
        length = c_int()
        native.check(native.lib().llmh_cache_length(self._handle, int(slot), byref(length)))
        return length.value

    # ------------------------------------------------------------------ views for a step

    def table_width(self, group_index: int) -> int:
        return self.groups[group_index].ring_pages

    def block_table_rows(self, group_index: int, slots) -> torch.Tensor:
        """int32 [len(slots), width] on the host: one row of physical pages per
        slot, 0 where the slot has no page yet."""
        slots = [int(s) for s in slots]
        out = torch.zeros((len(slots), self.groups[group_index].ring_pages), dtype=torch.int32)
        native.check(native.lib().llmh_cache_table_rows(self._handle, int(group_index), len(slots),
                                                        native.ints(slots), c_void_p(out.data_ptr())))
        return out

    def layer_view(self, entry: int):
        """(group index, keys, values) of the schedule entry that owns storage:
        keys and values are [pages, Hkv, 64, D]."""
        where = self.entry_group[entry]
        if where is None:
            return None
        g, i = where
        group = self.groups[g]
        if group.storage is None:
            return g, group.keys[i], group.values[i]
        return g, group.storage[i, 0], group.storage[i, 1]

    def state_view(self, entry: int):
        return self.states[entry]

    def held_tokens(self) -> int:
        """Tokens held now, each sequence rounded up to whole pages."""
        return native.lib().llmh_cache_held_tokens(self._handle)

    def bytes(self) -> int:
        total = sum(t.numel() * t.element_size() for g in self.groups
                    for t in (g.storage, g.keys, g.values) if t is not None)
        total += sum(s.numel() * s.element_size() for s in self.states if s is not None)
        return total

    def check(self) -> None:
        """No slot or page lost, held twice, or shared between two slots."""
        native.check(native.lib().llmh_cache_check(self._handle))
