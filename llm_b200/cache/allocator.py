"""Free lists of slots and pages.

A slot stands for one live sequence; a page holds the keys and values of 64
consecutive positions of one sequence for every layer of a group. Both come
from free lists and go back to them when the sequence ends; taking a slot or
page that is held, or returning one that is free, is an error, never silent.
The lists themselves live in the native host library (`csrc/host/free_list.hpp`);
this class is a handle on one of them.
"""
from __future__ import annotations

from ctypes import byref, c_int, c_void_p

from .. import native


class FreeList:
    """Integers 0 .. count-1, handed out lowest first and taken back."""

    def __init__(self, count: int, what: str, _borrowed=None, _owner=None):
        self.what = what
        self._owned = _borrowed is None
        self._owner = _owner             # a borrowed list lives as long as the cache it belongs to
        if self._owned:
            handle = c_void_p()
            native.check(native.lib().llmh_free_list_create(int(count), what.encode(), byref(handle)))
            self._handle = handle
        else:
            self._handle = c_void_p(_borrowed)

    def __del__(self):
        if getattr(self, "_owned", False) and self._handle:
            native.lib().llmh_free_list_destroy(self._handle)
            self._handle = None

    def _counts(self):
        count, n_free = c_int(), c_int()
        native.lib().llmh_free_list_counts(self._handle, byref(count), byref(n_free))
        return count.value, n_free.value

    @property
    def count(self) -> int:
        return self._counts()[0]

    @property
    def n_free(self) -> int:
        return self._counts()[1]

    @property
    def n_held(self) -> int:
        count, n_free = self._counts()
        return count - n_free

    def take(self) -> int:
        item = c_int()
        native.check(native.lib().llmh_free_list_take(self._handle, byref(item)))
        return item.value

    def give_back(self, item: int) -> None:
        native.check(native.lib().llmh_free_list_give_back(self._handle, int(item)))

    def is_held(self, item: int) -> bool:
        return bool(native.lib().llmh_free_list_is_held(self._handle, int(item)))

    def check(self) -> None:
        """Every item is either free once or held, never both or neither."""
        native.check(native.lib().llmh_free_list_check(self._handle))
