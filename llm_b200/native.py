"""The native host library (`csrc/host/*.cpp`), loaded through its C boundary.

It holds the host-side runtime that does not touch the GPU: the cache's
bookkeeping (slots, pages, page tables), the checks and the packing of a step,
the placement of scratch buffers and the safetensors reader, the parts that
MythEclipse/llm has in its Rust engine crate (apps/engine/src/model.rs:351-436,
workspace.rs, gguf.rs). The Python classes above it keep the tensors and the
composition of the model; they ask this library what goes where. It is
compiled with the host C++ compiler on first use; without it the package
raises.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, byref, c_char_p, c_double, c_int, c_longlong, c_void_p

from .errors import CacheFull, ContextFull, FormatError, LlmError

_lib = None

OK, FORMAT, INVARIANT, CACHE_FULL, CONTEXT_FULL, IO = range(6)


_P = c_void_p
_INTS, _LONGS = POINTER(c_int), POINTER(c_longlong)
_BATCH = [c_int, _INTS, _INTS, _INTS, _INTS, _INTS]      # n, slots, counts, tokens, want counts, wants

# name: (result type, argument types); the declarations are in the .cpp files of csrc/host
_SIGNATURES = {
    "llmh_plan_constant": (c_int, [c_int]),
    "llmh_last_error": (c_char_p, []),
    "llmh_last_error_numbers": (None, [_LONGS, _LONGS]),
    "llmh_free_list_create": (c_int, [c_int, c_char_p, POINTER(_P)]),
    "llmh_free_list_destroy": (None, [_P]),
    "llmh_free_list_take": (c_int, [_P, _INTS]),
    "llmh_free_list_give_back": (c_int, [_P, c_int]),
    "llmh_free_list_is_held": (c_int, [_P, c_int]),
    "llmh_free_list_counts": (None, [_P, _INTS, _INTS]),
    "llmh_free_list_check": (c_int, [_P]),
    "llmh_cache_create": (c_int, [c_longlong, c_int, c_int, c_int, c_int, _INTS, POINTER(_P)]),
    "llmh_cache_destroy": (None, [_P]),
    "llmh_cache_list": (_P, [_P, c_int]),
    "llmh_cache_group_info": (None, [_P, c_int, _INTS, _INTS]),
    "llmh_cache_max_tokens": (c_longlong, [_P]),
    "llmh_cache_acquire": (c_int, [_P, _INTS]),
    "llmh_cache_release": (c_int, [_P, c_int]),
    "llmh_cache_reserve": (c_int, [_P, c_int, c_longlong]),
    "llmh_cache_reserve_many": (c_int, [_P, c_int, _INTS, _LONGS]),
    "llmh_cache_can_hold": (c_int, [_P, c_int, _LONGS]),
    "llmh_cache_length": (c_int, [_P, c_int, _INTS]),
    "llmh_cache_set_length": (c_int, [_P, c_int, c_int]),
    "llmh_cache_held_tokens": (c_longlong, [_P]),
    "llmh_cache_slot_pages": (c_int, [_P, c_int, c_int, _INTS, c_int, _INTS]),
    "llmh_cache_table_rows": (c_int, [_P, c_int, c_int, _INTS, _P]),
    "llmh_cache_check": (c_int, [_P]),
    "llmh_step_check": (c_int, [_P, *_BATCH, c_int, c_int]),
    "llmh_step_reserve": (c_int, [_P, c_int, _INTS, _INTS]),
    "llmh_step_sections": (c_int, [_P]),
    "llmh_step_layout": (c_int, [_P, c_int, _INTS, _INTS, _LONGS, _LONGS, _LONGS]),
    "llmh_step_pack": (c_int, [_P, *_BATCH, _P, c_longlong, _LONGS, _LONGS, _LONGS]),
    "llmh_step_commit": (c_int, [_P, c_int, _INTS, _INTS]),
    "llmh_plan_place": (c_int, [c_int, POINTER(c_char_p), _LONGS, _INTS, _INTS, c_longlong, _LONGS, _LONGS]),
    "llmh_json_parse": (c_int, [c_char_p, c_longlong, c_char_p, POINTER(_P)]),
    "llmh_json_free": (None, [_P]),
    "llmh_json_count": (c_int, [_P]),
    "llmh_json_node": (c_int, [_P, c_int, _INTS, POINTER(c_char_p), POINTER(c_char_p), _LONGS, POINTER(c_double),
                               _INTS]),
    "llmh_generation_create": (c_int, [c_int, _INTS, _INTS, _INTS, c_int, POINTER(_P)]),
    "llmh_generation_destroy": (None, [_P]),
    "llmh_generation_live": (c_int, [_P, _INTS]),
    "llmh_generation_drop_exhausted": (c_int, [_P, _INTS, _INTS, _INTS, _INTS]),
    "llmh_generation_plan_onward": (c_int, [_P, _INTS, _INTS, _INTS]),
    "llmh_generation_take_tokens": (c_int, [_P, _INTS, _INTS, _INTS, _INTS, _INTS, _INTS, _INTS]),
    "llmh_generation_cancel": (c_int, [_P, _INTS, _INTS]),
    "llmh_tactics_choose": (c_int, [c_int, _INTS, c_char_p, c_int, c_char_p, c_int]),
    "llmh_tactics_set_disabled": (None, [c_char_p, c_int]),
    "llmh_tactics_is_disabled": (c_int, [c_char_p]),
    "llmh_tactics_rows": (c_int, [c_int]),
    "llmh_tactics_row": (c_int, [c_int, c_int, POINTER(c_char_p), _INTS, POINTER(c_char_p)]),
    "llmh_plan_create": (c_int, [c_int, POINTER(_P), _INTS, _INTS, _P, POINTER(_P)]),
    "llmh_plan_destroy": (None, [_P]),
    "llmh_plan_size": (c_int, [_P]),
    "llmh_plan_run": (c_int, [_P, _P, _INTS]),
    "llmh_random_normal": (c_int, [_P, c_int, c_longlong, ctypes.c_ulonglong, ctypes.c_float, ctypes.c_float]),
    "llmh_safetensors_open": (c_int, [c_char_p, POINTER(_P)]),
    "llmh_safetensors_close": (None, [_P]),
    "llmh_safetensors_count": (c_int, [_P]),
    "llmh_safetensors_entry": (c_int, [_P, c_int, POINTER(c_char_p), POINTER(c_char_p), _INTS, POINTER(_LONGS),
                                       POINTER(_P), _LONGS]),
    "llmh_safetensors_metadata_count": (c_int, [_P]),
    "llmh_safetensors_metadata_item": (c_int, [_P, c_int, POINTER(c_char_p), POINTER(c_char_p)]),
}


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        from .ops.build import load_host_library
        loaded = load_host_library()
        for name, (result, arguments) in _SIGNATURES.items():
            function = getattr(loaded, name)
            function.restype = result
            function.argtypes = arguments
        _lib = loaded
    return _lib


def check(code: int) -> None:
    """Raise the library's error for a non-zero return code."""
    if code == OK:
        return
    text = lib().llmh_last_error().decode("utf-8", "replace")
    if code == CONTEXT_FULL:
        first, second = c_longlong(), c_longlong()
        lib().llmh_last_error_numbers(byref(first), byref(second))
        raise ContextFull(first.value, second.value)
    if code == CACHE_FULL:
        raise CacheFull(text)
    if code in (FORMAT, IO):
        raise FormatError(text)
    raise LlmError(text)


def ints(values, ctype=c_int):
    """A C array from a sequence of Python ints."""
    values = list(values)
    return (ctype * len(values))(*values)


def plan_constant(name: str) -> int:
    """A constant of csrc/plan.h, the one definition shared by kernels, host library and Python."""
    return lib().llmh_plan_constant({"page": 0, "glu_block": 1, "max_head_dim": 2}[name])


def read_json(text, where: str = "text"):
    """The value of a JSON document (bytes or str), read by the host library's own reader;
    FormatError with the byte position if it is not JSON."""
    data = text.encode("utf-8") if isinstance(text, str) else bytes(text)
    document = c_void_p()
    check(lib().llmh_json_parse(data, len(data), where.encode("utf-8", "replace"), byref(document)))
    try:
        kind, key, string = c_int(), c_char_p(), c_char_p()
        integer, real, children = c_longlong(), c_double(), c_int()
        at = [0]

        def build():
            check(lib().llmh_json_node(document, at[0], byref(kind), byref(key), byref(string), byref(integer),
                                       byref(real), byref(children)))
            at[0] += 1
            k, n = kind.value, children.value
            if k == 0:
                return None
            if k == 1:
                return bool(integer.value)
            if k == 2:
                return integer.value
            if k == 3:
                return real.value
            if k == 4:
                return string.value.decode("utf-8")
            if k == 5:
                return [build() for _ in range(n)]
            out = {}
            for _ in range(n):
                check(lib().llmh_json_node(document, at[0], byref(kind), byref(key), byref(string),
                                           byref(integer), byref(real), byref(children)))
                name = key.value.decode("utf-8")
                out[name] = build()
            return out

        return build()
    finally:
        lib().llmh_json_free(document)
