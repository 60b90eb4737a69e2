"""The native host library through its C boundary: the checks and the packing of a step,
the placement of scratch buffers, and the JSON reader behind the safetensors reader."""
import json
import struct
from ctypes import byref, c_longlong

import pytest
import torch

from llm_b200 import native
from llm_b200.cache import KvRequest, PagedCache
from llm_b200.engine.step import Entry, _Batch
from llm_b200.engine.workspace import BufferRequest, plan
from llm_b200.errors import ContextFull, FormatError, LlmError
from llm_b200.weights import SafetensorsFile


def make_cache():
    requests = [KvRequest(2, 16), KvRequest(2, 16, window=70), KvRequest(2, 16)]
    return PagedCache(requests, [None] * 3, max_tokens=64 * 12, max_seq_len=64 * 6, max_slots=4,
                      dtype=torch.float32, device="cpu", step_tokens=64)


def check(cache, entries, vocab=100, max_seq_len=64 * 6):
    batch = _Batch(entries)
    native.check(native.lib().llmh_step_check(cache._handle, *batch.arguments(), vocab, max_seq_len))


def test_a_step_is_refused_before_anything_changes():
    cache = make_cache()
    a, b = cache.acquire(), cache.acquire()
    check(cache, [Entry(a, [1, 2, 3], [2]), Entry(b, [4], [])])
    with pytest.raises(FormatError, match="appears twice"):
        check(cache, [Entry(a, [1], [0]), Entry(a, [2], [0])])
    with pytest.raises(FormatError, match="brings no token"):
        check(cache, [Entry(a, [], [])])
    with pytest.raises(FormatError, match="token id 100 is outside the vocabulary of 100"):
        check(cache, [Entry(a, [5, 100], [0])])
    with pytest.raises(FormatError, match="token id -1"):
        check(cache, [Entry(a, [-1], [0])])
    with pytest.raises(FormatError, match="wanted place 3 is outside the 3 tokens of slot"):
        check(cache, [Entry(a, [1, 2, 3], [3])])
    with pytest.raises(LlmError, match="slot 3 is not held"):
        check(cache, [Entry(3, [1], [0])])
    with pytest.raises(FormatError, match="32-bit"):
        check(cache, [Entry(a, [2 ** 40], [0])])
    cache.reserve(a, 64 * 6)
    cache.set_length(a, 64 * 6 - 1)
    check(cache, [Entry(a, [1], [0])])
    with pytest.raises(ContextFull) as full:
        check(cache, [Entry(a, [1, 2], [0])])
    assert (full.value.used, full.value.capacity) == (64 * 6 + 1, 64 * 6)
    assert cache.length(a) == 64 * 6 - 1 and cache.length(b) == 0
    cache.check()


def test_packing_of_an_unequal_batch():
    cache = make_cache()
    lib = native.lib()
    slots = [cache.acquire() for _ in range(3)]
    cache.release(slots[1])                                    # leaves slots 0 and 2
    a, c = slots[0], slots[2]
    cache.reserve(a, 70)
    cache.set_length(a, 70)                                    # a continues at position 70
    entries = [Entry(c, list(range(10, 15)), [4, 0]), Entry(a, [7, 8], [1])]
    batch = _Batch(entries)
    native.check(lib.llmh_step_reserve(cache._handle, batch.n, batch.slots, batch.counts))
    n_sections = lib.llmh_step_sections(cache._handle)
    assert n_sections == 8 + 2                                 # two cache groups: full, window
    offsets, sizes = (c_longlong * n_sections)(), (c_longlong * n_sections)()
    total, summary = c_longlong(), (c_longlong * 5)()
    native.check(lib.llmh_step_layout(cache._handle, batch.n, batch.counts, batch.want_counts, offsets, sizes,
                                      byref(total)))
    host = torch.full((total.value + 8,), -7, dtype=torch.int32)
    native.check(lib.llmh_step_pack(cache._handle, *batch.arguments(), host.data_ptr(), total.value, offsets,
                                    sizes, summary))
    section = lambda i: host[offsets[i]:offsets[i] + sizes[i]].tolist()
    assert all(o % 4 == 0 for o in offsets)                    # 16-byte boundaries
    assert section(0) == [10, 11, 12, 13, 14, 7, 8]
    assert section(1) == [0, 1, 2, 3, 4, 70, 71]
    assert section(2) == [0] * 5 + [1] * 2
    assert section(3) == [0, 5, 7]
    assert section(4) == [5, 72]
    assert section(5) == [c, a]
    assert section(6) == [4, 0, 6]                             # rows among the packed tokens
    assert section(7) == [1, 0]                                # the longer sequence (72 positions) first
    for g in range(2):
        width = cache.table_width(g)
        assert section(8 + g) == cache.block_table_rows(g, [c, a]).reshape(-1).tolist()
        assert sizes[8 + g] == 2 * width
    assert list(summary) == [7, 3, 0, 72, total.value]
    assert host[total.value:].tolist() == [-7] * 8             # nothing written past the end
    with pytest.raises(LlmError, match="the step needs"):
        native.check(lib.llmh_step_pack(cache._handle, *batch.arguments(), host.data_ptr(), 8, offsets, sizes,
                                        summary))
    native.check(lib.llmh_step_commit(cache._handle, batch.n, batch.slots, batch.counts))
    assert cache.length(c) == 5 and cache.length(a) == 72
    cache.check()


def test_a_decode_batch_is_recognised():
    cache = make_cache()
    lib = native.lib()
    slots = [cache.acquire() for _ in range(4)]
    batch = _Batch([Entry(s, [3], [0]) for s in slots])
    native.check(lib.llmh_step_reserve(cache._handle, batch.n, batch.slots, batch.counts))
    n = lib.llmh_step_sections(cache._handle)
    offsets, sizes, summary = (c_longlong * n)(), (c_longlong * n)(), (c_longlong * 5)()
    host = torch.zeros(4096, dtype=torch.int32)
    native.check(lib.llmh_step_pack(cache._handle, *batch.arguments(), host.data_ptr(), host.numel(), offsets,
                                    sizes, summary))
    assert summary[2] == 1 and summary[3] == 1


def test_planner_refuses_bad_requests_and_orders_by_first_use():
    f32 = torch.float32
    with pytest.raises(ValueError, match="share the name"):
        plan([BufferRequest("x", (4,), f32, 0, 1), BufferRequest("x", (4,), f32, 1, 2)])
    with pytest.raises(ValueError, match="read before it is written"):
        plan([BufferRequest("x", (4,), f32, 3, 1)])
    p = plan([BufferRequest("late", (100,), f32, 2, 3), BufferRequest("early", (100,), f32, 0, 1),
              BufferRequest("long", (10,), f32, 0, 3)])
    p.check()
    assert p.placements["early"].offset == 0                   # placed first: first use 0, name before "long"
    assert p.placements["late"].offset == 0                    # reuses the bytes of "early"
    assert p.placements["long"].offset == 512 and p.total == 768


def write_raw(path, header_text: bytes, data: bytes = b""):
    path.write_bytes(struct.pack("<Q", len(header_text)) + header_text + data)


def test_json_reader_behind_the_safetensors_header(tmp_path):
    name = 'layer "ü"\\\n\t\U0001F600'
    header = {name: {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
              "__metadata__": {"k": "vé", "ignored": 3}}
    path = tmp_path / "a.safetensors"
    write_raw(path, json.dumps(header).encode("utf-8"), struct.pack("<2f", 1.5, -2.0))      # \\u escapes
    f = SafetensorsFile(path)
    assert f.names() == [name] and f.metadata == {"k": "vé"}
    assert f.tensor(name).tolist() == [1.5, -2.0]
    write_raw(path, json.dumps(header, ensure_ascii=False).encode("utf-8"), struct.pack("<2f", 1.5, -2.0))
    assert SafetensorsFile(path).names() == [name]                                           # raw UTF-8
    for bad in [b'{"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]},}',         # trailing comma
                b'{"a": {"dtype": "F32", "shape": [1.5], "data_offsets": [0, 4]}}',        # a real as a size
                b'{"a": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 4]}}',
                b'{"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}} x',         # text after the value
                b'{"a": {"dtype": "F32", "shape": [1], "data_offsets": [0]}}',
                b'{"a": "\\q"}', b'[1, 2]', b'{"a": {"dtype": "F32", "shape": [4611686018427387904, 4], "data_offsets": [0, 4]}}',
                b'[' * 100]:
        write_raw(path, bad, b"\0" * 4)
        with pytest.raises(FormatError):
            SafetensorsFile(path)


def test_a_tensor_keeps_its_file_mapped(tmp_path):
    import gc
    path = tmp_path / "b.safetensors"
    header = {"w": {"dtype": "I32", "shape": [3], "data_offsets": [0, 12]}}
    write_raw(path, json.dumps(header).encode(), struct.pack("<3i", 4, 5, 6))
    t = SafetensorsFile(path).tensor("w")
    gc.collect()
    assert t.tolist() == [4, 5, 6]


def test_generation_schedule_decisions():
    """Stop tokens are neither emitted nor fed, limits end a sequence after the token that reaches
    them, a full context ends it after the token that was sampled from its last position, and
    sequences that may emit nothing leave before sampling."""
    from llm_b200.engine.generate import GenerationRequest, _Schedule
    reqs = [GenerationRequest([1], max_tokens=3, stop_tokens=(9,)),       # ends by its limit
            GenerationRequest([1], max_tokens=5, stop_tokens=(9, 7)),     # draws a stop token
            GenerationRequest([1], max_tokens=0),                         # may emit nothing
            GenerationRequest([1], max_tokens=8)]                         # runs into the context's end
    s = _Schedule(reqs, max_seq_len=10)
    assert s.live() == [0, 1, 2, 3]
    rows, exhausted = s.drop_exhausted()
    assert rows == [0, 1, 3] and exhausted == [2] and s.live() == [0, 1, 3]
    onward = s.plan_onward([4, 4, 9])                     # sequence 3 holds 9 of 10 positions: room for one
    assert onward == [0, 1, 2]
    counts, finished, going = s.take_tokens([5, 6, 4])
    assert counts == [1, 1, 1] and finished == [] and going == [0, 1, 2]
    assert s.drop_exhausted() == ([0, 1, 2], [])
    onward = s.plan_onward([5, 5, 10])                    # sequence 3 is full now: it does not go on
    assert onward == [0, 1]
    counts, finished, going = s.take_tokens([5, 7, 4])
    assert counts == [1, 0, 1]                            # the stop token is not output
    assert finished == [(1, "eos"), (3, "context_full")] and going == [0] and s.live() == [0]
    assert s.plan_onward([6]) == []                       # its third token is its last: nothing to queue
    counts, finished, going = s.take_tokens([9])
    assert counts == [0] and finished == [(0, "eos")] and s.live() == []
    t = _Schedule(reqs[:2], max_seq_len=10)
    assert t.cancel() == [0, 1] and t.live() == []
    with pytest.raises(LlmError):
        _Schedule(reqs[:1], 10).take_tokens([1])          # tokens without a planned step


def test_json_reader_gives_the_values_python_would(tmp_path):
    text = ('{"a": 1, "b": -2.5e3, "c": [true, false, null, "x\\u00e9\\n", [], {}], "d": {"e": {"f": [1, 2]}},'
            ' "n": 123456789012345678, "s": ""}')
    assert native.read_json(text) == json.loads(text)
    assert native.read_json("12345678901234567890") == 1.2345678901234567e19      # beyond 64 bits: a real
    assert native.read_json(b"[]") == [] and native.read_json("3") == 3 and native.read_json('"q"') == "q"
    for bad in ['{"a": 1,}', "{'a': 1}", '{"a" 1}', "[1 2]", "", "nul", '{"a": 01x}', '"\\x"', "[" * 80]:
        with pytest.raises(FormatError):
            native.read_json(bad, "here")
    from llm_b200.config import load_config
    (tmp_path / "config.json").write_text("[1, 2]")
    with pytest.raises(FormatError, match="must be a JSON object"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text('{"architectures": ["LlamaForCausalLM"],')
    with pytest.raises(FormatError, match="not JSON"):
        load_config(tmp_path)


def test_a_plan_calls_its_doors_in_order_with_their_slots_and_stops_at_a_failure():
    """llmh_plan_run (csrc/host/plan_run.cpp) with doors made here: every door gets its own block of
    8-byte slots, the stream is written into the slot that was named for it, and the first non-zero
    code ends the walk with the index of the launch that returned it."""
    import ctypes
    from llm_b200 import native
    lib = native.lib()
    seen = []
    DOOR = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(ctypes.c_ulonglong))

    def make(n_slots, code=0):
        def door(slots):
            seen.append([slots[i] for i in range(n_slots)])
            return code
        return DOOR(door)

    doors = [make(3), make(1), make(2)]
    slots = (ctypes.c_ulonglong * 6)(11, 12, 0, 0, 21, 0)
    handle = ctypes.c_void_p()
    native.check(lib.llmh_plan_create(
        3, (ctypes.c_void_p * 3)(*[ctypes.cast(d, ctypes.c_void_p).value for d in doors]),
        native.ints([3, 1, 2]), native.ints([2, 0, -1]), ctypes.cast(slots, ctypes.c_void_p), ctypes.byref(handle)))
    assert lib.llmh_plan_size(handle) == 3
    failed = ctypes.c_int(7)
    assert lib.llmh_plan_run(handle, ctypes.c_void_p(0xABC0), ctypes.byref(failed)) == 0 and failed.value == -1
    assert seen == [[11, 12, 0xABC0], [0xABC0], [21, 0]]
    lib.llmh_plan_destroy(handle)
    # a door that fails ends the walk
    seen.clear()
    doors = [make(1), make(1, code=5), make(1)]
    native.check(lib.llmh_plan_create(
        3, (ctypes.c_void_p * 3)(*[ctypes.cast(d, ctypes.c_void_p).value for d in doors]),
        native.ints([1, 1, 1]), native.ints([-1, -1, -1]), ctypes.cast((ctypes.c_ulonglong * 3)(1, 2, 3), ctypes.c_void_p),
        ctypes.byref(handle)))
    assert lib.llmh_plan_run(handle, None, ctypes.byref(failed)) == 5 and failed.value == 1
    assert seen == [[1], [2]]
    lib.llmh_plan_destroy(handle)
    with pytest.raises(Exception):
        native.check(lib.llmh_plan_create(1, (ctypes.c_void_p * 1)(None), native.ints([1]), native.ints([0]),
                                          ctypes.cast(slots, ctypes.c_void_p), ctypes.byref(handle)))
