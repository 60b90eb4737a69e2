"""Python bindings of the CUDA kernels in `llm_b200/csrc`.

Every function takes torch tensors that live on the GPU, checks what the
kernel cannot check itself, picks the kernel variant for the shape
(`tactics`) and launches on torch's current stream. There is no CPU path
and no library fallback: a missing or failing library raises KernelError.

The parts call these functions as attributes of this module
(`ops.rmsnorm(...)`).
"""
from __future__ import annotations

import atexit
import ctypes
import functools
import os
import sys

import torch

from .. import native
from ..errors import KernelError
from . import tactics
from .build import all_sources, ensure_built, load_library

PAGE = native.plan_constant("page")              # positions per cache page (csrc/plan.h)
BFLOAT16_ONLY = ("gemm_tc", "gemm_skinny", "attention_decode", "attention_prefill",
                 "attention_prefill_tc")

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
_c_int, _c_float, _c_void = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


def _code(dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} has no kernel (float32 and bfloat16 are built)") from None


def _ptr(t):
    if t is None:
        return None
    if _recording is not None:
        _recording.keep.append(t)          # a recorded pass points at this tensor: it must outlive the record
    return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream's handle (the short way where this torch has it: a launch costs the host
    a few microseconds, the stream object's construction as much again)."""
    if _raw_stream is not None and _current_device is not None:
        return ctypes.c_void_p(_raw_stream(_current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("llm_b200 kernels need tensors on a CUDA device; there is no CPU path")


def _check_out(out, shape, dtype, what: str):
    """Refuse a caller's `out` that the kernel would not fill as the caller thinks: the kernels
    write rows of the result's own width one after the other, so a buffer of another shape,
    dtype or layout would be overrun or garbled without a word."""
    if out is None:
        return
    _require_cuda(out)
    if tuple(out.shape) != tuple(shape) or out.dtype != dtype or not out.is_contiguous():
        raise KernelError(f"{what}: out is {tuple(out.shape)} {out.dtype}"
                          f"{'' if out.is_contiguous() else ' (not contiguous)'}, the result is "
                          f"{tuple(shape)} {dtype}")


_launches = 0


def launch_count() -> int:
    """Kernels of this library launched so far by this process. A step that is
    replayed from a CUDA graph adds the kernels the graph holds."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


# LLMB_PROFILE=1: every launch between two CUDA events, a table of milliseconds and calls per
# kernel entry at exit (the per-launch timing of MythEclipse/llm's LLM_PROFILE=1,
# apps/engine/src/cuda/mod.rs:1857-1866,1917-1972). Profiling switches graph replay off.
PROFILING = os.environ.get("LLMB_PROFILE", "0") not in ("", "0")
_profile: dict = {}


def _report_profile() -> None:
    if not _profile:
        return
    torch.cuda.synchronize()
    rows = []
    for name, events in _profile.items():
        ms = sum(a.elapsed_time(b) for a, b in events)
        rows.append((ms, len(events), name))
    total = sum(r[0] for r in rows) or 1.0
    print(f"[llm_b200] kernel time by entry point ({total:.2f} ms in all)", file=sys.stderr)
    for ms, calls, name in sorted(rows, reverse=True):
        print(f"  {name:28s}{ms:10.3f} ms{calls:8d} calls{ms / calls * 1e3:10.1f} us/call"
              f"{100 * ms / total:7.1f} %", file=sys.stderr)


if PROFILING:
    atexit.register(_report_profile)


# ----------------------------------------------------------------------------- recorded passes

_recording = None           # the Recording that launches are being entered into, or None
_scratch_generation = 0     # grows when a scratch buffer that recorded passes point at is replaced


class Recording:
    """The launches of one pass as they were made: (library, entry point, ctypes arguments)."""

    def __init__(self):
        self.calls, self.keep, self.kernels = [], [], 0


def begin_recording() -> Recording:
    """From here on every launch of this module is also entered into the returned Recording
    (it still runs), until end_recording()."""
    global _recording
    _recording = Recording()
    return _recording


def end_recording() -> None:
    global _recording
    _recording = None


class RecordedPass:
    """A Recording turned into a native plan (csrc/host/plan_run.cpp): `run()` makes the same
    launches with the same arguments on the current stream through the entry points' packed
    doors, in one call of the native host library. The tensors the launches point at are kept
    alive here. Valid while no scratch buffer of this module was replaced
    (`scratch_generation`)."""

    def __init__(self, recording: Recording):
        doors, counts, stream_slots, slots = [], [], [], []
        self._keep = [recording.keep]
        for lib_name, fn_name, args in recording.calls:
            lib = load_library(lib_name)
            door = ctypes.cast(getattr(lib, fn_name + "_packed"), ctypes.c_void_p).value
            doors.append(door)
            counts.append(len(args))
            stream_slots.append(len(args) - 1)            # every launching entry point ends with its stream
            for a in args:
                slots.append(self._slot(a))
        n = len(doors)
        block = (ctypes.c_ulonglong * max(len(slots), 1))(*slots)
        handle = ctypes.c_void_p()
        native.check(native.lib().llmh_plan_create(
            n, (ctypes.c_void_p * max(n, 1))(*doors), native.ints(counts), native.ints(stream_slots),
            ctypes.cast(block, ctypes.c_void_p), ctypes.byref(handle)))
        self._handle = handle
        self.kernels = recording.kernels
        self.launches = n
        self.scratch_generation = _scratch_generation
        self._libraries = [c[0] for c in recording.calls]
        self._failed = ctypes.c_int(-1)

    def _slot(self, a) -> int:
        """The 8-byte slot of a ctypes argument: an address, a widened integer, or a double's bits."""
        if a is None:
            return 0
        if isinstance(a, ctypes.c_void_p):
            return a.value or 0
        if isinstance(a, (ctypes.c_int, ctypes.c_longlong, ctypes.c_ulonglong)):
            return a.value & 0xFFFFFFFFFFFFFFFF
        if isinstance(a, ctypes.c_float):
            return ctypes.c_ulonglong.from_buffer_copy(ctypes.c_double(a.value)).value
        target = getattr(a, "_obj", None)                 # byref(structure): the structure lives on here
        if target is not None:
            self._keep.append(target)
            return ctypes.addressof(target)
        raise KernelError(f"a launch argument of type {type(a).__name__} cannot be recorded")

    def __del__(self):
        handle = getattr(self, "_handle", None)
        if handle and native is not None:                 # (modules are gone when the interpreter ends)
            native.lib().llmh_plan_destroy(handle)
            self._handle = None

    def run(self) -> None:
        global _launches
        code = native.lib().llmh_plan_run(self._handle, _stream(), ctypes.byref(self._failed))
        _launches += self.kernels
        if code != 0:
            lib_name = self._libraries[self._failed.value]
            reader = getattr(load_library(lib_name), f"llmb_{lib_name}_last_error")
            reader.restype = ctypes.c_char_p
            raise KernelError(f"recorded launch {self._failed.value} ({lib_name}): "
                              f"{reader().decode('utf-8', 'replace')}")


def scratch_generation() -> int:
    return _scratch_generation


def _call(lib_name: str, fn_name: str, *args, kernels: int = 1):
    global _launches
    lib = load_library(lib_name)
    _launches += kernels
    if _recording is not None:
        _recording.calls.append((lib_name, fn_name, args))
        _recording.kernels += kernels
    if PROFILING and not torch.cuda.is_current_stream_capturing():
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        code = getattr(lib, fn_name)(*args)
        end.record()
        _profile.setdefault(fn_name, []).append((begin, end))
    else:
        code = getattr(lib, fn_name)(*args)
    if code != 0:
        reader = getattr(lib, f"llmb_{lib_name}_last_error")
        reader.restype = ctypes.c_char_p
        raise KernelError(f"{fn_name}: {reader().decode('utf-8', 'replace')}")


# ----------------------------------------------------------------------------- row-wise

def embed(tokens, table, out=None, scale: float = 1.0, emit=None):
    """x[t, :] = table[tokens[t], :] * scale as float32 [T, hidden]. With `emit` (an Emit) the
    rows are also written as bfloat16 with the sum of their squares: the first norm's input."""
    _require_cuda(tokens, table)
    n, (vocab, hidden) = tokens.numel(), table.shape
    _check_out(out, (n, hidden), torch.float32, "embed")
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    if emit is not None:
        emit.check(n, hidden)
        emit.parts = 1
    _call("elementwise", "llmb_embed", _ptr(tokens), _ptr(table), _c_int(_code(table.dtype)),
          _ptr(out), _c_int(n), _c_int(hidden), _c_int(vocab), _c_float(scale),
          _ptr(emit.rows) if emit is not None else None, _ptr(emit.sumsq) if emit is not None else None,
          _stream())
    return out


SUMSQ_LD = 64          # floats per row of a sum-of-squares array (LLMB_SUMSQ_LD of csrc/fusion.h)


class Emit:
    """Where a product that adds into the residual stream (or the embedding) leaves the next
    norm's input: `rows` bfloat16 [T, hidden], the updated residual rows, and `sumsq` float32
    [T, 64], partial sums of their squares; `parts` says how many of the 64 are in use (set by
    the op that wrote them)."""
    __slots__ = ("rows", "sumsq", "parts")

    def __init__(self, rows, sumsq):
        self.rows, self.sumsq, self.parts = rows, sumsq, 0

    def check(self, n: int, width: int) -> None:
        _require_cuda(self.rows, self.sumsq)
        if (tuple(self.rows.shape) != (n, width) or self.rows.dtype != torch.bfloat16 or not self.rows.is_contiguous()
                or tuple(self.sumsq.shape) != (n, SUMSQ_LD) or self.sumsq.dtype != torch.float32
                or not self.sumsq.is_contiguous()):
            raise KernelError(f"emit: rows must be contiguous bfloat16 [{n}, {width}] and sumsq float32 "
                              f"[{n}, {SUMSQ_LD}]")


class FoldedNorm:
    """The input of a product whose norm is folded into it: `rows` are the un-normalised rows as
    bfloat16, the norm's gain is already multiplied into the weight's columns, and the product
    scales result row t by 1 / sqrt(sum(sumsq[t, :parts]) / width + eps)."""
    __slots__ = ("rows", "sumsq", "parts", "eps", "width")

    def __init__(self, rows, sumsq, parts: int, eps: float, width: int):
        self.rows, self.sumsq, self.parts, self.eps, self.width = rows, sumsq, parts, eps, width


class RopeWrite:
    """The rotation and cache write behind the q/k/v product (the arguments of rope_cache_write)."""
    __slots__ = ("table", "tok_pos", "tok_seq", "block_table", "ring_pages", "k_cache", "v_cache",
                 "n_heads", "n_kv_heads", "head_dim", "interleaved", "write_cache")

    def __init__(self, table, tok_pos, tok_seq, block_table, ring_pages, k_cache, v_cache, n_heads,
                 n_kv_heads, head_dim, interleaved=False, write_cache=True):
        self.table, self.tok_pos, self.tok_seq, self.block_table = table, tok_pos, tok_seq, block_table
        self.ring_pages, self.k_cache, self.v_cache = ring_pages, k_cache, v_cache
        self.n_heads, self.n_kv_heads, self.head_dim = n_heads, n_kv_heads, head_dim
        self.interleaved, self.write_cache = interleaved, write_cache


class _Fusion(ctypes.Structure):
    """llmb_gemm_fusion of csrc/fusion.h."""
    _fields_ = [("norm_sumsq", ctypes.c_void_p), ("norm_parts", ctypes.c_int), ("norm_eps", ctypes.c_float),
                ("norm_width", ctypes.c_float), ("emit_rows", ctypes.c_void_p), ("emit_sumsq", ctypes.c_void_p),
                ("rope", ctypes.c_int), ("interleaved", ctypes.c_int), ("write_cache", ctypes.c_int),
                ("n_heads", ctypes.c_int), ("n_kv_heads", ctypes.c_int), ("head_dim", ctypes.c_int),
                ("rope_table", ctypes.c_void_p), ("tok_pos", ctypes.c_void_p), ("tok_seq", ctypes.c_void_p),
                ("block_table", ctypes.c_void_p), ("table_stride", ctypes.c_int), ("ring_pages", ctypes.c_int),
                ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p)]


FUSED_NORM, FUSED_EMIT, FUSED_ROPE = 1, 2, 4


def cast_sumsq(x, emit: Emit):
    """emit.rows = bfloat16(x), emit.sumsq[:, 0] = the rows' sums of squares (x float32 [T, hidden])."""
    _require_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("cast_sumsq: x must be contiguous float32")
    emit.check(x.shape[0], x.shape[1])
    _call("elementwise", "llmb_cast_sumsq", _ptr(x), _ptr(emit.rows), _ptr(emit.sumsq), _c_int(x.shape[0]),
          _c_int(x.shape[1]), _stream())
    emit.parts = 1
    return emit


def random_normal_(out, key: int, mean: float, deviation: float):
    """out[i] = mean + deviation * N(0, 1) drawn from (key, i); float32 or bfloat16, contiguous."""
    _require_cuda(out)
    if not out.is_contiguous():
        raise KernelError("random_normal_: the tensor must be contiguous")
    _call("elementwise", "llmb_random_normal", _ptr(out), _c_int(_code(out.dtype)),
          ctypes.c_longlong(out.numel()), ctypes.c_ulonglong(key), _c_float(mean), _c_float(deviation),
          _stream())
    return out


def scale_(x, scale: float):
    """x *= scale in place (float32, contiguous)."""
    _require_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("scale_: the tensor must be contiguous float32")
    _call("elementwise", "llmb_scale", _ptr(x), ctypes.c_longlong(x.numel()), _c_float(scale), _stream())
    return x


def rmsnorm(x, gain, eps, out_dtype, rows=None, out=None):
    """out[r, :] = x[rows[r] or r, :] / sqrt(mean(x^2) + eps) * gain; x and gain float32."""
    _require_cuda(x, gain, rows)
    hidden = x.shape[-1]
    n = rows.numel() if rows is not None else x.shape[0]
    if x.dtype != torch.float32 or gain.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("rmsnorm: x and gain must be float32, x contiguous")
    _check_out(out, (n, hidden), out_dtype, "rmsnorm")
    if out is None:
        out = torch.empty((n, hidden), dtype=out_dtype, device=x.device)
    _call("elementwise", "llmb_rmsnorm", _ptr(x), _ptr(gain), _ptr(rows), _ptr(out),
          _c_int(_code(out_dtype)), _c_int(n), _c_int(hidden), _c_float(eps), _stream())
    return out


def swiglu(gate_up, out=None):
    """act[t, f] = silu(gate_up[t, f]) * gate_up[t, F + f]."""
    _require_cuda(gate_up)
    n, two_f = gate_up.shape
    width = two_f // 2
    if not gate_up.is_contiguous():
        raise KernelError("swiglu: the input must be contiguous")
    _check_out(out, (n, width), gate_up.dtype, "swiglu")
    if out is None:
        out = torch.empty((n, width), dtype=gate_up.dtype, device=gate_up.device)
    _call("elementwise", "llmb_swiglu", _ptr(gate_up), _ptr(out), _c_int(_code(gate_up.dtype)),
          _c_int(n), _c_int(width), _stream())
    return out


def rope_cache_write(qkv, rope_table, tok_pos, tok_seq, block_table, ring_pages, k_cache, v_cache,
                     n_heads, n_kv_heads, head_dim, interleaved=False, write_cache=True):
    """Rotate q (in place) and k of the fused [T, (Hq + 2 Hkv) D] projection by the
    angles of `rope_table` [positions, n_rot] (None: no rotation; n_rot <= D: only the
    first n_rot elements of a head are rotated) and store k and v of every token into the
    paged cache [pages, Hkv, 64, D]."""
    _require_cuda(qkv, rope_table, tok_pos, tok_seq, block_table, k_cache, v_cache)
    n = qkv.shape[0]
    if qkv.dim() != 2 or qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim or not qkv.is_contiguous():
        raise KernelError(f"rope_cache_write: qkv {tuple(qkv.shape)} is not contiguous "
                          f"[T, ({n_heads} + 2 * {n_kv_heads}) * {head_dim}]")
    n_rot = head_dim if rope_table is None else rope_table.shape[1]
    if rope_table is not None and (rope_table.dtype != torch.float32 or not rope_table.is_contiguous()
                                   or n_rot > head_dim or n_rot % 2):
        raise KernelError(f"rope_cache_write: the table of angles must be contiguous float32 "
                          f"[positions, n_rot] with an even n_rot <= {head_dim}")
    _call("elementwise", "llmb_rope_cache_write", _ptr(qkv), _c_int(_code(qkv.dtype)),
          _ptr(rope_table), _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table),
          _c_int(block_table.shape[1]), _c_int(ring_pages), _ptr(k_cache), _ptr(v_cache),
          _c_int(n), _c_int(n_heads), _c_int(n_kv_heads), _c_int(head_dim), _c_int(n_rot),
          _c_int(1 if interleaved else 0), _c_int(1 if write_cache else 0), _stream())


# ----------------------------------------------------------------------------- matrix product

_scratch: dict = {}
_retired: list = []      # outgrown scratch buffers, kept alive for CUDA graphs that hold their address


def _split_scratch(device, floats: int, counters: int):
    """Partial sums and tile counters of the split-K products, one pair per
    device, shared by every call on the stream (calls run one after the other).
    It grows when a call needs more; an outgrown pair is kept alive because a
    captured step may still hold its address."""
    held = _scratch.get(device)
    if held is None or held[0].numel() < floats or held[1].numel() < counters:
        n_floats = max(floats, held[0].numel() if held else 0, 1 << 23)
        n_counters = max(counters, held[1].numel() if held else 0, 1 << 14)
        global _scratch_generation
        if held is not None:
            _retired.append(held)
            _scratch_generation += 1
        held = (torch.empty(n_floats, dtype=torch.float32, device=device),
                torch.zeros(n_counters, dtype=torch.int32, device=device))
        _scratch[device] = held
    return held


def _skinny_scratch(device, m, n, k):
    lib = load_library("gemm_skinny")
    lib.llmb_gemm_skinny_scratch_bytes.restype = ctypes.c_longlong
    need = lib.llmb_gemm_skinny_scratch_bytes(_c_int(m), _c_int(n), _c_int(k))
    return _split_scratch(device, need // 4, (n + 15) // 16)


@functools.lru_cache(maxsize=4096)
def _tc_needs(m: int, n: int, k: int) -> tuple:
    """(floats of partial sums, tile counters, kernels launched) of a tcgen05 product of this shape."""
    lib = load_library("gemm_tc")
    lib.llmb_gemm_tc_scratch_floats.restype = ctypes.c_longlong
    return (lib.llmb_gemm_tc_scratch_floats(_c_int(m), _c_int(n), _c_int(k)),
            lib.llmb_gemm_tc_counters(_c_int(m), _c_int(n), _c_int(k)),
            lib.llmb_gemm_tc_kernels(_c_int(m), _c_int(n), _c_int(k)))


def _tc_scratch(device, m, n, k):
    floats, counters, _ = _tc_needs(m, n, k)
    return _split_scratch(device, floats, counters)


def tensor_core_status() -> int:
    """0, or the code of a bounded wait that ran out in a tcgen05 kernel since the
    last call (1 producer, 2 mma issuer, 3 epilogue). Call after a synchronisation."""
    return load_library("gemm_tc").llmb_gemm_tc_status()


def check_device_status() -> None:
    """Raise if a kernel of a loaded library reported a wait that ran out. Cheap (it
    reads a word of host memory); meaningful after the stream was synchronised."""
    from .build import _loaded
    for name in ("gemm_tc", "attention_prefill_tc"):
        if name in _loaded:
            code = getattr(_loaded[name], f"llmb_{name}_status")()
            if code != 0:
                raise KernelError(f"{name}: a bounded wait ran out (code {code}); the results of the "
                                  "last steps are not valid")


GLU_BLOCK = native.plan_constant("glu_block")    # gate and up rows alternate in blocks of this many rows (csrc/plan.h)


def glu_fusable(n_rows: int, k: int, dtype) -> bool:
    """Whether `linear(..., glu=True)` serves a gate/up matrix of n_rows = 2 F rows."""
    return dtype == torch.bfloat16 and n_rows % (2 * GLU_BLOCK) == 0 and k % 8 == 0


def _tc_kernels(m: int, n: int, k: int) -> int:
    """Kernels one call of the tcgen05 product launches (2 where the split-K sum is its own kernel)."""
    return _tc_needs(m, n, k)[2]


def _fusion_struct(norm, emit, rope):
    f = _Fusion()
    if norm is not None:
        f.norm_sumsq, f.norm_parts = norm.sumsq.data_ptr(), norm.parts
        f.norm_eps, f.norm_width = norm.eps, float(norm.width)
    if emit is not None:
        f.emit_rows, f.emit_sumsq = emit.rows.data_ptr(), emit.sumsq.data_ptr()
    if rope is not None:
        f.rope, f.interleaved, f.write_cache = 1, int(bool(rope.interleaved)), int(bool(rope.write_cache))
        f.n_heads, f.n_kv_heads, f.head_dim = rope.n_heads, rope.n_kv_heads, rope.head_dim
        f.rope_table = rope.table.data_ptr() if rope.table is not None else None
        f.tok_pos, f.tok_seq = rope.tok_pos.data_ptr(), rope.tok_seq.data_ptr()
        f.block_table, f.table_stride = rope.block_table.data_ptr(), rope.block_table.shape[1]
        f.ring_pages, f.k_cache, f.v_cache = rope.ring_pages, rope.k_cache.data_ptr(), rope.v_cache.data_ptr()
    return f


@functools.lru_cache(maxsize=4096)
def _tc_emit_parts(m: int, n: int, k: int) -> int:
    return load_library("gemm_tc").llmb_gemm_tc_emit_parts(_c_int(m), _c_int(n), _c_int(k))


def _check_norm(norm, m, k):
    if (norm.sumsq.dtype != torch.float32 or tuple(norm.sumsq.shape) != (m, SUMSQ_LD)
            or not norm.sumsq.is_contiguous() or not 1 <= norm.parts <= SUMSQ_LD):
        raise KernelError(f"linear: a folded norm needs sums of squares as contiguous float32 [{m}, {SUMSQ_LD}] "
                          f"with 1 to {SUMSQ_LD} parts in use")


def linear(a, w, bias=None, out_dtype=None, residual=None, out=None, glu=False, norm=None, emit=None,
           rope=None):
    """a [M, K] . w [N, K]^T (+ bias [N], float32). With `residual` (float32
    [M, N]) the product is added to it in place and it is returned; otherwise a
    new [M, N] tensor of `out_dtype` (default: a's dtype). With `glu`, w holds
    gate and up rows alternating in blocks of 16 and the result is
    silu(gate) * up as [M, N / 2] in a's dtype, computed in the product's epilogue.

    What can ride along (bfloat16; where the shape's kernel does not have it, a kernel of its
    own runs behind the product, with the same result):
    `norm` (FoldedNorm): a holds un-normalised rows, w has the norm's gain folded in, and the
    rows of the result are scaled by the norm's 1 / sqrt(mean square + eps) before the bias.
    `emit` (Emit, with `residual`): the updated residual rows as bfloat16 and the partial sums
    of their squares, for the next norm. `rope` (RopeWrite): the result is the q/k/v projection;
    queries and keys are rotated, queries stay in the result, keys and values go to the cache."""
    _require_cuda(a, w, bias, residual)
    (m, k), (n, k2) = a.shape, w.shape
    if norm is not None:
        _check_norm(norm, m, k)
    if emit is not None:
        if residual is None:
            raise KernelError("linear: emit needs a residual")
        emit.check(m, n)
    fused = norm is not None or emit is not None or rope is not None
    if glu:
        if not glu_fusable(n, k, a.dtype) or bias is not None or residual is not None or a.stride(0) % 8:
            raise KernelError("linear: the gated epilogue needs bfloat16, 2 F rows with F % 16 == 0, "
                              "K % 8 == 0, no bias and no residual")
        _check_out(out, (m, n // 2), a.dtype, "linear")
        result = out if out is not None else torch.empty((m, n // 2), dtype=a.dtype, device=a.device)
        partials, counters = _tc_scratch(a.device, m, n, k)
        if emit is not None or rope is not None:
            raise KernelError("linear: the gated epilogue takes a folded norm only")
        _call("gemm_tc", "llmb_gemm_tc_ex", _ptr(a), _c_int(a.stride(0)), _ptr(w), None, _ptr(result),
              _c_int(_code(a.dtype)), None, _ptr(partials), ctypes.c_longlong(partials.numel()),
              _ptr(counters), _c_int(counters.numel()), _c_int(m), _c_int(n), _c_int(k),
              _c_int(n // 2), _c_int(1), _c_int(0 if tactics.is_disabled("gemm_tc_pair") else 1),
              ctypes.byref(_fusion_struct(norm, None, None)) if norm is not None else None, None,
              _stream(), kernels=_tc_kernels(m, n, k))
        return result
    if k != k2 or a.dtype != w.dtype:
        raise KernelError(f"linear: a {tuple(a.shape)} {a.dtype} does not fit w {tuple(w.shape)} {w.dtype}")
    if a.stride(1) != 1 or not w.is_contiguous():
        raise KernelError("linear: operands must be row-major")
    if residual is not None:
        target_dtype, result = torch.float32, residual
        if residual.shape != (m, n) or residual.dtype != torch.float32 or not residual.is_contiguous():
            raise KernelError("linear: residual must be contiguous float32 [M, N]")
    else:
        target_dtype = out_dtype or a.dtype
        _check_out(out, (m, n), target_dtype, "linear")
        result = out if out is not None else torch.empty((m, n), dtype=target_dtype, device=a.device)
    variant = tactics.choose_linear(m, n, k, a.dtype, target_dtype, a.stride(0),
                                    a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)
    if fused and a.dtype != torch.bfloat16:
        raise KernelError("linear: norm, emit and rope ride only with bfloat16 products")
    if variant == "gemm_tc" and fused:
        partials, counters = _tc_scratch(a.device, m, n, k)
        applied = _c_int(0)
        _call("gemm_tc", "llmb_gemm_tc_ex", _ptr(a), _c_int(a.stride(0)), _ptr(w), _ptr(bias),
              _ptr(result if residual is None else None), _c_int(_code(target_dtype)),
              _ptr(residual), _ptr(partials), ctypes.c_longlong(partials.numel()),
              _ptr(counters), _c_int(counters.numel()), _c_int(m), _c_int(n), _c_int(k), _c_int(n),
              _c_int(0), _c_int(0 if tactics.is_disabled("gemm_tc_pair") else 1),
              ctypes.byref(_fusion_struct(norm, emit, rope)), ctypes.byref(applied), _stream(),
              kernels=_tc_kernels(m, n, k))
        if emit is not None:
            if applied.value & FUSED_EMIT:
                emit.parts = _tc_emit_parts(m, n, k)
            else:
                cast_sumsq(residual, emit)
        if rope is not None and not applied.value & FUSED_ROPE:
            rope_cache_write(result, rope.table, rope.tok_pos, rope.tok_seq, rope.block_table, rope.ring_pages,
                             rope.k_cache, rope.v_cache, rope.n_heads, rope.n_kv_heads, rope.head_dim,
                             rope.interleaved, rope.write_cache)
        return result
    if fused:
        # a variant without the fused epilogues: the plain product, then each part as its own kernel
        if norm is not None and residual is not None:
            raise KernelError("linear: a folded norm with a residual has no kernel")
        result = linear(a, w, None if norm is not None else bias, out_dtype, residual, out)
        if norm is not None:
            _call("elementwise", "llmb_scale_rows", _ptr(result), _c_int(_code(result.dtype)), _c_int(m), _c_int(n),
                  _ptr(norm.sumsq), _c_int(norm.parts), _c_float(norm.eps), _c_float(float(norm.width)),
                  _ptr(bias), _stream())
        if emit is not None:
            cast_sumsq(residual, emit)
        if rope is not None:
            rope_cache_write(result, rope.table, rope.tok_pos, rope.tok_seq, rope.block_table, rope.ring_pages,
                             rope.k_cache, rope.v_cache, rope.n_heads, rope.n_kv_heads, rope.head_dim,
                             rope.interleaved, rope.write_cache)
        return result
    if variant == "gemm_tc":
        partials, counters = _tc_scratch(a.device, m, n, k)
        _call("gemm_tc", "llmb_gemm_tc", _ptr(a), _c_int(a.stride(0)), _ptr(w), _ptr(bias),
              _ptr(result if residual is None else None), _c_int(_code(target_dtype)),
              _ptr(residual), _ptr(partials), ctypes.c_longlong(partials.numel()),
              _ptr(counters), _c_int(counters.numel()), _c_int(m), _c_int(n), _c_int(k), _c_int(n),
              _c_int(0), _c_int(0 if tactics.is_disabled("gemm_tc_pair") else 1), _stream(),
              kernels=_tc_kernels(m, n, k))
    elif variant == "gemm_skinny":
        partials, counters = _skinny_scratch(a.device, m, n, k)
        _call("gemm_skinny", "llmb_gemm_skinny", _ptr(a), _c_int(a.stride(0)), _ptr(w), _ptr(bias),
              _ptr(result if residual is None else None), _c_int(_code(target_dtype)),
              _ptr(residual), _ptr(partials), ctypes.c_longlong(partials.numel() * 4),
              _ptr(counters), _c_int(counters.numel()), _c_int(m), _c_int(n), _c_int(k), _c_int(n),
              _stream())
    elif variant == "gemm_simt":
        _call("gemm_simt", "llmb_gemm_simt", _ptr(a), _ptr(w), _ptr(bias),
              _ptr(result if residual is None else None), _ptr(residual),
              _c_int(_code(a.dtype)), _c_int(_code(target_dtype)), _c_int(m), _c_int(n), _c_int(k),
              _c_int(a.stride(0)), _c_int(n), _stream())
    else:
        raise KernelError(f"linear: no kernel named {variant}")
    return result


# ----------------------------------------------------------------------------- attention

_attention_scratch: dict = {}      # outgrown buffers join `_retired` above


def decode_splits(n_seqs: int, n_kv_heads: int, max_len: int) -> int:
    """Into how many slices the keys of every sequence are cut for decode
    attention. Blocks are (slice, kv head, sequence) and two fit on an SM: the
    count is the largest power of two that keeps all blocks in one wave of
    2 x 148 (measured on a B200 at 8,192 positions: batch 8 is fastest with 4
    slices = 256 blocks, batch 1 with 16 to 32), and never less than two pages
    a slice. When the batch alone exceeds a wave, slices still shorten the
    longest block of work (sequences of a batch differ in length, and the step
    ends with its longest slice): one slice per 16 pages of the longest
    sequence, at most four (batch 64 at equal lengths: 28 us with one slice
    against 39 us with four at 512 positions, 334 against 352 us with four at
    8,192; 16 sequences of 64 to 2,176 positions with 32 kv heads decode
    fastest with two). One slice writes the result itself and skips the
    combining kernel. The count depends on the
    length only through the power-of-two bucket of its page count, so that all
    steps replayed from one captured graph agree on it."""
    if os.environ.get("LLMB_DECODE_SPLITS"):             # for measurements: force a slice count
        return int(os.environ["LLMB_DECODE_SPLITS"])
    pages = max(1, (max_len + PAGE - 1) // PAGE)
    floor_pages = max(1, 1 << max(0, (pages - 1).bit_length() - 1))      # the bucket is (floor, 2 floor] pages
    pairs = max(1, n_seqs * n_kv_heads)
    want = 296 // pairs if pairs < 296 else min(4, max(1, floor_pages // 16))
    splits = 1
    while splits * 2 <= want and splits * 2 <= 32:
        splits *= 2
    while splits > 1 and splits > floor_pages // 2:
        splits //= 2
    return splits


def attention(qkv, k_cache, v_cache, block_table, ring_pages, tok_pos, tok_seq, n_heads,
              n_kv_heads, head_dim, scale, window=0, out=None, decode=False, seq_lens=None,
              max_len=0, cu_seqlens=None, max_new=0, seq_order=None):
    """Causal grouped-query attention of the new tokens' queries (the first
    Hq * D columns of `qkv`) over the paged cache, which already holds the new
    tokens' keys and values. Returns [T, Hq * D] in qkv's dtype. `seq_order`
    (optional, int32 [B]): the sequences by falling length; the kernels that
    take one block of work per sequence then start the longest first."""
    _require_cuda(qkv, k_cache, v_cache, block_table, tok_pos, tok_seq)
    n = qkv.shape[0]
    _check_out(out, (n, n_heads * head_dim), qkv.dtype, "attention")
    if out is None:
        out = torch.empty((n, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    variant = tactics.choose_attention(decode, qkv.dtype, n_heads, n_kv_heads, head_dim, window,
                                       cu_seqlens is not None and seq_lens is not None,
                                       qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0)
    if variant == "attention_prefill_tc":
        _call("attention_prefill_tc", "llmb_attention_prefill_tc", _ptr(qkv), _c_int(qkv.stride(0)),
              _c_int(n), _ptr(k_cache), _ptr(v_cache), _c_int(k_cache.shape[0]), _ptr(block_table),
              _c_int(block_table.shape[1]), _c_int(ring_pages), _ptr(cu_seqlens), _ptr(seq_lens),
              _ptr(seq_order), _ptr(out), _c_int(out.stride(0)), _c_int(cu_seqlens.numel() - 1),
              _c_int(max_new), _c_int(n_heads), _c_int(n_kv_heads), _c_int(head_dim), _c_float(scale),
              _c_int(window), _stream())
    elif variant == "attention_prefill":
        _call("attention_prefill", "llmb_attention_prefill", _ptr(qkv), _c_int(qkv.stride(0)),
              _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]),
              _c_int(ring_pages), _ptr(cu_seqlens), _ptr(seq_lens), _ptr(out), _c_int(out.stride(0)),
              _c_int(cu_seqlens.numel() - 1), _c_int(max_new), _c_int(n_heads), _c_int(n_kv_heads),
              _c_int(head_dim), _c_float(scale), _c_int(window), _stream())
    elif variant == "attention_decode":
        splits = decode_splits(n, n_kv_heads, max_len)
        lib = load_library("attention_decode")
        lib.llmb_attention_decode_scratch_floats.restype = ctypes.c_longlong
        need = lib.llmb_attention_decode_scratch_floats(_c_int(n), _c_int(n_heads), _c_int(head_dim),
                                                        _c_int(splits))
        scratch = _attention_scratch.get(qkv.device)
        if scratch is None or scratch.numel() < need:
            if scratch is not None:
                global _scratch_generation
                _retired.append(scratch)
                _scratch_generation += 1
            scratch = torch.empty(max(need, 1 << 23), dtype=torch.float32, device=qkv.device)
            _attention_scratch[qkv.device] = scratch
        _call("attention_decode", "llmb_attention_decode", _ptr(qkv), _c_int(qkv.stride(0)),
              _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]),
              _c_int(ring_pages), _ptr(seq_lens), _ptr(seq_order), _ptr(out), _c_int(out.stride(0)),
              _ptr(scratch),
              ctypes.c_longlong(scratch.numel()), _c_int(n), _c_int(n_heads), _c_int(n_kv_heads),
              _c_int(head_dim), _c_float(scale), _c_int(window), _c_int(splits), _stream(),
              kernels=2 if splits > 1 else 1)
    elif variant == "attention_generic":
        _call("attention_generic", "llmb_attention_generic", _ptr(qkv), _c_int(qkv.stride(0)),
              _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]),
              _c_int(ring_pages), _ptr(tok_pos), _ptr(tok_seq), _ptr(out), _c_int(out.stride(0)),
              _c_int(_code(qkv.dtype)), _c_int(n), _c_int(n_heads), _c_int(n_kv_heads),
              _c_int(head_dim), _c_float(scale), _c_int(window), _stream())
    else:
        raise KernelError(f"attention: no kernel named {variant}")
    return out


# ----------------------------------------------------------------------------- sampling

def argmax_rows(logits, out=None):
    """First maximum of every row of float32 logits [B, V] as int32 [B]."""
    _require_cuda(logits)
    n, vocab = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _call("sampling", "llmb_argmax_rows", _ptr(logits), _c_int(logits.stride(0)), _c_int(n),
          _c_int(vocab), _ptr(out), _stream())
    return out


def sample_rows(logits, params, iparams, recent, recent_len, rng_state, out, status, record=False,
                state_rows=None):
    """The whole sampling chain for every row; see csrc/sampling.cu. `logits`
    (float32 [B, V]) is changed where the repeat penalty applies. params float32 [B, 4],
    iparams int32 [B, 2], recent int32 [B, cap] or None, recent_len int32 [B], rng_state
    int64 [B], out int32 [B], status int32 [B]. With `record` the kernel also enters every
    drawn token into its row's window (recent, recent_len). `state_rows` (int32 [B], optional):
    row i of the logits belongs to the sequence whose parameters, window, generator and status
    are in row state_rows[i] of those arrays (which may then have more rows than the logits)."""
    _require_cuda(logits, params, iparams, recent, rng_state, out, status)
    n, vocab = logits.shape
    _call("sampling", "llmb_sample_rows", _ptr(logits), _c_int(logits.stride(0)), _c_int(n),
          _c_int(vocab), _ptr(params), _ptr(iparams), _ptr(recent), _ptr(recent_len),
          _c_int(recent.shape[1] if recent is not None else 0), _ptr(rng_state), _ptr(out),
          _ptr(status), _c_int(1 if record else 0), _ptr(state_rows), _stream())
    return out


def required_libraries() -> list:
    """Names of the kernel files the decoder parts of this package use."""
    return ["elementwise", "gemm_simt", "gemm_skinny", "gemm_tc", "attention_generic",
            "attention_decode", "attention_prefill", "attention_prefill_tc", "sampling"]


__all__ = ["PAGE", "GLU_BLOCK", "glu_fusable", "embed", "scale_", "random_normal_", "begin_recording", "end_recording", "RecordedPass", "scratch_generation", "Emit", "FoldedNorm", "RopeWrite", "cast_sumsq", "SUMSQ_LD", "rmsnorm", "swiglu", "rope_cache_write", "linear", "attention",
           "argmax_rows", "sample_rows", "launch_count", "count_launches", "tensor_core_status", "check_device_status", "ensure_built", "load_library", "all_sources",
           "required_libraries", "tactics"]
