"""The generation loop over batches of requests.

Per sequence the order is that of MythEclipse/llm's loop
(apps/engine/src/generate.rs:78-127): prefill; then sample from the current
logits; a stop token ends the sequence without being emitted or fed; else emit,
stop if the context is full, and feed the token for the next logits. Here a
batch of requests with unequal prompts starts together (one prefill step),
every live sequence then advances by one token per step, sequences that end
leave the batch (their slot goes back to the cache) and the rest go on; when
the batch is empty the next batch starts. Stop reasons and the timing fields
are those of generate.rs:20-49,129-160. Who is live, who goes on and who leaves
for which reason is decided by the native host library
(`csrc/host/generation.cpp`); this module owns slots, steps, sampling, timing
and callbacks.
"""
from __future__ import annotations

import time
from ctypes import byref, c_int, c_void_p
from dataclasses import dataclass, field

import torch

from .. import native
from ..errors import ContextFull, FormatError
from ..sampling import BatchSampler, SamplingParams
from .step import Entry


@dataclass
class GenerationRequest:
    prompt: list
    max_tokens: int = 256
    params: SamplingParams = field(default_factory=SamplingParams)
    stop_tokens: tuple = ()


@dataclass
class GenerationResult:
    tokens: list
    stop_reason: str                 # 'eos', 'max_tokens', 'cancelled', 'context_full'
    prompt_tokens: int
    generated_tokens: int = 0
    prefill_ms: float = 0.0
    ttft_ms: float = 0.0
    decode_ms: float = 0.0
    total_ms: float = 0.0
    tokens_per_second: float = 0.0


def plan_batches(requests, fits, max_batch: int) -> list:
    """Cut the requests, in their order, into batches: a batch takes requests
    while it has fewer than `max_batch` and `fits(list of final lengths)` says
    the cache can hold them all to their end. A request that does not fit even
    alone is an error."""
    batches, current, lengths = [], [], []
    for index, final_length in requests:
        if current and (len(current) >= max_batch or not fits(lengths + [final_length])):
            batches.append(current)
            current, lengths = [], []
        if not fits([final_length]):
            raise ContextFull(final_length, 0)
        current.append(index)
        lengths.append(final_length)
    if current:
        batches.append(current)
    return batches


def generate(engine, requests, max_batch: int | None = None, on_token=None, cancel=None) -> list:
    """Run every request to its end and return one GenerationResult each, in
    the order of the requests. `on_token(request index, token)` is called for
    every emitted token; `cancel()` returning True ends all live sequences with
    reason 'cancelled'."""
    requests = list(requests)
    context = engine.max_seq_len
    for i, r in enumerate(requests):
        if len(r.prompt) == 0:
            raise FormatError(f"request {i} has an empty prompt")
        if len(r.prompt) > context:
            raise ContextFull(len(r.prompt), context)
        r.params.check(engine.vocab)
    results = [None] * len(requests)
    final = [(i, min(len(r.prompt) + max(r.max_tokens, 0), context)) for i, r in enumerate(requests)]
    batches = plan_batches(final, engine.cache.can_hold, max_batch or engine.max_slots)
    for batch in batches:
        _run_batch(engine, requests, batch, results, on_token, cancel)
    return results


_REASONS = ("eos", "max_tokens", "cancelled", "context_full")       # codes of csrc/host/generation.cpp


class _Schedule:
    """The batch's decisions, kept by the native host library (`csrc/host/generation.cpp`):
    who is live, who goes on, who leaves and why."""

    def __init__(self, reqs, max_seq_len: int):
        n = len(reqs)
        self.n = n
        stops = [int(t) for r in reqs for t in r.stop_tokens]
        handle = c_void_p()
        native.check(native.lib().llmh_generation_create(
            n, native.ints(int(r.max_tokens) for r in reqs), native.ints(len(r.stop_tokens) for r in reqs),
            native.ints(stops), int(max_seq_len), byref(handle)))
        self._handle = handle
        self._a, self._b, self._c, self._d = ((c_int * max(n, 1))() for _ in range(4))

    def __del__(self):
        if getattr(self, "_handle", None):
            native.lib().llmh_generation_destroy(self._handle)
            self._handle = None

    def live(self) -> list:
        return list(self._a[:native.lib().llmh_generation_live(self._handle, self._a)])

    def drop_exhausted(self):
        """(rows of the live list that stay, sequences that leave with 'max_tokens')."""
        kept, done = c_int(), c_int()
        native.check(native.lib().llmh_generation_drop_exhausted(self._handle, self._a, byref(kept), self._b,
                                                                 byref(done)))
        return list(self._a[:kept.value]), list(self._b[:done.value])

    def plan_onward(self, lengths) -> list:
        count = c_int()
        native.check(native.lib().llmh_generation_plan_onward(self._handle, native.ints(lengths), self._a,
                                                              byref(count)))
        return list(self._a[:count.value])

    def take_tokens(self, tokens):
        """(emitted flag per live row, [(sequence, reason)] that leave, rows of the planned step that stay)."""
        done, going = c_int(), c_int()
        native.check(native.lib().llmh_generation_take_tokens(
            self._handle, native.ints(tokens), self._a, self._b, self._c, byref(done), self._d, byref(going)))
        finished = [(self._b[i], _REASONS[self._c[i]]) for i in range(done.value)]
        return list(self._a[:len(tokens)]), finished, list(self._d[:going.value])

    def cancel(self) -> list:
        done = c_int()
        native.check(native.lib().llmh_generation_cancel(self._handle, self._a, byref(done)))
        return list(self._a[:done.value])


def _run_batch(engine, requests, batch, results, on_token, cancel) -> None:
    started = time.perf_counter()
    slots = engine.acquire(len(batch))
    reqs = [requests[i] for i in batch]
    emitted = [[] for _ in batch]
    reason = ["max_tokens"] * len(batch)
    first_token_at = [None] * len(batch)
    sampler = BatchSampler([r.params for r in reqs], engine.vocab, engine.device)
    schedule = _Schedule(reqs, engine.max_seq_len)
    released = set()

    def finish(b, why):
        reason[b] = why
        if b not in released:
            engine.release([slots[b]])
            released.add(b)

    # ids travel device -> pinned host memory while the next step is already queued
    on_gpu = str(getattr(engine, "device", "cpu")).startswith("cuda")
    # (and behind them the sampler's refusal flags, read with every step's ids)
    staging = torch.empty(2 * len(batch), dtype=torch.int32, pin_memory=on_gpu)
    flags = staging[len(batch):]
    copied = torch.cuda.Event() if on_gpu else None

    try:
        live = schedule.live()
        logits = engine.step([Entry(slots[b], reqs[b].prompt, [len(reqs[b].prompt) - 1])
                              for b in live])
        prefill_done = None
        while live:
            if cancel is not None and cancel():
                for b in schedule.cancel():
                    finish(b, "cancelled")
                break
            # sequences that may not emit anything leave before sampling
            rows, exhausted = schedule.drop_exhausted()
            if exhausted:
                for b in exhausted:
                    finish(b, "max_tokens")
                logits = logits[rows] if rows else logits[:0]
                live = schedule.live()
                if not live:
                    break
            sampled = sampler.sample(logits, live)               # int32 on the device
            staging[:len(live)].copy_(sampled, non_blocking=True)
            if not sampler.all_greedy:
                flags.copy_(sampler.status, non_blocking=True)
            if copied is not None:
                copied.record()
            # Who goes on is known before the ids are: everyone whose limits allow one more
            # token. Their next step is queued now, fed with the ids on the device; a
            # sequence that turns out to have drawn a stop token simply drops that step.
            onward = schedule.plan_onward([engine.length(slots[b]) for b in live])
            next_logits = None
            if onward:
                feed = sampled if len(onward) == len(live) else sampled[
                    torch.tensor(onward, dtype=torch.long, device=sampled.device)]
                next_logits = engine.step([Entry(slots[live[k]], [0], [0]) for k in onward],
                                          device_tokens=feed)
            if copied is not None:
                copied.synchronize()                             # the ids, not the queued step
            tokens = staging[:len(live)].tolist()
            sampler.check_status(flags)
            engine.check()
            now = time.perf_counter()
            if prefill_done is None:
                prefill_done = now
            counts, finished, going_rows = schedule.take_tokens(tokens)
            for b, token, counted in zip(live, tokens, counts):
                if not counted:
                    continue
                emitted[b].append(token)
                if first_token_at[b] is None:
                    first_token_at[b] = now
                if on_token is not None:
                    on_token(batch[b], token)
            for b, why in finished:
                finish(b, why)
            live = schedule.live()
            if live:
                logits = next_logits if len(going_rows) == len(onward) else next_logits[going_rows]
    finally:
        for b in range(len(batch)):
            if b not in released:
                engine.release([slots[b]])
                released.add(b)
    ended = time.perf_counter()
    for b, index in enumerate(batch):
        n = len(emitted[b])
        first = first_token_at[b] if first_token_at[b] is not None else ended
        total_ms = (ended - started) * 1e3
        ttft_ms = (first - started) * 1e3
        decode_ms = max(total_ms - ttft_ms, 0.0)
        results[index] = GenerationResult(
            tokens=emitted[b], stop_reason=reason[b], prompt_tokens=len(reqs[b].prompt),
            generated_tokens=n, prefill_ms=((prefill_done or ended) - started) * 1e3,
            ttft_ms=ttft_ms, decode_ms=decode_ms, total_ms=total_ms,
            tokens_per_second=((n - 1) * 1e3 / decode_ms) if n > 1 and decode_ms > 0 else 0.0)
