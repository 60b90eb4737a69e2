"""The step function: a batch of sequences, the tokens each brings, logits out.

MythEclipse/llm has two entry points for one sequence, `forward` for a chunk
and `forward_decode` for one token, over a shared body
(apps/engine/src/model.rs:652-730, 755-825). Here one `Engine.step` serves a
batch: every sequence brings its next tokens (all of its prompt in the first
step, one token in each later step), tokens are packed without padding,
positions come from each sequence's own length, and logits are returned for
the places the caller asks for. A step runs only the tokens it is given, on
top of what earlier steps left in the cache.
"""
from __future__ import annotations

import os
from array import array
from ctypes import byref, c_int, c_longlong
from dataclasses import dataclass
from itertools import chain

import torch

from .. import native, ops
from ..cache import PAGE, PagedCache, round_up
from ..errors import FormatError, LlmError
from ..parts.base import StepContext
from .workspace import Workspace


GRAPH_AFTER_STEPS = 2      # plain steps of a shape before it is captured
MAX_GRAPHS = 128           # captured shapes (batch size, bucket of pages) an engine keeps
RECORD_AFTER_PASSES = 1    # plain passes of a shape before the next one is recorded
MAX_RECORDS = 32           # recorded passes an engine keeps
MAX_RECORDED_LOGITS = 1 << 25   # a recorded pass holds its logits buffer: none for more values than this


@dataclass
class Entry:
    """One sequence's share of a step."""
    slot: int
    tokens: list                 # its next tokens (at least one)
    want: list                   # indices into `tokens` whose logits are wanted


@dataclass
class _HostStep:
    """The host-side fields of a StepContext, known before anything is on the device."""
    n_tokens: int
    n_seqs: int
    decode: bool
    new_counts: list
    starts: list
    max_len: int


class _Batch:
    """The entries of a step as the C arrays that the native host library reads."""

    def __init__(self, entries):
        try:
            self.tokens = array("i", chain.from_iterable(e.tokens for e in entries))
            self.wants = array("i", chain.from_iterable(e.want for e in entries))
        except (OverflowError, TypeError) as error:
            raise FormatError(f"token ids and wanted places must be 32-bit integers ({error})") from None
        self.n = len(entries)
        self.slots = native.ints(e.slot for e in entries)
        self.counts = native.ints(len(e.tokens) for e in entries)
        self.want_counts = native.ints(len(e.want) for e in entries)

    @staticmethod
    def _pointer(values):
        return (c_int * len(values)).from_buffer(values) if len(values) else None

    def arguments(self):
        return (self.n, self.slots, self.counts, self._pointer(self.tokens), self.want_counts,
                self._pointer(self.wants))


class Engine:
    """A bound model, its cache and the step function.

    max_tokens: tokens that all live sequences hold together, each rounded up
        to a multiple of 64 (sizes the page pools).
    max_seq_len: longest single sequence (default: the model's limit, capped
        by max_tokens).
    max_slots: most sequences alive at once (default: max_tokens / 64).
    step_tokens: most new tokens of one sequence in one pass over the layers;
        longer prompts are cut into passes (each attends to everything cached
        before it, as the chunks of apps/engine/src/session.rs:109-130 do).
    pass_tokens: most tokens of all sequences together in one pass (bounds the scratch
        arena); a larger step is run as several passes over subsets of its tokens.
    use_graphs: replay decode steps from CUDA graphs (only if every part of the
        model says it can be captured).
    """

    def __init__(self, model, max_tokens: int, max_seq_len: int | None = None,
                 max_slots: int | None = None, step_tokens: int | None = None,
                 use_graphs: bool = True, pass_tokens: int = 65536):
        if model.embedding is None:
            raise LlmError("the model has no weights bound")
        self.model = model
        self.dtype = model.dtype
        self.device = model.device
        max_tokens = round_up(max(int(max_tokens), PAGE))
        limit = model.spec.max_positions
        self.max_seq_len = min(max_seq_len or limit, limit, max_tokens)
        self.max_slots = max_slots or max(1, max_tokens // PAGE)
        self.step_tokens = step_tokens or self.max_seq_len
        self.pass_tokens = max(int(pass_tokens), 1)
        ops.ensure_built(model.libraries())
        # every product and attention shape of this model must have a kernel: a size that none
        # accepts (a head size above the kernels' limit) is refused here, not in the first step
        self.kernel_plan = model.plan_identity()
        model.prepare(self.max_seq_len)
        kv, states = model.cache_requests()
        self.cache = PagedCache(kv, states, max_tokens, self.max_seq_len, self.max_slots,
                                self.dtype, self.device, self.step_tokens)
        self.vocab = model.spec.vocab
        self.steps_run = 0
        self.workspace = Workspace(self.device, model.scratch_requests)
        self.use_graphs = (use_graphs and self.device.type == "cuda"
                           and os.environ.get("LLMB_NO_GRAPHS", "0") in ("", "0")
                           and not ops.PROFILING
                           and getattr(model, "graph_safe", lambda: False)())
        self._graphs, self._graph_seen, self._graph_pool = {}, {}, None
        self.graph_replays = 0            # decode steps run from a captured graph so far
        # passes that are not replayed from a graph (prompts, mixed steps, the first steps of a
        # decode shape) are recorded per shape and then walked by the native host library
        self.use_records = (self.device.type == "cuda" and not ops.PROFILING
                            and os.environ.get("LLMB_NO_RECORDS", "0") in ("", "0"))
        self._records, self._record_seen = {}, {}
        self.records_run = 0
        self._ring, self._ring_at = [(None, None)] * 4, 0

    # ------------------------------------------------------------------ sequences

    def acquire(self, count: int = 1) -> list:
        return [self.cache.acquire() for _ in range(count)]

    def release(self, slots) -> None:
        for slot in slots:
            self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def check(self) -> None:
        """After a synchronisation: raise if a kernel reported a failed wait."""
        ops.check_device_status()

    # ------------------------------------------------------------------ the step

    def step(self, entries, device_tokens=None) -> torch.Tensor:
        """Run the new tokens of every entry as one batch and return float32
        logits [wanted, vocab] on the device, in the order of the entries and of
        each entry's `want`. Everything is checked before anything is launched
        or changed: empty token lists, ids outside the vocabulary, wanted places
        outside the tokens, sequences that would outgrow the context, pages that
        are not there.

        `device_tokens` (int32 on the device, one id per entry) serves a decode
        step whose ids the host has not seen yet (they were just sampled on the
        device): every entry then brings one placeholder token, and the ids are
        taken from that tensor on the stream."""
        entries = [e if isinstance(e, Entry) else Entry(*e) for e in entries]
        for e in entries:
            e.tokens, e.want = list(e.tokens), list(e.want)
        if device_tokens is not None and (len(device_tokens) != len(entries)
                                          or any(len(e.tokens) != 1 for e in entries)):
            raise FormatError("device_tokens needs exactly one token per entry")
        if not entries:
            return torch.empty((0, self.vocab), dtype=torch.float32, device=self.device)
        # checked, and pages taken for the whole step (all or nothing), by the native host library
        batch = _Batch(entries)
        lib, cache = native.lib(), self.cache._handle
        native.check(lib.llmh_step_check(cache, *batch.arguments(), self.vocab, self.max_seq_len))
        native.check(lib.llmh_step_reserve(cache, batch.n, batch.slots, batch.counts))
        longest = max(len(e.tokens) for e in entries)
        total = sum(len(e.tokens) for e in entries)
        if longest <= self.step_tokens and total <= self.pass_tokens:
            return self._pass(entries, device_tokens, batch)
        # Cut the step into passes: at most step_tokens new tokens of a sequence and at most
        # pass_tokens tokens in all per pass. A sequence's pieces run in order (each attends
        # to what the earlier ones cached); sequences do not depend on each other, so any
        # grouping gives the same logits. The caller's order of wanted rows is restored.
        done = [0] * len(entries)
        pieces, order = [], []
        while any(done[i] < len(e.tokens) for i, e in enumerate(entries)):
            part, keys, members, budget = [], [], [], self.pass_tokens
            for i, e in enumerate(entries):
                start = done[i]
                take = min(len(e.tokens) - start, self.step_tokens, budget)
                if take <= 0:
                    continue
                want = [(j, w - start) for j, w in enumerate(e.want) if start <= w < start + take]
                part.append(Entry(e.slot, e.tokens[start:start + take], [w for _, w in want]))
                keys += [(i, j) for j, _ in want]
                members.append(i)
                done[i] += take
                budget -= take
            # ids that are still on the device (one per entry): each pass takes its entries' ids
            feed = None if device_tokens is None else device_tokens[
                torch.tensor(members, dtype=torch.long, device=device_tokens.device)]
            pieces.append(self._pass(part, feed))
            order += keys
        logits = torch.cat(pieces)
        wanted = sorted(range(len(order)), key=lambda r: order[r])
        return logits[torch.tensor(wanted, dtype=torch.long, device=self.device)]

    def _pass(self, entries, device_tokens=None, batch=None) -> torch.Tensor:
        batch = batch or _Batch(entries)
        lib, cache = native.lib(), self.cache._handle
        n_sections = lib.llmh_step_sections(cache)
        offsets, sizes = (c_longlong * n_sections)(), (c_longlong * n_sections)()
        total, summary = c_longlong(), (c_longlong * 5)()
        native.check(lib.llmh_step_layout(cache, batch.n, batch.counts, batch.want_counts, offsets, sizes, byref(total)))
        total = total.value
        host = self._host_buffer(total)
        native.check(lib.llmh_step_pack(cache, *batch.arguments(), host.data_ptr(), host.numel(),
                                        offsets, sizes, summary))
        offsets, sizes = list(offsets), list(sizes)
        n_tokens, decode, max_len = summary[0], bool(summary[2]), summary[3]
        counts = list(batch.counts)
        seq_lens = host[offsets[4]:offsets[4] + batch.n].tolist()
        starts = [after - c for after, c in zip(seq_lens, counts)]
        n_groups = n_sections - 8

        def context(dev):
            def view(i):
                return dev[offsets[i]:offsets[i] + sizes[i]]
            n_seqs = batch.n
            ctx = StepContext(
                n_tokens=n_tokens, n_seqs=n_seqs, dtype=self.dtype, device=self.device,
                tok_pos=view(1), tok_seq=view(2), cu_seqlens=view(3), seq_lens=view(4),
                slot_ids=view(5), seq_order=view(7), cache=self.cache,
                block_tables=[view(8 + g).view(n_seqs, -1) for g in range(n_groups)],
                decode=decode, new_counts=counts, starts=starts, max_len=max_len,
                workspace=self.workspace.for_tokens(n_tokens))
            return ctx, view(0), view(6)

        logits = None
        graphable = self.use_graphs and decode and all(e.want == [0] for e in entries)
        if graphable:
            logits = self._replay(len(entries), max_len, host, total, context, device_tokens)
        if logits is None and self.use_records and not graphable:
            step = _HostStep(n_tokens, batch.n, decode, counts, starts, max_len)
            key = self.model.replay_key(step, sizes[6])
            if key is not None and sizes[6] * self.vocab <= MAX_RECORDED_LOGITS:
                logits = self._run_recorded(key, batch.n, host, total, context, device_tokens)
        if logits is None:
            dev = host[:max(total, 4)].to(self.device, non_blocking=True)
            self._host_done(host)
            ctx, tokens_dev, rows_dev = context(dev)
            if device_tokens is not None:
                tokens_dev.copy_(device_tokens)
            logits = self.model.forward(tokens_dev, ctx, rows_dev)
        native.check(lib.llmh_step_commit(cache, batch.n, batch.slots, batch.counts))
        self.steps_run += 1
        return logits

    # ------------------------------------------------------------------ recorded passes

    def _run_recorded(self, key, n_seqs, host, total, context, device_tokens):
        """Run the pass from the record of an earlier pass with the same key (Part.replay_key), or
        record it while it runs (from the second pass of that key on), or return None (the first).
        A record is the list of the pass's launches with their arguments; the native host library
        makes them again in one call (ops.RecordedPass), where the layer loop of
        apps/engine/src/model.rs:755-825 runs natively as a whole. Every value that differs between
        two passes of one key (tokens, positions, lengths, slots, pages, wanted rows) lies in the
        record's own device buffer, which is refreshed before the launches."""
        from ..ops import tactics
        stamp = (ops.scratch_generation(), tactics.generation,
                 self.workspace.arena.data_ptr() if self.workspace.arena is not None else 0)
        held = self._records.get(key)
        if held is not None and held[3] != stamp:
            del self._records[key]
            held = None
        if held is None:
            seen = self._record_seen.get(key, 0) + 1
            self._record_seen[key] = seen
            if len(self._record_seen) > 4096:
                self._record_seen.clear()
            if seen <= RECORD_AFTER_PASSES:
                return None
            meta = torch.zeros(max(total, 4), dtype=torch.int32, device=self.device)
            meta[:total].copy_(host[:total], non_blocking=True)
            self._host_done(host)
            ctx, tokens_dev, rows_dev = context(meta)
            if device_tokens is not None:
                tokens_dev.copy_(device_tokens)
            recording = ops.begin_recording()
            try:
                logits = self.model.forward(tokens_dev, ctx, rows_dev)
            finally:
                ops.end_recording()
            # the arena may have grown while this pass was planned: the stamp is taken afterwards
            stamp = (ops.scratch_generation(), tactics.generation, self.workspace.arena.data_ptr())
            if len(self._records) >= MAX_RECORDS:
                self._records.pop(next(iter(self._records)))
            self._records[key] = (ops.RecordedPass(recording), meta, logits, stamp)
            return logits.clone()
        plan, meta, logits, _ = held
        meta[:total].copy_(host[:total], non_blocking=True)
        self._host_done(host)
        if device_tokens is not None:
            meta[:n_seqs].copy_(device_tokens)               # the tokens are the buffer's first section
        plan.run()
        self.records_run += 1
        return logits.clone()

    # ------------------------------------------------------------------ host staging

    def _host_buffer(self, n_ints: int) -> torch.Tensor:
        """A pinned staging buffer that no copy in flight still reads: a ring of
        four, each guarded by the event recorded after its last copy."""
        if self.device.type != "cuda":
            return torch.zeros(n_ints, dtype=torch.int32)
        self._ring_at = (self._ring_at + 1) % len(self._ring)
        buffer, event = self._ring[self._ring_at]
        if buffer is None or buffer.numel() < n_ints:
            buffer = torch.zeros(max(n_ints, 4096), dtype=torch.int32, pin_memory=True)
            event = torch.cuda.Event()
            self._ring[self._ring_at] = (buffer, event)
        else:
            event.synchronize()
        return buffer

    def _host_done(self, buffer) -> None:
        if self.device.type == "cuda":
            self._ring[self._ring_at][1].record()

    # ------------------------------------------------------------------ captured decode steps

    def _replay(self, n_seqs, max_len, host, total, context, device_tokens=None):
        """Decode steps of one shape (sequences, power-of-two bucket of pages)
        run from a CUDA graph once that shape has been seen GRAPH_AFTER_STEPS
        times, as the decode graphs of apps/engine/src/model.rs:699-729 are
        keyed by split count and captured after some plain steps. Every value
        that changes between steps (tokens, positions, lengths, pages) is read
        by the kernels from one device buffer that is refreshed before the
        replay."""
        pages = max(1, (max_len + PAGE - 1) // PAGE)
        key = (n_seqs, (pages - 1).bit_length())        # buckets (2^(k-1), 2^k] pages: a context of 2^k pages ends in its bucket
        graph = self._graphs.get(key)
        if graph is None:
            seen = self._graph_seen.get(key, 0) + 1
            self._graph_seen[key] = seen
            if seen <= GRAPH_AFTER_STEPS:
                return None
            meta = torch.zeros(total, dtype=torch.int32, device=self.device)
            meta.copy_(host[:total], non_blocking=True)
            ctx, tokens_dev, rows_dev = context(meta)
            if device_tokens is not None:
                tokens_dev.copy_(device_tokens)
            before = ops.launch_count()
            torch.cuda.synchronize(self.device)
            cuda_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cuda_graph, pool=self._graph_pool):
                out = self.model.forward(tokens_dev, ctx, rows_dev)
            if self._graph_pool is None:
                self._graph_pool = cuda_graph.pool()
            graph = (cuda_graph, meta, out, ops.launch_count() - before)
            ops.count_launches(-graph[3])            # capturing ran nothing
            if len(self._graphs) >= MAX_GRAPHS:      # the shape captured longest ago goes
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = graph
        cuda_graph, meta, out, kernels = graph
        meta.copy_(host[:total], non_blocking=True)
        self._host_done(host)
        if device_tokens is not None:
            meta[:n_seqs].copy_(device_tokens)           # the tokens are the buffer's first section
        cuda_graph.replay()
        self.graph_replays += 1
        ops.count_launches(kernels)
        return out.clone()
