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
from dataclasses import dataclass

import torch

from .. import ops
from ..cache import PAGE, PagedCache, round_up
from ..errors import ContextFull, FormatError, LlmError
from ..parts.base import StepContext
from .workspace import Workspace


GRAPH_AFTER_STEPS = 2      # plain steps of a shape before it is captured


@dataclass
class Entry:
    """One sequence's share of a step."""
    slot: int
    tokens: list                 # its next tokens (at least one)
    want: list                   # indices into `tokens` whose logits are wanted


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
        if device_tokens is not None and (len(device_tokens) != len(entries)
                                          or any(len(e.tokens) != 1 for e in entries)):
            raise FormatError("device_tokens needs exactly one token per entry")
        if not entries:
            return torch.empty((0, self.vocab), dtype=torch.float32, device=self.device)
        seen = set()
        for e in entries:
            if e.slot in seen:
                raise FormatError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if len(e.tokens) == 0:
                raise FormatError(f"slot {e.slot} brings no token")
            e.tokens = [int(t) for t in e.tokens]
            e.want = [int(w) for w in e.want]
            if min(e.tokens) < 0 or max(e.tokens) >= self.vocab:
                bad = next(t for t in e.tokens if not 0 <= t < self.vocab)
                raise FormatError(f"token id {bad} is outside the vocabulary of {self.vocab}")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise FormatError(f"wanted place {w} is outside the {len(e.tokens)} tokens "
                                      f"of slot {e.slot}")
            new_length = self.cache.length(e.slot) + len(e.tokens)
            if new_length > self.max_seq_len:
                raise ContextFull(new_length, self.max_seq_len)
        # pages for the whole step, all or nothing
        self.cache.reserve_many([(e.slot, self.cache.length(e.slot) + len(e.tokens))
                                 for e in entries])
        longest = max(len(e.tokens) for e in entries)
        total = sum(len(e.tokens) for e in entries)
        if longest <= self.step_tokens and total <= self.pass_tokens:
            return self._pass(entries, device_tokens)
        # Cut the step into passes: at most step_tokens new tokens of a sequence and at most
        # pass_tokens tokens in all per pass. A sequence's pieces run in order (each attends
        # to what the earlier ones cached); sequences do not depend on each other, so any
        # grouping gives the same logits. The caller's order of wanted rows is restored.
        done = [0] * len(entries)
        pieces, order = [], []
        while any(done[i] < len(e.tokens) for i, e in enumerate(entries)):
            part, keys, budget = [], [], self.pass_tokens
            for i, e in enumerate(entries):
                start = done[i]
                take = min(len(e.tokens) - start, self.step_tokens, budget)
                if take <= 0:
                    continue
                want = [(j, w - start) for j, w in enumerate(e.want) if start <= w < start + take]
                part.append(Entry(e.slot, e.tokens[start:start + take], [w for _, w in want]))
                keys += [(i, j) for j, _ in want]
                done[i] += take
                budget -= take
            pieces.append(self._pass(part))
            order += keys
        logits = torch.cat(pieces)
        wanted = sorted(range(len(order)), key=lambda r: order[r])
        return logits[torch.tensor(wanted, dtype=torch.long, device=self.device)]

    def _pass(self, entries, device_tokens=None) -> torch.Tensor:
        cache = self.cache
        tokens, tok_pos, tok_seq, cu, seq_lens, rows, starts, counts = [], [], [], [0], [], [], [], []
        for b, e in enumerate(entries):
            start = cache.length(e.slot)
            n = len(e.tokens)
            base = len(tokens)
            tokens += e.tokens
            tok_pos += range(start, start + n)
            tok_seq += [b] * n
            cu.append(base + n)
            seq_lens.append(start + n)
            rows += [base + w for w in e.want]
            starts.append(start)
            counts.append(n)
        slots = [e.slot for e in entries]
        sections = [tokens, tok_pos, tok_seq, cu, seq_lens, slots, rows]
        tables = [cache.block_table_rows(g, slots) for g in range(len(cache.groups))]
        offsets, total = [], 0
        for size in [len(s) for s in sections] + [t.numel() for t in tables]:
            offsets.append(total)
            total += (size + 3) // 4 * 4            # every section starts 16-byte aligned
        host = self._host_buffer(max(total, 4))
        flat = torch.tensor([v for s in sections for v in s], dtype=torch.int32)
        at = 0
        for s, offset in zip(sections, offsets):
            host[offset:offset + len(s)] = flat[at:at + len(s)]
            at += len(s)
        for t, offset in zip(tables, offsets[len(sections):]):
            host[offset:offset + t.numel()] = t.reshape(-1)
        sizes = [len(s) for s in sections] + [t.numel() for t in tables]
        decode = all(c == 1 for c in counts)
        max_len = max(seq_lens)

        def context(dev):
            def view(i):
                return dev[offsets[i]:offsets[i] + sizes[i]]
            n_seqs = len(slots)
            ctx = StepContext(
                n_tokens=len(tokens), n_seqs=n_seqs, dtype=self.dtype, device=self.device,
                tok_pos=view(1), tok_seq=view(2), cu_seqlens=view(3), seq_lens=view(4),
                slot_ids=view(5), cache=self.cache,
                block_tables=[view(7 + g).view(n_seqs, -1) for g in range(len(tables))],
                decode=decode, new_counts=counts, starts=starts, max_len=max_len,
                workspace=self.workspace.for_tokens(len(tokens)))
            return ctx, view(0), view(6)

        logits = None
        if self.use_graphs and decode and all(e.want == [0] for e in entries):
            logits = self._replay(len(entries), max_len, host, total, context, device_tokens)
        if logits is None:
            dev = host[:max(total, 4)].to(self.device, non_blocking=True)
            self._host_done(host)
            ctx, tokens_dev, rows_dev = context(dev)
            if device_tokens is not None:
                tokens_dev.copy_(device_tokens)
            logits = self.model.forward(tokens_dev, ctx, rows_dev)
        for e, new_length in zip(entries, seq_lens):
            cache.set_length(e.slot, new_length)
        self.steps_run += 1
        return logits

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
        key = (n_seqs, pages.bit_length())
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
            self._graphs[key] = graph
        cuda_graph, meta, out, kernels = graph
        meta.copy_(host[:total], non_blocking=True)
        self._host_done(host)
        if device_tokens is not None:
            meta[:n_seqs].copy_(device_tokens)           # the tokens are the buffer's first section
        cuda_graph.replay()
        ops.count_launches(kernels)
        return out.clone()
