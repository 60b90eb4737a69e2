"""The decoder as a list of blocks run in the order of a schedule."""
from __future__ import annotations

import torch

from .. import ops
from ..errors import FormatError
from ..parts import build_block, build_norm
from ..parts.base import to_run_dtype
from ..weights.loader import ParamSpec, load_checkpoint
from .workspace import BufferRequest


class DecoderModel:
    """Embedding, blocks in schedule order, final norm and head, built from a
    ModelSpec. The layer loop and the head on the wanted rows only follow the
    forward pass of MythEclipse/llm (apps/engine/src/model.rs:755-825); which
    parts a layer has and in which order layers run is data of the spec."""

    def __init__(self, spec):
        self.spec = spec
        self.blocks = [build_block(b) for b in spec.blocks]
        self.final_norm = build_norm(spec.final_norm)
        for i, item in enumerate(spec.schedule):
            if not 0 <= item.layer < len(self.blocks):
                raise FormatError(f"schedule entry {i} names layer {item.layer} of {len(self.blocks)}")
            if item.cache_of is not None and not (
                    0 <= item.cache_of < i and spec.schedule[item.cache_of].cache_of is None):
                raise FormatError(f"schedule entry {i} reads the cache of entry {item.cache_of}, "
                                  "which is not an earlier entry with a cache of its own")
        self.embedding = None
        self.head = None
        self.dtype = None
        self.device = None

    # ------------------------------------------------------------------ weights

    def parameters(self) -> dict:
        out = {self.spec.embedding: ParamSpec((self.spec.vocab, self.spec.hidden))}
        for block in self.blocks:
            out.update(block.parameters())
        out.update(self.final_norm.parameters())
        if self.spec.head is not None:
            out[self.spec.head] = ParamSpec((self.spec.vocab, self.spec.hidden))
        return out

    def libraries(self) -> list:
        """The kernel files a run of this model in its dtype needs (what gets compiled)."""
        names = ["elementwise", "gemm_simt", "gemm_skinny", "gemm_tc"]
        for block in self.blocks:
            names += list(block.libraries)
        names += list(self.final_norm.libraries)
        names = list(dict.fromkeys(names))
        if self.dtype == torch.float32:                 # the 32-bit path runs on the CUDA cores only
            names = [n for n in names if n not in ops.BFLOAT16_ONLY]
        return names

    def kernel_shapes(self, dtype=None, token_counts=(1, 8, 2048)) -> list:
        """Every distinct kernel choice of a forward pass: (label, family, chooser arguments)."""
        dtype = dtype or self.dtype or torch.bfloat16
        seen, out = set(), []
        shapes = [s for block in self.blocks for s in block.kernel_shapes(dtype, token_counts)]
        for n in token_counts:
            shapes.append((f"head product, {min(n, 64)} rows", "linear",
                           dict(m=min(n, 64), n=self.spec.vocab, k=self.spec.hidden, in_dtype=dtype,
                                out_dtype=torch.float32, lda=self.spec.hidden, aligned=True)))
        for label, family, shape in shapes:
            key = (label, family, tuple(sorted((k, str(v)) for k, v in shape.items())))
            if key not in seen:
                seen.add(key)
                out.append((label, family, shape))
        return out

    def plan_identity(self, dtype=None) -> str:
        """Changes exactly when the choice of a kernel variant for this model changes."""
        from ..ops import tactics
        return tactics.plan_identity((family, shape) for _, family, shape in self.kernel_shapes(dtype))

    def replay_key(self, step, n_rows: int):
        """The key under which a pass may be run again from its record (Part.replay_key), or None
        if a part of the model does not allow it."""
        keys = []
        for block in self.blocks:
            key = block.replay_key(step)
            if key is None:
                return None
            keys.append(key)
        final = self.final_norm.replay_key(step)
        if final is None:
            return None
        return (step.n_tokens, step.n_seqs, n_rows, tuple(keys), final)

    def graph_safe(self) -> bool:
        return all(b.graph_safe for b in self.blocks) and self.final_norm.graph_safe

    def bind(self, tensors: dict, dtype, device) -> "DecoderModel":
        """Move the tensors to the device in the run's dtype; parts may fuse
        them. `tensors` may hold CPU or device tensors; entries are dropped as
        they are consumed so that a large model is not held twice."""
        self.dtype, self.device = dtype, torch.device(device)
        self.embedding = to_run_dtype(tensors[self.spec.embedding], dtype, device)
        self.head = (self.embedding if self.spec.head is None
                     else to_run_dtype(tensors[self.spec.head], dtype, device))
        for block in self.blocks:
            block.bind(tensors, dtype, device)
            for name in block.parameters():
                tensors.pop(name, None)
        self.final_norm.bind(tensors, dtype, device)
        return self

    def prepare(self, max_positions: int) -> None:
        for block in self.blocks:
            block.prepare(max_positions, self.device)

    def weight_bytes(self) -> int:
        """Bytes of every matrix a decode step reads once (the embedding table
        is read row by row and counted only as the head when tied)."""
        seen, total = set(), 0
        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        add(self.head)
        for item in self.spec.schedule:
            block = self.blocks[item.layer]
            for part in block.parts:
                for value in part.weights():
                    add(value)
        return total

    def scratch_requests(self, n_tokens: int) -> list:
        """Scratch of one layer pass for n_tokens tokens. Layers run one after the other and
        share one plan: per buffer name the largest request of any block (in bytes) with the
        union of the lifetimes, so that blocks whose sizes differ all fit. A block asks for
        its own shape (`ctx.scratch(name, shape, dtype)`) and gets a view of the front of the
        planned buffer."""
        merged, order = {}, []
        for block in self.blocks:
            for r in block.scratch_requests(n_tokens, self.dtype):
                held = merged.get(r.name)
                if held is None:
                    merged[r.name] = r
                    order.append(r.name)
                    continue
                larger = r if r.nbytes > held.nbytes else held
                merged[r.name] = BufferRequest(r.name, larger.shape, larger.dtype,
                                               min(r.first_use, held.first_use),
                                               max(r.last_use, held.last_use))
        return [merged[name] for name in order]

    # ------------------------------------------------------------------ cache needs

    def cache_requests(self):
        """Per schedule entry: the KvRequest of runs that own keys and values
        (None for runs that read another entry's), and the StateRequest."""
        kv, states = [], []
        for item in self.spec.schedule:
            mixer = self.blocks[item.layer].mixer
            kv.append(mixer.kv_request() if item.cache_of is None else None)
            states.append(mixer.state_request())
        return kv, states

    # ------------------------------------------------------------------ forward

    def forward(self, tokens, ctx, logit_rows):
        """tokens int32 [T] on the device; logit_rows int32 [R]: packed token
        indices whose logits are wanted. Returns float32 [R, vocab]."""
        # A block that folds its first norm into the product behind it (PreNormBlock in bfloat16)
        # reads that norm's input from where the last update of x left it: the embedding leaves it
        # for the first block, every block's last product for the block that runs next.
        schedule = self.spec.schedule
        n = tokens.numel()

        def wanted_by(position):
            if position >= len(schedule):
                return None
            block = self.blocks[schedule[position].layer]
            return block.input_emit(ctx, n, self.device) if getattr(block, "chains_norms", False) else None

        emit = wanted_by(0)
        x = ops.embed(tokens, self.embedding, scale=getattr(self.spec, "embedding_scale", 1.0), emit=emit)
        for entry, item in enumerate(schedule):
            cache_entry = entry if item.cache_of is None else item.cache_of
            block = self.blocks[item.layer]
            if getattr(block, "chains_norms", False):
                emit_next = wanted_by(entry + 1)
                block.forward(x, ctx, entry, cache_entry, normed=emit, emit_next=emit_next)
                emit = emit_next
            else:
                block.forward(x, ctx, entry, cache_entry)
                emit = None
        if logit_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab), dtype=torch.float32, device=x.device)
        z = self.final_norm.forward(x, ctx.dtype, rows=logit_rows)
        logits = ops.linear(z, self.head, out_dtype=torch.float32)
        if getattr(self.spec, "logit_scale", 1.0) != 1.0:
            ops.scale_(logits, self.spec.logit_scale)
        return logits


def declared_parameters(spec) -> dict:
    """Every tensor name a model of this spec binds, with shape and role."""
    return DecoderModel(spec).parameters()


def load_model(folder, dtype=torch.bfloat16, device="cuda:0") -> DecoderModel:
    """Read `folder`/config.json, pick the configuration class by its
    architecture name, check the checkpoint's tensors against what the model
    declares (one error for everything that is wrong) and bind them."""
    from ..config import load_config
    config = load_config(folder)
    model = DecoderModel(config.model_spec())
    model.config = config
    tensors = load_checkpoint(folder, model.parameters())
    return model.bind(tensors, dtype, device)


class _RandomTensors:
    """What `bind` reads its tensors from when there is no checkpoint: every declared tensor is
    made on the device at the moment a part asks for it, and nothing is kept, so a large
    model is never held twice."""

    def __init__(self, expected: dict, seed: int, std: float, gain_noise: float, device):
        self.expected, self.seed, self.std, self.gain_noise, self.device = expected, seed, std, gain_noise, device

    def __getitem__(self, name):
        from ..weights.random_init import random_tensors
        return random_tensors({name: self.expected[name]}, self.seed, torch.bfloat16, self.std,
                              self.gain_noise, self.device)[name]

    def __contains__(self, name):
        return name in self.expected

    def pop(self, name, default=None):
        return default


def random_model(config, seed: int, dtype=torch.bfloat16, device="cuda:0", std: float = 0.02,
                 gain_noise: float = 0.02) -> DecoderModel:
    """A model with random weights made on `device`, without a model folder: the same
    tensors, bit for bit, that `write_random_model(folder, config, seed)` writes (bfloat16
    storage) and `load_model` reads back, bound by the same `bind`."""
    model = DecoderModel(config.model_spec())
    model.config = config
    return model.bind(_RandomTensors(model.parameters(), seed, std, gain_noise, device), dtype, device)
