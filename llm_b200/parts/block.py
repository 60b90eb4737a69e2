"""How a layer's parts are arranged."""
from __future__ import annotations

import os

import torch

from .. import ops
from .base import (Block, build_feed_forward, build_mixer, build_norm, register_block)

# LLMB_NO_FUSION=1: every norm stays a kernel of its own (for comparisons)
FOLD_NORMS = os.environ.get("LLMB_NO_FUSION", "0") in ("", "0")


class PreNormBlock(Block):
    """x += mixer(norm(x)); x += feed_forward(norm(x)): the norm feeds the part,
    the residual keeps the un-normed stream (apps/engine/src/model.rs:835-864 of
    MythEclipse/llm).

    In bfloat16 runs a norm is folded into the part behind it where that part offers it
    (`Part.fold_input_norm`): the part's first product reads the bfloat16 copy of the residual
    rows and scales by the norm's factor in its epilogue, and the product that last updated
    the residual (the part before, the block before, or the embedding) has left that copy and
    the rows' sums of squares. MythEclipse/llm fuses its norm into the consumer's input in the
    same spirit (apps/engine/kernels/gpu.cu:351-407)."""

    #: `forward` takes `normed=` and `emit_next=` (see there)
    chains_norms = True

    def __init__(self, spec):
        self.spec = spec
        self.mixer_norm = build_norm(spec.mixer_norm)
        self.mixer = build_mixer(spec.mixer)
        self.ffn_norm = build_norm(spec.ffn_norm)
        self.feed_forward = build_feed_forward(spec.feed_forward)

    @property
    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts)

    @property
    def libraries(self):
        return tuple(lib for p in self.parts for lib in p.libraries)

    def parameters(self):
        out = {}
        for p in self.parts:
            out.update(p.parameters())
        return out

    def bind(self, tensors, dtype, device):
        for p in self.parts:
            p.bind(tensors, dtype, device)
        self.folded_mixer = self._fold(self.mixer_norm, self.mixer, dtype)
        self.folded_ffn = self._fold(self.ffn_norm, self.feed_forward, dtype)

    folded_mixer = folded_ffn = False

    @staticmethod
    def _fold(norm, part, dtype) -> bool:
        if not FOLD_NORMS or dtype != torch.bfloat16 or not getattr(norm, "foldable", False):
            return False
        return bool(part.fold_input_norm(norm.gain))

    def replay_key(self, step):
        keys = [p.replay_key(step) for p in self.parts]
        return None if any(k is None for k in keys) else tuple(keys)

    def input_emit(self, ctx, n_tokens: int, device):
        """Where the product that last updates the residual before this block leaves the folded
        mixer norm's input (None: the mixer norm is a kernel of its own)."""
        if not self.folded_mixer:
            return None
        return self._emit(ctx, "mixer", n_tokens, device)

    def _emit(self, ctx, which: str, n_tokens: int, device):
        hidden = self.spec.mixer_norm.size
        rows = ctx.scratch("h_" + which, (n_tokens, hidden), torch.bfloat16)
        sums = ctx.scratch("s_" + which, (n_tokens, ops.SUMSQ_LD), torch.float32)
        if rows is None or sums is None:
            rows = torch.empty((n_tokens, hidden), dtype=torch.bfloat16, device=device)
            sums = torch.empty((n_tokens, ops.SUMSQ_LD), dtype=torch.float32, device=device)
        return ops.Emit(rows, sums)

    def prepare(self, max_positions, device):
        for p in self.parts:
            p.prepare(max_positions, device)

    def weights(self):
        return [w for p in self.parts for w in p.weights()]

    def kernel_shapes(self, dtype, token_counts):
        return [shape for p in self.parts for shape in p.kernel_shapes(dtype, token_counts)]

    def scratch_requests(self, n_tokens, dtype):
        """The normed inputs of both halves plus what the mixer and the feed-forward
        declare, their phases lined up one after the other. A folded norm's input (bfloat16 rows
        and sums of squares) takes the normed input's place; the mixer's is written by the last
        product of the layer before, so it lives through the whole layer."""
        from ..engine.workspace import BufferRequest
        hidden = self.spec.mixer_norm.size
        mixer = self.mixer.scratch_requests(n_tokens, dtype)
        ffn = self.feed_forward.scratch_requests(n_tokens, dtype)
        mixer_end = 1 + max([r.last_use for r in mixer] + [0])
        ffn_start = mixer_end + 2
        ffn_end = ffn_start + max([r.last_use for r in ffn] + [0])
        sums = (n_tokens, ops.SUMSQ_LD)
        if self.folded_mixer:
            out = [BufferRequest("h_mixer", (n_tokens, hidden), torch.bfloat16, 0, ffn_end + 1),
                   BufferRequest("s_mixer", sums, torch.float32, 0, ffn_end + 1)]
        else:
            out = [BufferRequest("h_mixer", (n_tokens, hidden), dtype, 0, mixer_end)]
        out += [r.shifted(1, "mixer.") for r in mixer]
        if self.folded_ffn:
            out += [BufferRequest("h_ffn", (n_tokens, hidden), torch.bfloat16, 1, ffn_end),
                    BufferRequest("s_ffn", sums, torch.float32, 1, ffn_end)]
        else:
            out.append(BufferRequest("h_ffn", (n_tokens, hidden), dtype, mixer_end + 1, ffn_end))
        out += [r.shifted(ffn_start, "ffn.") for r in ffn]
        return out

    def forward(self, x, ctx, entry, cache_entry, normed=None, emit_next=None):
        """`normed` (an ops.Emit that was filled, or None): the folded mixer norm's input, left by
        the product that last updated x. `emit_next` (an ops.Emit, or None): where this block's
        last product leaves the same for the block that runs next."""
        views = ctx.workspace
        n = x.shape[0]

        def prefixed(prefix):
            if views is not None:
                views.prefix = prefix

        # ---- mixer
        if self.folded_mixer:
            if normed is None:
                normed = ops.cast_sumsq(x, self._emit(ctx, "mixer", n, x.device))
            h = ops.FoldedNorm(normed.rows, normed.sumsq, normed.parts, self.spec.mixer_norm.eps,
                               self.spec.mixer_norm.size)
        else:
            h = self.mixer_norm.forward(x, ctx.dtype, out=ctx.scratch("h_mixer", tuple(x.shape), ctx.dtype))
        emit_ffn = self._emit(ctx, "ffn", n, x.device) if self.folded_ffn else None
        prefixed("mixer.")
        if emit_ffn is not None and self.mixer.emits:
            self.mixer.forward(h, ctx, entry, cache_entry, x, emit=emit_ffn)
        else:
            self.mixer.forward(h, ctx, entry, cache_entry, x)
            if emit_ffn is not None:
                ops.cast_sumsq(x, emit_ffn)
        prefixed("")
        # ---- feed-forward
        if emit_ffn is not None:
            h = ops.FoldedNorm(emit_ffn.rows, emit_ffn.sumsq, emit_ffn.parts, self.spec.ffn_norm.eps,
                               self.spec.ffn_norm.size)
        else:
            h = self.ffn_norm.forward(x, ctx.dtype, out=ctx.scratch("h_ffn", tuple(x.shape), ctx.dtype))
        prefixed("ffn.")
        if emit_next is not None and self.feed_forward.emits:
            self.feed_forward.forward(h, ctx, x, emit=emit_next)
        else:
            self.feed_forward.forward(h, ctx, x)
            if emit_next is not None:
                prefixed("")
                ops.cast_sumsq(x, emit_next)
        prefixed("")


register_block("pre_norm", PreNormBlock)
