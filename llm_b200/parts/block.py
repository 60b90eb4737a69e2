"""How a layer's parts are arranged."""
from __future__ import annotations

from .base import (Block, build_feed_forward, build_mixer, build_norm, register_block)


class PreNormBlock(Block):
    """x += mixer(norm(x)); x += feed_forward(norm(x)): the norm feeds the part,
    the residual keeps the un-normed stream (apps/engine/src/model.rs:835-864 of
    MythEclipse/llm)."""

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

    def prepare(self, max_positions, device):
        for p in self.parts:
            p.prepare(max_positions, device)

    def weights(self):
        return [w for p in self.parts for w in p.weights()]

    def kernel_shapes(self, dtype, token_counts):
        return [shape for p in self.parts for shape in p.kernel_shapes(dtype, token_counts)]

    def scratch_requests(self, n_tokens, dtype):
        """The normed inputs of both halves plus what the mixer and the feed-forward
        declare, their phases lined up one after the other."""
        from ..engine.workspace import BufferRequest
        hidden = self.spec.mixer_norm.size
        mixer = self.mixer.scratch_requests(n_tokens, dtype)
        ffn = self.feed_forward.scratch_requests(n_tokens, dtype)
        mixer_end = 1 + max([r.last_use for r in mixer] + [0])
        ffn_start = mixer_end + 2
        out = [BufferRequest("h_mixer", (n_tokens, hidden), dtype, 0, mixer_end)]
        out += [r.shifted(1, "mixer.") for r in mixer]
        ffn_end = ffn_start + max([r.last_use for r in ffn] + [0])
        out.append(BufferRequest("h_ffn", (n_tokens, hidden), dtype, mixer_end + 1, ffn_end))
        out += [r.shifted(ffn_start, "ffn.") for r in ffn]
        return out

    def forward(self, x, ctx, entry, cache_entry):
        views = ctx.workspace
        h = self.mixer_norm.forward(x, ctx.dtype, out=ctx.scratch("h_mixer", tuple(x.shape), ctx.dtype))
        if views is not None:
            views.prefix = "mixer."
        self.mixer.forward(h, ctx, entry, cache_entry, x)
        if views is not None:
            views.prefix = ""
        h = self.ffn_norm.forward(x, ctx.dtype, out=ctx.scratch("h_ffn", tuple(x.shape), ctx.dtype))
        if views is not None:
            views.prefix = "ffn."
        self.feed_forward.forward(h, ctx, x)
        if views is not None:
            views.prefix = ""


register_block("pre_norm", PreNormBlock)
