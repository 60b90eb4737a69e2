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

    def forward(self, x, ctx, entry, cache_entry):
        h = self.mixer_norm.forward(x, ctx.dtype)
        self.mixer.forward(h, ctx, entry, cache_entry, x)
        h = self.ffn_norm.forward(x, ctx.dtype)
        self.feed_forward.forward(h, ctx, x)


register_block("pre_norm", PreNormBlock)
