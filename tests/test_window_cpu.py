"""A model whose layers differ in what they keep: one attention layer sees every
earlier key, one only a window of them. The cache gives each kind a group of its
own (the window group a ring of pages), long prompts are cut into passes, and the
result equals the plain implementation with the same windows. Host logic only
(kernels replaced by their plain statements); the GPU twin is in
test_toy_parts_gpu.py."""
from dataclasses import dataclass

import torch

import plain_llama as P
from tiny import random_tokens


def define_windowed():
    from llm_b200.config import ConfigReader, register_architecture
    from llm_b200.parts.spec import (AttentionSpec, BlockSpec, GatedMlpSpec, ModelSpec, NormSpec,
                                     PositionSpec, ScheduleEntry, names)

    @dataclass(frozen=True)
    class WindowedConfig:
        hidden: int
        vocab: int
        window: int

        @classmethod
        def from_dict(cls, raw, where="config.json"):
            r = ConfigReader(raw, where)
            return cls(r.integer("hidden"), r.integer("vocab"), r.integer("window"))

        def to_dict(self):
            return {"architectures": ["ToyWindowed"], "hidden": self.hidden, "vocab": self.vocab,
                    "window": self.window}

        def model_spec(self):
            h = self.hidden
            rope = PositionSpec(head_dim=16, theta=10000.0, max_positions=1024)
            blocks = []
            for i, window in enumerate((0, self.window, 0)):
                p = f"layers.{i}."
                mixer = AttentionSpec(hidden=h, n_heads=4, n_kv_heads=2, head_dim=16, scale=0.25,
                                      bias=False, window=window, position=rope,
                                      names=names(q=p + "q", k=p + "k", v=p + "v", o=p + "o"))
                ffn = GatedMlpSpec(hidden=h, intermediate=48, activation="silu",
                                   names=names(gate=p + "gate", up=p + "up", down=p + "down"))
                blocks.append(BlockSpec(NormSpec(h, 1e-5, p + "n1"), mixer, NormSpec(h, 1e-5, p + "n2"), ffn))
            return ModelSpec("ToyWindowed", self.vocab, h, 1024, "embed", tuple(blocks),
                             tuple(ScheduleEntry(i) for i in range(3)), NormSpec(h, 1e-5, "final_norm"),
                             None)

    register_architecture("ToyWindowed", WindowedConfig)
    return WindowedConfig


def plain_windowed(config, w, tokens):
    n = len(tokens)
    x = P.embedding(w["embed"], tokens)
    inv_freq = P.rope_inverse_frequencies(16, 10000.0)
    positions = list(range(n))
    for i, window in enumerate((0, config.window, 0)):
        p = f"layers.{i}."
        hn = P.rms_norm(x, w[p + "n1"], 1e-5)
        q = P.rope_rotate((hn @ w[p + "q"].T).view(n, 4, 16), positions, inv_freq)
        k = P.rope_rotate((hn @ w[p + "k"].T).view(n, 2, 16), positions, inv_freq)
        v = (hn @ w[p + "v"].T).view(n, 2, 16)
        x = x + P.causal_attention(q, k, v, 0.25, window=window).reshape(n, 64) @ w[p + "o"].T
        hn = P.rms_norm(x, w[p + "n2"], 1e-5)
        x = x + P.gated_mlp(hn, w[p + "gate"], w[p + "up"], w[p + "down"])
    return P.rms_norm(x, w["final_norm"], 1e-5) @ w["embed"].T


def run_windowed(tmp_path, device, dtype, tolerance):
    from llm_b200.engine import Engine, Entry, load_model
    from llm_b200.weights import write_random_model
    config = define_windowed()(hidden=64, vocab=200, window=70)
    folder = write_random_model(tmp_path / "windowed", config, seed=5, dtype=torch.bfloat16, std=0.08)
    _, weights = P.read_model_folder(folder)
    model = load_model(folder, dtype, device)
    # passes of at most 48 tokens: the window group is a ring of (70 + 48 - 2) // 64 + 2 = 3 pages
    engine = Engine(model, max_tokens=2048, max_seq_len=512, step_tokens=48)
    kinds = [(g.kind, g.window, g.ring_pages) for g in engine.cache.groups]
    assert kinds == [("full", 0, 8), ("window", 70, 3)]
    seqs = [random_tokens(n, 200, n) for n in (300, 75, 9)]
    expected = [plain_windowed(config, weights, s) for s in seqs]
    slots = engine.acquire(3)
    heads = [len(s) - 5 for s in seqs]
    logits = engine.step([Entry(sl, s[:n], [0, n - 1]) for sl, s, n in zip(slots, seqs, heads)])
    for b in range(3):
        for row, place in ((2 * b, 0), (2 * b + 1, heads[b] - 1)):
            want = expected[b][place]
            assert float((logits[row].float().cpu() - want).abs().max()) <= tolerance * max(1.0, float(want.abs().max()))
    for k in range(5):
        logits = engine.step([Entry(sl, [s[n + k]], [0]) for sl, s, n in zip(slots, seqs, heads)])
        for b in range(3):
            want = expected[b][heads[b] + k]
            assert float((logits[b].float().cpu() - want).abs().max()) <= tolerance * max(1.0, float(want.abs().max()))
    engine.release(slots)
    engine.cache.check()
    assert all(g.pool.n_held == 0 for g in engine.cache.groups)


def test_full_and_windowed_layers_in_one_model(tmp_path, plain_kernels):
    run_windowed(tmp_path, "cpu", torch.float32, 2e-4)
