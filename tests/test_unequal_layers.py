"""A model whose layers differ in size, with a partly rotated head and scale factors.

Defined here, outside the library: block 0 has the narrow attention and the wide feed-forward,
block 1 the wide attention (more heads, a bias) and the narrow feed-forward, so no block's
scratch plan contains the other's; the heads rotate only their first 16 of 32 elements (block 1
with interleaved pairs); the embedding is scaled by 3 and the logits by 0.5. Checked: the shared
scratch plan holds the largest request under every name and hands every block its own shape, a
buffer of the wrong shape is refused by the kernels' bindings, and the logits equal the plain
whole-sequence computation (CPU with the plain kernels, GPU in both dtypes)."""
import math
from dataclasses import dataclass

import pytest
import torch

import plain_llama as P
from tiny import random_tokens

HIDDEN, VOCAB, D, ROT = 64, 200, 32, 16
SHAPES = [dict(heads=2, kv=1, ffn=96, bias=False, pairing="half"),
          dict(heads=6, kv=2, ffn=48, bias=True, pairing="interleaved")]


def define():
    from llm_b200.config import register_architecture
    from llm_b200.parts.spec import (AttentionSpec, BlockSpec, GatedMlpSpec, ModelSpec, NormSpec,
                                     PositionSpec, ScheduleEntry, names)

    @dataclass(frozen=True)
    class TwoShapes:
        max_positions: int = 512

        @classmethod
        def from_dict(cls, raw, where="config.json"):
            return cls(int(raw.get("max_positions", 512)))

        def to_dict(self):
            return {"architectures": ["TwoShapes"], "max_positions": self.max_positions}

        def model_spec(self):
            blocks = []
            for i, s in enumerate(SHAPES):
                rope = PositionSpec(head_dim=D, theta=10000.0, max_positions=self.max_positions,
                                    pairing=s["pairing"], rotary_dim=ROT)
                p = f"l{i}."
                roles = {r: p + r for r in ("q", "k", "v", "o")}
                if s["bias"]:
                    roles.update({r + "_bias": p + r + "_bias" for r in ("q", "k", "v", "o")})
                mixer = AttentionSpec(hidden=HIDDEN, n_heads=s["heads"], n_kv_heads=s["kv"], head_dim=D,
                                      scale=1.0 / math.sqrt(D), bias=s["bias"], window=0, position=rope,
                                      names=names(**roles))
                ffn = GatedMlpSpec(hidden=HIDDEN, intermediate=s["ffn"], activation="silu",
                                   names=names(gate=p + "gate", up=p + "up", down=p + "down"))
                blocks.append(BlockSpec(NormSpec(HIDDEN, 1e-5, p + "n1"), mixer,
                                        NormSpec(HIDDEN, 1e-5, p + "n2"), ffn))
            return ModelSpec("TwoShapes", VOCAB, HIDDEN, self.max_positions, "embed", tuple(blocks),
                             (ScheduleEntry(0), ScheduleEntry(1)), NormSpec(HIDDEN, 1e-5, "norm"), "head",
                             embedding_scale=3.0, logit_scale=0.5)

    register_architecture("TwoShapes", TwoShapes)
    return TwoShapes


def plain_forward(w, tokens):
    n = len(tokens)
    positions = list(range(n))
    inv_freq = P.rope_inverse_frequencies(ROT, 10000.0)
    x = P.embedding(w["embed"], tokens) * 3.0
    for i, s in enumerate(SHAPES):
        p = f"l{i}."
        h = P.rms_norm(x, w[p + "n1"], 1e-5)
        q, k, v = (h @ w[p + r].T + (w[p + r + "_bias"] if s["bias"] else 0.0) for r in ("q", "k", "v"))
        q = P.rope_rotate(q.view(n, s["heads"], D), positions, inv_freq, s["pairing"])
        k = P.rope_rotate(k.view(n, s["kv"], D), positions, inv_freq, s["pairing"])
        a = P.causal_attention(q, k, v.view(n, s["kv"], D), 1.0 / math.sqrt(D))
        x = x + a.reshape(n, -1) @ w[p + "o"].T + (w[p + "o_bias"] if s["bias"] else 0.0)
        h = P.rms_norm(x, w[p + "n2"], 1e-5)
        x = x + P.gated_mlp(h, w[p + "gate"], w[p + "up"], w[p + "down"])
    return (P.rms_norm(x, w["norm"], 1e-5) @ w["head"].T) * 0.5


def make(tmp_path, dtype, device):
    from llm_b200.engine import Engine, load_model
    from llm_b200.weights import write_random_model
    config = define()()
    folder = write_random_model(tmp_path / "two_shapes", config, 3, dtype, std=0.08)
    _, weights = P.read_model_folder(folder)
    model = load_model(folder, dtype, device)
    return model, weights, Engine(model, max_tokens=1024, use_graphs=device != "cpu")


def run(engine, weights, tolerance):
    from llm_b200.engine import Entry
    seqs = [random_tokens(n, VOCAB, 40 + n) for n in (37, 5, 70)]
    slots = engine.acquire(len(seqs))
    logits = engine.step([Entry(s, t[:-4], list(range(len(t) - 4))) for s, t in zip(slots, seqs)])
    tail = []
    for k in range(4, 0, -1):
        tail.append(engine.step([Entry(s, [t[-k]], [0]) for s, t in zip(slots, seqs)]))
    at = 0
    for b, t in enumerate(seqs):
        want = plain_forward(weights, t)
        got = torch.cat([logits[at:at + len(t) - 4]] + [step[b:b + 1] for step in tail]).cpu()
        at += len(t) - 4
        scale = max(1.0, float(want.abs().max()))
        assert float((got - want).abs().max()) <= tolerance * scale
    engine.release(slots)
    engine.cache.check()


def test_the_plan_holds_the_largest_request_of_every_name(tmp_path, plain_kernels):
    model, weights, engine = make(tmp_path, torch.float32, "cpu")
    per_block = [{r.name: r for r in b.scratch_requests(10, torch.float32)} for b in model.blocks]
    assert per_block[0]["mixer.qkv"].nbytes < per_block[1]["mixer.qkv"].nbytes
    assert per_block[0]["ffn.act"].nbytes > per_block[1]["ffn.act"].nbytes
    merged = {r.name: r for r in model.scratch_requests(10)}
    for name in merged:
        assert merged[name].nbytes == max(p[name].nbytes for p in per_block if name in p)
    views = engine.workspace.for_tokens(10)
    views.plan.check()
    views.prefix = "mixer."
    narrow = views.get("qkv", (10, (2 + 2) * D), torch.float32)
    wide = views.get("qkv", (10, (6 + 4) * D), torch.float32)
    assert narrow.shape == (10, 4 * D) and wide.shape == (10, 10 * D)
    assert narrow.data_ptr() == wide.data_ptr() and narrow.is_contiguous()
    with pytest.raises(ValueError, match="planned with"):
        views.get("qkv", (10, 11 * D), torch.float32)
    run(engine, weights, 2e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unequal_layers_on_the_gpu(tmp_path, dtype):
    model, weights, engine = make(tmp_path, dtype, "cuda:0")
    run(engine, weights, 5e-5 if dtype == torch.float32 else 4e-2)


@pytest.mark.gpu
def test_an_out_buffer_of_the_wrong_shape_is_refused():
    from llm_b200 import ops
    from llm_b200.errors import KernelError
    a = torch.randn(8, 64, device="cuda:0", dtype=torch.bfloat16)
    w = torch.randn(96, 64, device="cuda:0", dtype=torch.bfloat16)
    good = torch.empty(8, 96, device="cuda:0", dtype=torch.bfloat16)
    ops.linear(a, w, out=good)
    for bad in (torch.empty(8, 128, device="cuda:0", dtype=torch.bfloat16),
                torch.empty(8, 96, device="cuda:0", dtype=torch.float32),
                torch.empty(8, 192, device="cuda:0", dtype=torch.bfloat16)[:, ::2]):
        with pytest.raises(KernelError, match="out is"):
            ops.linear(a, w, out=bad)
    x = torch.randn(8, 64, device="cuda:0")
    gain = torch.ones(64, device="cuda:0")
    with pytest.raises(KernelError, match="out is"):
        ops.rmsnorm(x, gain, 1e-5, torch.bfloat16, out=torch.empty(8, 32, device="cuda:0", dtype=torch.bfloat16))
    with pytest.raises(KernelError, match="out is"):
        ops.swiglu(good, out=torch.empty(8, 96, device="cuda:0", dtype=torch.bfloat16))
    with pytest.raises(KernelError, match="out is"):
        ops.embed(torch.zeros(8, dtype=torch.int32, device="cuda:0"), w,
                  out=torch.empty(8, 32, device="cuda:0"))
