"""Parts defined here, outside the library, can be registered, built and
stepped: a mixer that keeps state of its own (a decaying sum per sequence), in
one model with attention layers, a layer that runs twice, and a layer that
reads another layer's cache. No file of the library knows these."""
from dataclasses import dataclass

import pytest
import torch

from tiny import random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@dataclass(frozen=True)
class DecaySpec:
    hidden: int
    decay: float
    weight: str
    kind: str = "toy_decay"


def define_toy():
    from llm_b200.cache import StateRequest
    from llm_b200.config import ConfigReader, register_architecture
    from llm_b200.parts import Mixer, register_mixer
    from llm_b200.parts.spec import (AttentionSpec, BlockSpec, GatedMlpSpec, ModelSpec, NormSpec,
                                     PositionSpec, ScheduleEntry, names)
    from llm_b200.weights import ParamSpec

    class DecayMixer(Mixer):
        """state <- decay * state + h_t; output = (state) W^T, token after token."""

        def __init__(self, spec):
            self.spec = spec
            self.w = None

        def parameters(self):
            return {self.spec.weight: ParamSpec((self.spec.hidden, self.spec.hidden))}

        def bind(self, tensors, dtype, device):
            self.w = tensors[self.spec.weight].to(device=device, dtype=torch.float32)

        def state_request(self):
            return StateRequest((self.spec.hidden,), torch.float32)

        def forward(self, h, ctx, entry, cache_entry, residual):
            state = ctx.cache.state_view(entry)
            at = 0
            for b, n in enumerate(ctx.new_counts):
                slot = int(ctx.slot_ids[b])
                s = state[slot].clone()
                for t in range(at, at + n):
                    s = self.spec.decay * s + h[t].float()
                    residual[t] += s @ self.w.T
                state[slot] = s
                at += n

    register_mixer("toy_decay", DecayMixer)

    @dataclass(frozen=True)
    class ToyConfig:
        hidden: int
        vocab: int
        decay: float

        @classmethod
        def from_dict(cls, raw, where="config.json"):
            r = ConfigReader(raw, where)
            return cls(r.integer("hidden"), r.integer("vocab"), r.number("decay"))

        def to_dict(self):
            return {"architectures": ["ToyHybrid"], "hidden": self.hidden, "vocab": self.vocab,
                    "decay": self.decay}

        def model_spec(self):
            h = self.hidden
            rope = PositionSpec(head_dim=16, theta=10000.0, max_positions=512)
            def attention(i):
                p = f"layers.{i}.attn."
                return AttentionSpec(hidden=h, n_heads=4, n_kv_heads=2, head_dim=16, scale=0.25,
                                     bias=False, window=0, position=rope,
                                     names=names(q=p + "q", k=p + "k", v=p + "v", o=p + "o"))
            def mlp(i):
                p = f"layers.{i}.mlp."
                return GatedMlpSpec(hidden=h, intermediate=40, activation="silu",
                                    names=names(gate=p + "gate", up=p + "up", down=p + "down"))
            def block(i, mixer):
                return BlockSpec(NormSpec(h, 1e-5, f"layers.{i}.n1"), mixer,
                                 NormSpec(h, 1e-5, f"layers.{i}.n2"), mlp(i))
            blocks = (block(0, attention(0)), block(1, DecaySpec(h, self.decay, "layers.1.mix")),
                      block(2, attention(2)))
            # layer 0, the stateful layer, layer 0 again (a cache of its own), then
            # layer 2 reading the keys and values of the first run of layer 0
            schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0),
                        ScheduleEntry(2, cache_of=0))
            return ModelSpec("ToyHybrid", self.vocab, h, 512, "embed", blocks, schedule,
                             NormSpec(h, 1e-5, "final_norm"), None)

    register_architecture("ToyHybrid", ToyConfig)
    return ToyConfig


def plain_toy(config, w, tokens):
    """The toy model on whole sequences with the plain parts."""
    import plain_llama as P
    h, n = config.hidden, len(tokens)
    x = P.embedding(w["embed"], tokens)
    inv_freq = P.rope_inverse_frequencies(16, 10000.0)
    positions = list(range(n))
    first_kv = {}
    def attention(i, x, shared=None):
        p = f"layers.{i}.attn."
        hn = P.rms_norm(x, w[f"layers.{i}.n1"], 1e-5)
        q = P.rope_rotate((hn @ w[p + "q"].T).view(n, 4, 16), positions, inv_freq)
        if shared is None:
            k = P.rope_rotate((hn @ w[p + "k"].T).view(n, 2, 16), positions, inv_freq)
            v = (hn @ w[p + "v"].T).view(n, 2, 16)
        else:
            k, v = shared
        a = P.causal_attention(q, k, v, 0.25).reshape(n, 64)
        return x + a @ w[p + "o"].T, (k, v)
    def mlp(i, x):
        p = f"layers.{i}.mlp."
        hn = P.rms_norm(x, w[f"layers.{i}.n2"], 1e-5)
        return x + P.gated_mlp(hn, w[p + "gate"], w[p + "up"], w[p + "down"])
    x, kv0 = attention(0, x)
    x = mlp(0, x)
    hn = P.rms_norm(x, w["layers.1.n1"], 1e-5)
    s = torch.zeros(h)
    mixed = torch.zeros_like(x)
    for t in range(n):
        s = config.decay * s + hn[t]
        mixed[t] = s @ w["layers.1.mix"].T
    x = mlp(1, x + mixed)
    x, _ = attention(0, x)
    x = mlp(0, x)
    x, _ = attention(2, x, shared=kv0)
    x = mlp(2, x)
    return P.rms_norm(x, w["final_norm"], 1e-5) @ w["embed"].T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_model_with_state_steps_like_its_plain_form(tmp_path, dtype):
    import plain_llama
    from llm_b200.engine import Engine, Entry, load_model
    from llm_b200.weights import write_random_model
    ToyConfig = define_toy()
    config = ToyConfig(hidden=64, vocab=200, decay=0.5)
    folder = write_random_model(tmp_path / "toy", config, seed=3, dtype=torch.bfloat16, std=0.08)
    _, weights = plain_llama.read_model_folder(folder)
    model = load_model(folder, dtype, DEV)
    engine = Engine(model, max_tokens=1024)
    seqs = [random_tokens(n, 200, n) for n in (20, 5, 70)]
    expected = [plain_toy(config, weights, s) for s in seqs]
    for round_index in range(2):          # the second round reuses slots: state must restart at zero
        slots = engine.acquire(3)
        heads = [len(s) - 4 for s in seqs]
        logits = engine.step([Entry(sl, s[:n], [n - 1]) for sl, s, n in zip(slots, seqs, heads)])
        got = [[logits[b]] for b in range(3)]
        for k in range(4):
            logits = engine.step([Entry(sl, [s[n + k]], [0]) for sl, s, n in zip(slots, seqs, heads)])
            for b in range(3):
                got[b].append(logits[b])
        for b in range(3):
            g = torch.stack(got[b]).float().cpu()
            want = expected[b][heads[b] - 1:]
            scale = float(want.abs().max())
            limit = 2e-4 if dtype == torch.float32 else 0.04
            assert float((g - want).abs().max()) <= limit * max(scale, 1.0), (round_index, b)
        engine.release(slots)
        engine.cache.check()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_full_and_windowed_layers_in_one_model_on_the_gpu(tmp_path, dtype):
    """One layer sees every key, one a window of 70 kept in a ring of three pages, prompts
    cut into passes of 48: the kernels' window and ring addressing against the plain form."""
    from test_window_cpu import run_windowed
    run_windowed(tmp_path, DEV, dtype, 2e-4 if dtype == torch.float32 else 0.04)


# ----------------------------------------------------------------------------- routing, other positions

@dataclass(frozen=True)
class RoutedSpec:
    hidden: int
    intermediate: int
    n_experts: int
    prefix: str
    kind: str = "toy_routed"


@dataclass(frozen=True)
class InterpolatedSpec:
    """Rotary angles of position / stretch (positions squeezed into a shorter range)."""
    head_dim: int
    theta: float
    max_positions: int
    stretch: float
    kind: str = "toy_interpolated"


def define_routed_toy():
    from llm_b200 import ops
    from llm_b200.config import ConfigReader, register_architecture
    from llm_b200.parts import FeedForward, PositionEncoding, register_feed_forward, register_position
    from llm_b200.parts.spec import (AttentionSpec, BlockSpec, ModelSpec, NormSpec, PositionSpec,
                                     ScheduleEntry, names)
    from llm_b200.weights import ParamSpec

    class RoutedMlp(FeedForward):
        """Every token goes to the one expert with the largest router logit (logits in 32-bit,
        first maximum wins); each expert is a gated MLP run with the library's products on the
        rows that chose it."""

        def __init__(self, spec):
            self.spec = spec

        def parameters(self):
            s, out = self.spec, {}
            out[s.prefix + "router"] = ParamSpec((s.n_experts, s.hidden))
            for e in range(s.n_experts):
                out[f"{s.prefix}{e}.gate"] = ParamSpec((s.intermediate, s.hidden))
                out[f"{s.prefix}{e}.up"] = ParamSpec((s.intermediate, s.hidden))
                out[f"{s.prefix}{e}.down"] = ParamSpec((s.hidden, s.intermediate))
            return out

        def bind(self, tensors, dtype, device):
            s = self.spec
            self.router = tensors[s.prefix + "router"].to(device=device, dtype=torch.float32)
            self.experts = [tuple(tensors[f"{s.prefix}{e}.{r}"].to(device=device, dtype=dtype).contiguous()
                                  for r in ("gate", "up", "down")) for e in range(s.n_experts)]

        def forward(self, h, ctx, residual):
            logits = h.float() @ self.router.T                      # 32-bit, whatever the run dtype
            choice = logits.argmax(dim=1)
            for e, (gate, up, down) in enumerate(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                x = h[rows].contiguous()
                act = ops.swiglu(torch.cat([ops.linear(x, gate), ops.linear(x, up)], dim=1))
                update = torch.zeros((rows.numel(), self.spec.hidden), dtype=torch.float32, device=h.device)
                ops.linear(act, down, residual=update)
                residual[rows] += update

    register_feed_forward("toy_routed", RoutedMlp)

    class InterpolatedRope(PositionEncoding):
        interleaved = True

        def __init__(self, spec):
            self.spec = spec
            self.table = None

        def prepare(self, max_positions, device):
            s = self.spec
            n = min(max_positions, s.max_positions)
            inv = torch.pow(torch.tensor(s.theta, dtype=torch.float64),
                            -2.0 * torch.arange(s.head_dim // 2, dtype=torch.float64) / s.head_dim)
            angle = (torch.arange(n, dtype=torch.float64) / s.stretch)[:, None] * inv[None, :]
            self.table = torch.cat([angle.cos(), angle.sin()], 1).float().to(device).contiguous()

    register_position("toy_interpolated", InterpolatedRope)

    @dataclass(frozen=True)
    class RoutedConfig:
        hidden: int
        vocab: int
        experts: int
        stretch: float

        @classmethod
        def from_dict(cls, raw, where="config.json"):
            r = ConfigReader(raw, where)
            return cls(r.integer("hidden"), r.integer("vocab"), r.integer("experts"), r.number("stretch"))

        def to_dict(self):
            return {"architectures": ["ToyRouted"], "hidden": self.hidden, "vocab": self.vocab,
                    "experts": self.experts, "stretch": self.stretch}

        def model_spec(self):
            h = self.hidden
            positions = (InterpolatedSpec(16, 10000.0, 512, self.stretch), None)   # layer 1: no encoding
            def block(i):
                p = f"layers.{i}."
                attention = AttentionSpec(hidden=h, n_heads=3, n_kv_heads=1, head_dim=16, scale=0.25,
                                          bias=False, window=0, position=positions[i],
                                          names=names(q=p + "q", k=p + "k", v=p + "v", o=p + "o"))
                return BlockSpec(NormSpec(h, 1e-6, p + "n1"), attention, NormSpec(h, 1e-6, p + "n2"),
                                 RoutedSpec(h, 24, self.experts, p + "experts."))
            blocks = (block(0), block(1))
            return ModelSpec("ToyRouted", self.vocab, h, 512, "embed", blocks,
                             (ScheduleEntry(0), ScheduleEntry(1)), NormSpec(h, 1e-6, "final_norm"), "head")

    register_architecture("ToyRouted", RoutedConfig)
    return RoutedConfig


def plain_routed(config, w, tokens):
    import plain_llama as P
    n = len(tokens)
    x = P.embedding(w["embed"], tokens)
    inv_freq = P.rope_inverse_frequencies(16, 10000.0)
    squeezed = [p / config.stretch for p in range(n)]
    choices = []
    for i in range(2):
        p = f"layers.{i}."
        hn = P.rms_norm(x, w[p + "n1"], 1e-6)
        q, k = (hn @ w[p + "q"].T).view(n, 3, 16), (hn @ w[p + "k"].T).view(n, 1, 16)
        if i == 0:
            q = P.rope_rotate(q, squeezed, inv_freq, "interleaved")
            k = P.rope_rotate(k, squeezed, inv_freq, "interleaved")
        v = (hn @ w[p + "v"].T).view(n, 1, 16)
        x = x + P.causal_attention(q, k, v, 0.25).reshape(n, 48) @ w[p + "o"].T
        hn = P.rms_norm(x, w[p + "n2"], 1e-6)
        choice = (hn @ w[p + "experts.router"].T).argmax(dim=1)
        update = torch.zeros_like(x)
        for t in range(n):
            e = int(choice[t])
            update[t] = P.gated_mlp(hn[t:t + 1], w[f"{p}experts.{e}.gate"], w[f"{p}experts.{e}.up"],
                                    w[f"{p}experts.{e}.down"])[0]
        x = x + update
        choices.append(choice)
    return P.rms_norm(x, w["final_norm"], 1e-6) @ w["head"].T, choices


def test_routed_feed_forward_and_other_position_encodings(tmp_path):
    """A feed-forward that routes every token to one of three experts, a rotary encoding with
    squeezed positions, and a layer without any position encoding: registered from here, built by
    the library's loader and stepped (prompts, then token by token) in 32-bit against their plain
    form. Every expert must have been chosen, or the test would not test routing."""
    import plain_llama
    from llm_b200.engine import Engine, Entry, load_model
    from llm_b200.weights import write_random_model
    RoutedConfig = define_routed_toy()
    config = RoutedConfig(hidden=48, vocab=150, experts=3, stretch=4.0)
    folder = write_random_model(tmp_path / "routed", config, seed=5, dtype=torch.float32, std=0.3)
    _, weights = plain_llama.read_model_folder(folder)
    model = load_model(folder, torch.float32, DEV)
    engine = Engine(model, max_tokens=512)
    seqs = [random_tokens(n, 150, 40 + n) for n in (33, 6)]
    slots = engine.acquire(2)
    heads = [len(s) - 3 for s in seqs]
    logits = engine.step([Entry(sl, s[:n], list(range(n))) for sl, s, n in zip(slots, seqs, heads)])
    got = [[logits[:heads[0]]], [logits[heads[0]:]]]
    for k in range(3):
        step = engine.step([Entry(sl, [s[n + k]], [0]) for sl, s, n in zip(slots, seqs, heads)])
        for b in range(2):
            got[b].append(step[b:b + 1])
    seen = set()
    for b in range(2):
        want, choices = plain_routed(config, weights, seqs[b])
        for choice in choices:
            seen |= set(choice.tolist())
        g = torch.cat(got[b]).cpu()
        assert float((g - want).abs().max()) <= 2e-4 * max(float(want.abs().max()), 1.0), b
    assert seen == {0, 1, 2}
    engine.release(slots)
