"""Plain, slow Llama decoder used as the oracle of every test.

Whole sequences only: no cache, no batching, no kernels. One function per
part, each citing the lines of MythEclipse/llm (paths inside that project)
whose formula it restates. It shares no code with the ``llm_b200`` package:
it reads ``config.json`` and ``model.safetensors`` with its own few lines.

MythEclipse/llm's model code is Rust and cannot be compiled in this
environment, so this file rests on the formulas of its sources, not on a
run of that code. Two points are restated for safetensors checkpoints,
which the project (a GGUF engine) does not read: the rotation pairs
``(p, p + D/2)`` instead of ``(2p, 2p+1)`` (GGUF files store the q/k rows
permuted for the latter, ``README.md:912-914``), and the llama3 frequency
scaling, attention bias and tied head are config.json options it has no
counterpart for.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
           "I32": torch.int32, "I64": torch.int64, "F64": torch.float64}


def read_model_folder(folder, dtype=torch.float32):
    """config.json as a dict and every tensor of model.safetensors widened to `dtype`."""
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    blob = (folder / "model.safetensors").read_bytes()
    (header_len,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + header_len])
    tensors = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        begin, end = entry["data_offsets"]
        raw = bytearray(blob[8 + header_len + begin:8 + header_len + end])
        tensor = torch.frombuffer(raw, dtype=_DTYPES[entry["dtype"]]).reshape(entry["shape"])
        tensors[name] = tensor.to(dtype) if tensor.is_floating_point() else tensor.clone()
    return config, tensors


# --------------------------------------------------------------------------- parts

def embedding(table, tokens):
    """x[t, :] = table[token_t, :] (apps/engine/src/model.rs:741-751)."""
    return table[torch.as_tensor(tokens, dtype=torch.long)]


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight, eps inside the root, plain weight
    (apps/engine/src/ops.rs:4-12; scale in ops.rs:24-30)."""
    mean_square = (x * x).mean(dim=-1, keepdim=True)
    return x * (1.0 / torch.sqrt(mean_square + eps)) * weight


def rope_inverse_frequencies(head_dim, theta, scaling=None):
    """theta^(-2p/D) for pair p (apps/engine/src/ops.rs:128-131), then the
    llama3 rescaling of config.json's rope_scaling (no counterpart in
    MythEclipse/llm, which applies no frequency scaling:
    docs/superpowers/specs/2026-11-04-llm-local-inference-design.md:22)."""
    pairs = torch.arange(0, head_dim // 2, dtype=torch.float64)
    freq = theta ** (-2.0 * pairs / head_dim)
    if scaling is None:
        return freq
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind == "default":
        return freq
    assert kind == "llama3", kind
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    original = float(scaling["original_max_position_embeddings"])
    out = freq.clone()
    for p in range(freq.numel()):
        wavelength = 2.0 * math.pi / freq[p].item()
        if wavelength < original / high:
            continue
        if wavelength > original / low:
            out[p] = freq[p] / factor
        else:
            smooth = (original / wavelength - low) / (high - low)
            out[p] = (1.0 - smooth) * freq[p] / factor + smooth * freq[p]
    return out


def rope_rotate(x, positions, inv_freq, pairing="half"):
    """Rotate every head of x [n, heads, D] by angle position * inv_freq[p]
    (apps/engine/src/ops.rs:152-165). pairing 'interleaved' is the
    project's (2p, 2p+1); 'half' pairs (p, p + n_rot/2). n_rot = 2 * len(inv_freq) may be
    smaller than D: the elements beyond it pass through (the rope dimension count,
    apps/engine/src/model.rs:93-95)."""
    n_rot = 2 * len(inv_freq)
    angle = torch.as_tensor(positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
    cos = angle.cos().to(x.dtype)[:, None, :]
    sin = angle.sin().to(x.dtype)[:, None, :]
    if pairing == "interleaved":
        low, high = x[..., 0:n_rot:2], x[..., 1:n_rot:2]
    else:
        low, high = x[..., : n_rot // 2], x[..., n_rot // 2:n_rot]
    new_low = low * cos - high * sin
    new_high = low * sin + high * cos
    out = x.clone()
    if pairing == "interleaved":
        out[..., 0:n_rot:2], out[..., 1:n_rot:2] = new_low, new_high
    else:
        out[..., : n_rot // 2], out[..., n_rot // 2:n_rot] = new_low, new_high
    return out


def softmax(scores):
    """exp(s - max) / sum (apps/engine/src/ops.rs:95-106)."""
    shifted = scores - scores.max(dim=-1, keepdim=True).values
    e = shifted.exp()
    return e / e.sum(dim=-1, keepdim=True)


def causal_attention(q, k, v, scale, window=0):
    """One sequence from its first token: q [n, Hq, D], k, v [n, Hkv, D].
    Query t sees keys j <= t; head h reads kv head h // (Hq/Hkv)
    (apps/engine/src/compute.rs:1075-1126). With window > 0 only the last
    `window` keys (j > t - window) are seen."""
    n, n_heads, dim = q.shape
    group = n_heads // k.shape[1]
    out = torch.zeros_like(q)
    for head in range(n_heads):
        kv_head = head // group
        for t in range(n):
            first = 0 if window <= 0 else max(0, t - window + 1)
            keys = k[first:t + 1, kv_head]
            scores = (keys @ q[t, head]) * scale
            out[t, head] = softmax(scores) @ v[first:t + 1, kv_head]
    return out


def silu(z):
    """z / (1 + exp(-z)) (apps/engine/src/ops.rs:33-35)."""
    return z / (1.0 + torch.exp(-z))


def gated_mlp(h, gate, up, down):
    """down(silu(gate h) * (up h)) (apps/engine/src/model.rs:1180-1216)."""
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def attention_part(h, positions, w, prefix, config, inv_freq):
    """q/k/v projections, rotation, attention, output projection
    (apps/engine/src/model.rs:930-1040)."""
    heads = config["num_attention_heads"]
    kv_heads = config.get("num_key_value_heads", heads)
    dim = config.get("head_dim") or config["hidden_size"] // heads
    q = h @ w[prefix + "q_proj.weight"].T
    k = h @ w[prefix + "k_proj.weight"].T
    v = h @ w[prefix + "v_proj.weight"].T
    if config.get("attention_bias", False):
        q = q + w[prefix + "q_proj.bias"]
        k = k + w[prefix + "k_proj.bias"]
        v = v + w[prefix + "v_proj.bias"]
    n = h.shape[0]
    q = rope_rotate(q.view(n, heads, dim), positions, inv_freq)
    k = rope_rotate(k.view(n, kv_heads, dim), positions, inv_freq)
    a = causal_attention(q, k, v.view(n, kv_heads, dim), 1.0 / math.sqrt(dim))
    out = a.reshape(n, heads * dim) @ w[prefix + "o_proj.weight"].T
    if config.get("attention_bias", False):
        out = out + w[prefix + "o_proj.bias"]
    return out


def forward(config, w, tokens):
    """Logits [n, vocab] at every position of one whole sequence
    (layer loop apps/engine/src/model.rs:787-803, head model.rs:806-822)."""
    heads = config["num_attention_heads"]
    dim = config.get("head_dim") or config["hidden_size"] // heads
    eps = config.get("rms_norm_eps", 1e-6)
    inv_freq = rope_inverse_frequencies(dim, config.get("rope_theta", 10000.0),
                                        config.get("rope_scaling"))
    positions = list(range(len(tokens)))
    x = embedding(w["model.embed_tokens.weight"], tokens)
    for layer in range(config["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
        x = x + attention_part(h, positions, w, p + "self_attn.", config, inv_freq)
        h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + gated_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                          w[p + "mlp.down_proj.weight"])
    z = rms_norm(x, w["model.norm.weight"], eps)
    head = (w["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False)
            else w["lm_head.weight"])
    return z @ head.T


# --------------------------------------------------------------------------- sampling

MASK64 = (1 << 64) - 1


class PlainSampler:
    """Repeat penalty, temperature, top-k, top-p, min-p and the draw, in the
    order of apps/engine/src/sampler.rs:54-96; xorshift64* of sampler.rs:98-107."""

    def __init__(self, seed):
        self.state = (seed | 1) & MASK64

    def next_uniform(self):
        x = self.state
        x ^= x >> 12
        x ^= (x << 25) & MASK64
        x ^= x >> 27
        self.state = x
        value = (x * 0x2545F4914F6CDD1D) & MASK64
        return float(value >> 40) / float(1 << 24)

    def sample(self, logits, recent, temperature=0.7, top_k=40, top_p=0.75, min_p=0.25,
               repeat_penalty=1.1, repeat_last_n=64):
        logits = logits.to(torch.float32).clone()
        if repeat_penalty != 1.0 and repeat_last_n > 0:
            # a token that occurs twice in the window is penalised twice (sampler.rs:115-127)
            for token in recent[max(0, len(recent) - repeat_last_n):]:
                if token < logits.numel():
                    value = logits[token]
                    logits[token] = value / repeat_penalty if value > 0 else value * repeat_penalty
        if temperature <= 0.0:
            return argmax_first(logits)
        logits = logits * torch.tensor(1.0 / temperature, dtype=torch.float32)
        order = sorted(range(logits.numel()), key=lambda i: (-logits[i].item(), i))
        if 0 < top_k < len(order):
            order = order[:top_k]
        values = logits[order]
        probs = torch.exp(values - values[0])
        probs = probs / probs.sum()
        if 0.0 <= top_p < 1.0:
            cumulative = torch.cumsum(probs, 0)
            over = (cumulative > top_p).nonzero()
            keep = int(over[0]) + 1 if over.numel() else len(order)
            order, probs = order[:keep], probs[:keep]
        if min_p > 0.0:
            keep = int((probs >= probs[0] * min_p).sum())
            order, probs = order[:keep], probs[:keep]
        total = float(probs.sum())
        if total <= 0.0:
            return argmax_first(logits)
        target = self.next_uniform() * total
        for token, p in zip(order, probs.tolist()):
            target -= p
            if target <= 0.0:
                return token
        return order[0]


def argmax_first(values):
    """First maximum wins (apps/engine/src/sampler.rs:167-175)."""
    best = values.max()
    return int((values == best).nonzero()[0])


def generate(config, w, prompt, max_tokens, stop_tokens=(), context=None, seed=0, **sampling):
    """Prefill, then sample / stop / emit / step as apps/engine/src/generate.rs:96-127,
    re-running the whole sequence for every token. Returns (tokens, stop reason)."""
    sampler = PlainSampler(seed)
    sequence = list(prompt)
    emitted = []
    reason = "max_tokens"
    while len(emitted) < max_tokens:
        logits = forward(config, w, sequence)[-1]
        token = sampler.sample(logits, emitted, **sampling)
        if token in stop_tokens:
            reason = "eos"
            break
        emitted.append(token)
        if context is not None and len(sequence) >= context:
            reason = "context_full"
            break
        sequence.append(token)
    return emitted, reason
