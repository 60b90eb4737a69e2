"""Configuration of the Llama decoder, read from its own config.json keys."""
from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass
from typing import Optional

from ..errors import FormatError, Unsupported
from ..parts.spec import (AttentionSpec, BlockSpec, GatedMlpSpec, ModelSpec, NormSpec,
                          PositionSpec, ScheduleEntry, names)
from .base import ConfigReader

_LLAMA3_KEYS = ("factor", "low_freq_factor", "high_freq_factor",
                "original_max_position_embeddings")


@dataclass(frozen=True)
class LlamaConfig:
    """Sizes and constants of one Llama model.

    The fields and their defaults follow what the engine of MythEclipse/llm
    reads from a GGUF header (apps/engine/src/model.rs:86-101: kv heads
    default to heads, head_dim to hidden/heads, rope base 1e4, eps 1e-6) and
    its checks (model.rs:137-141: heads divisible by kv heads), under the
    names a Llama config.json uses.
    """
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[dict]
    max_position_embeddings: int
    tie_word_embeddings: bool
    attention_bias: bool
    eos_token_id: tuple
    hidden_act: str = "silu"

    architecture = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "LlamaConfig":
        r = ConfigReader(raw, where)
        hidden = r.integer("hidden_size", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        kv_heads = r.integer("num_key_value_heads", heads, minimum=1)
        head_dim = r.integer("head_dim", None)
        if head_dim is None:
            if hidden % heads:
                raise FormatError(f"{where}: hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads} and no head_dim is given")
            head_dim = hidden // heads
        if heads % kv_heads:
            raise FormatError(f"{where}: num_attention_heads {heads} is not a multiple of "
                              f"num_key_value_heads {kv_heads}")
        if head_dim < 2 or head_dim % 2:
            raise FormatError(f"{where}: head_dim {head_dim} must be even")
        act = r.string("hidden_act", "silu")
        if act != "silu":
            raise Unsupported(f"{where}: hidden_act '{act}' (only 'silu' is built)")
        if r.boolean("mlp_bias", False):
            raise Unsupported(f"{where}: mlp_bias true is not built")
        scaling = r.mapping("rope_scaling", None)
        if scaling is not None:
            scaling = cls._check_scaling(scaling, where)
        return cls(
            vocab_size=r.integer("vocab_size", minimum=1),
            hidden_size=hidden,
            intermediate_size=r.integer("intermediate_size", minimum=1),
            num_hidden_layers=r.integer("num_hidden_layers", minimum=1),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=r.number("rms_norm_eps", 1e-6, positive=True),
            rope_theta=r.number("rope_theta", 10000.0, positive=True),
            rope_scaling=scaling,
            max_position_embeddings=r.integer("max_position_embeddings", 2048, minimum=1),
            tie_word_embeddings=r.boolean("tie_word_embeddings", False),
            attention_bias=r.boolean("attention_bias", False),
            eos_token_id=r.integer_list("eos_token_id", None),
            hidden_act=act,
        )

    @staticmethod
    def _check_scaling(scaling: dict, where: str) -> Optional[dict]:
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise Unsupported(f"{where}: rope_scaling type '{kind}' (built: 'llama3', 'default')")
        out = {"rope_type": "llama3"}
        for key in _LLAMA3_KEYS:
            value = scaling.get(key)
            if isinstance(value, bool) or not isinstance(value, (int, float)) or not value > 0:
                raise FormatError(f"{where}: rope_scaling.{key} must be a positive number")
            out[key] = float(value)
        if out["high_freq_factor"] <= out["low_freq_factor"]:
            raise FormatError(f"{where}: rope_scaling.high_freq_factor must exceed low_freq_factor")
        return out

    def to_dict(self) -> dict:
        raw = asdict(self)
        raw["architectures"] = [self.architecture]
        raw["model_type"] = "llama"
        eos = list(self.eos_token_id)
        raw["eos_token_id"] = eos[0] if len(eos) == 1 else (eos or None)
        return raw

    def to_json(self) -> str:
        return json.dumps(self.to_dict(), indent=2) + "\n"

    # ------------------------------------------------------------------ the model as data

    def model_spec(self) -> ModelSpec:
        """Every layer with its parts, sizes, constants and tensor names."""
        position = PositionSpec(
            head_dim=self.head_dim, theta=self.rope_theta,
            max_positions=self.max_position_embeddings,
            scaling=tuple(sorted(self.rope_scaling.items())) if self.rope_scaling else None,
            pairing="half")
        blocks = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            roles = {r: f"{p}self_attn.{r}_proj.weight" for r in ("q", "k", "v", "o")}
            if self.attention_bias:
                roles.update({f"{r}_bias": f"{p}self_attn.{r}_proj.bias" for r in ("q", "k", "v", "o")})
            mixer = AttentionSpec(
                hidden=self.hidden_size, n_heads=self.num_attention_heads,
                n_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                scale=1.0 / math.sqrt(self.head_dim), bias=self.attention_bias, window=0,
                position=position, names=names(**roles))
            ffn = GatedMlpSpec(
                hidden=self.hidden_size, intermediate=self.intermediate_size,
                activation=self.hidden_act,
                names=names(gate=p + "mlp.gate_proj.weight", up=p + "mlp.up_proj.weight",
                            down=p + "mlp.down_proj.weight"))
            blocks.append(BlockSpec(
                mixer_norm=NormSpec(self.hidden_size, self.rms_norm_eps, p + "input_layernorm.weight"),
                mixer=mixer,
                ffn_norm=NormSpec(self.hidden_size, self.rms_norm_eps,
                                  p + "post_attention_layernorm.weight"),
                feed_forward=ffn))
        return ModelSpec(
            architecture=self.architecture, vocab=self.vocab_size, hidden=self.hidden_size,
            max_positions=self.max_position_embeddings,
            embedding="model.embed_tokens.weight", blocks=tuple(blocks),
            schedule=tuple(ScheduleEntry(i) for i in range(self.num_hidden_layers)),
            final_norm=NormSpec(self.hidden_size, self.rms_norm_eps, "model.norm.weight"),
            head=None if self.tie_word_embeddings else "lm_head.weight",
            stop_tokens=tuple(self.eos_token_id))
