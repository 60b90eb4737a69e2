"""config.json contents of the model shapes the benchmarks run with random weights."""
from __future__ import annotations

_LLAMA3 = {"rope_type": "llama3", "low_freq_factor": 1.0, "high_freq_factor": 4.0,
           "original_max_position_embeddings": 8192}

SHAPES = {
    "llama-3.1-8b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 32,
        "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
        "intermediate_size": 14336, "vocab_size": 128256, "rope_theta": 500000.0,
        "rope_scaling": dict(_LLAMA3, factor=8.0), "rms_norm_eps": 1e-5,
        "tie_word_embeddings": False, "attention_bias": False,
        "max_position_embeddings": 131072, "hidden_act": "silu",
    },
    "llama-2-7b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 32,
        "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 32, "head_dim": 128,
        "intermediate_size": 11008, "vocab_size": 32000, "rope_theta": 10000.0,
        "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
        "attention_bias": False, "max_position_embeddings": 4096, "hidden_act": "silu",
    },
    "llama-3.2-1b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 16,
        "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
        "intermediate_size": 8192, "vocab_size": 128256, "rope_theta": 500000.0,
        "rope_scaling": dict(_LLAMA3, factor=32.0), "rms_norm_eps": 1e-5,
        "tie_word_embeddings": True, "attention_bias": False,
        "max_position_embeddings": 131072, "hidden_act": "silu",
    },
}


def shape(name: str, layers: int | None = None) -> dict:
    """A copy of the named shape's config.json, optionally with fewer layers."""
    from .errors import FormatError
    if name not in SHAPES:
        raise FormatError(f"unknown shape '{name}' (known: {', '.join(sorted(SHAPES))})")
    raw = dict(SHAPES[name])
    if layers is not None:
        raw["num_hidden_layers"] = layers
    return raw
