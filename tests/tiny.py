"""The tiny configurations the tests run, and helpers to make model folders.

A and B differ in every size and option: layers, hidden, heads, kv heads
(groups of 2 and 3), head size, feed-forward width (172 is no multiple of 16),
vocabulary, rope base, llama3 scaling or none, eps, tied or separate head,
attention bias or none, context.
"""
from __future__ import annotations

import torch

TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 172, "vocab_size": 256,
    "rope_theta": 10000.0, "rope_scaling": None, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "attention_bias": False, "max_position_embeddings": 128,
    "hidden_act": "silu", "eos_token_id": 2,
}

TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 256, "vocab_size": 384,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "attention_bias": True,
    "max_position_embeddings": 256, "hidden_act": "silu", "eos_token_id": [1, 5],
}

# a third shape for long sequences: more heads per group, head size 64, 600 positions
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 8,
    "num_key_value_heads": 2, "head_dim": 48, "intermediate_size": 208, "vocab_size": 1000,
    "rope_theta": 50000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "attention_bias": False, "max_position_embeddings": 1024, "hidden_act": "silu",
}

# sizes the tensor-core kernels serve: head size 64, widths that are multiples of 64
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 320, "vocab_size": 512,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "attention_bias": True, "max_position_embeddings": 1024, "hidden_act": "silu",
}

# sizes no fast kernel takes: a width of 100 (rows of 200 bytes are no multiple of 16), head size
# 80, five heads without grouping, an odd feed-forward width and an odd vocabulary
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 100, "num_attention_heads": 5,
    "num_key_value_heads": 5, "head_dim": 80, "intermediate_size": 333, "vocab_size": 1001,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "attention_bias": False, "max_position_embeddings": 512, "hidden_act": "silu",
}

# the head size, grouping and kind of sizes of the Llama-3 family in small: head size 128, four
# query heads per kv head, a feed-forward width and a vocabulary that are no powers of two, llama3
# frequency scaling whose bands lie inside the tested lengths
TINY_F = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 512, "num_attention_heads": 4,
    "num_key_value_heads": 1, "head_dim": 128, "intermediate_size": 1408, "vocab_size": 5000,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 256},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "attention_bias": False,
    "max_position_embeddings": 2048, "hidden_act": "silu",
}

CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3), "E": (TINY_E, 4),
           "F": (TINY_F, 5)}


def make_folder(tmp_path, which: str, dtype=torch.bfloat16, std=None):
    """Write the model folder of tiny config `which` and return its path."""
    from llm_b200.config import config_from_dict
    from llm_b200.weights import write_random_model
    raw, seed = CONFIGS[which]
    config = config_from_dict(dict(raw))
    folder = tmp_path / f"tiny_{which}_{str(dtype).split('.')[-1]}"
    if not (folder / "model.safetensors").exists():
        # a larger std than 0.02 so that attention and the feed-forward matter
        # beside the residual stream at these tiny widths
        write_random_model(folder, config, seed, dtype, std=std if std is not None else 0.08)
    return folder


def random_tokens(n: int, vocab: int, seed: int) -> list:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=gen).tolist()
