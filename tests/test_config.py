"""Configuration: config.json keys, defaults, checks, the architecture registry."""
import json

import pytest

from tiny import TINY_A, TINY_B

from llm_b200.config import LlamaConfig, config_from_dict, known_architectures, load_config
from llm_b200.errors import FormatError, MissingKey, Unsupported


def test_every_size_comes_from_the_file():
    a, b = config_from_dict(dict(TINY_A)), config_from_dict(dict(TINY_B))
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads,
            a.head_dim, a.intermediate_size, a.vocab_size) == (2, 64, 4, 2, 16, 172, 256)
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads,
            b.head_dim, b.intermediate_size, b.vocab_size) == (3, 96, 3, 1, 32, 256, 384)
    assert a.rms_norm_eps == 1e-5 and b.rms_norm_eps == 1e-6
    assert a.rope_scaling is None and b.rope_scaling["factor"] == 8.0
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert b.attention_bias and not a.attention_bias
    assert a.eos_token_id == (2,) and b.eos_token_id == (1, 5)


def test_defaults_follow_the_reference():
    raw = {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 1, "hidden_size": 32,
           "num_attention_heads": 4, "intermediate_size": 8, "vocab_size": 10}
    c = config_from_dict(raw)
    assert c.num_key_value_heads == 4 and c.head_dim == 8          # apps/engine/src/model.rs:89-92
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-6      # model.rs:96-97
    assert not c.tie_word_embeddings and not c.attention_bias and c.eos_token_id == ()


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads",
                                 "intermediate_size", "vocab_size"])
def test_missing_key_is_named(key):
    raw = dict(TINY_A)
    del raw[key]
    with pytest.raises(MissingKey) as error:
        config_from_dict(raw)
    assert key in str(error.value)


def test_bad_values_are_refused():
    with pytest.raises(FormatError):
        config_from_dict(dict(TINY_A, num_key_value_heads=3))           # 4 heads over 3 kv heads
    with pytest.raises(FormatError):
        config_from_dict(dict(TINY_A, head_dim=15))
    with pytest.raises(FormatError):
        config_from_dict(dict(TINY_A, hidden_size="64"))
    with pytest.raises(Unsupported):
        config_from_dict(dict(TINY_A, hidden_act="gelu"))
    with pytest.raises(Unsupported):
        config_from_dict(dict(TINY_A, rope_scaling={"rope_type": "yarn", "factor": 2.0}))
    with pytest.raises(FormatError):
        config_from_dict(dict(TINY_B, rope_scaling={"rope_type": "llama3", "factor": 8.0}))
    with pytest.raises(Unsupported):
        config_from_dict(dict(TINY_A, mlp_bias=True))


def test_registry_picks_by_architecture_name(tmp_path):
    assert "LlamaForCausalLM" in known_architectures()
    with pytest.raises(Unsupported) as error:
        config_from_dict(dict(TINY_A, architectures=["MambaForCausalLM"]))
    assert "LlamaForCausalLM" in str(error.value)
    with pytest.raises(FormatError):
        config_from_dict({"hidden_size": 4})
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert isinstance(load_config(tmp_path), LlamaConfig)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(FormatError):
        load_config(tmp_path)


def test_round_trip_and_model_spec():
    c = config_from_dict(dict(TINY_B))
    again = config_from_dict(c.to_dict())
    assert again == c
    spec = c.model_spec()
    assert len(spec.blocks) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    mixer = spec.blocks[1].mixer
    assert (mixer.n_heads, mixer.n_kv_heads, mixer.head_dim, mixer.bias) == (3, 1, 32, True)
    assert mixer.tensor["q"] == "model.layers.1.self_attn.q_proj.weight"
    assert mixer.position.theta == 500000.0 and mixer.position.scaling_dict["factor"] == 8.0
    assert spec.blocks[0].mixer_norm.eps == 1e-6 and spec.head == "lm_head.weight"
    assert config_from_dict(dict(TINY_A)).model_spec().head is None


def test_llama3_frequencies_hit_all_three_branches():
    """Tiny B: pairs 0 and 1 keep their frequency, pair 2 is blended, the rest are divided
    by the factor (hand values from the llama3 rule, original length 64)."""
    import math

    from llm_b200.parts import inverse_frequencies
    scaling = dict(TINY_B["rope_scaling"])
    plain = [500000.0 ** (-2.0 * p / 32) for p in range(16)]
    got = inverse_frequencies(32, 500000.0, scaling).tolist()
    assert got[0] == plain[0] and got[1] == plain[1]
    wavelength = 2 * math.pi / plain[2]
    assert 64 / 4 < wavelength < 64 / 1
    smooth = (64 / wavelength - 1.0) / (4.0 - 1.0)
    assert got[2] == pytest.approx((1 - smooth) * plain[2] / 8 + smooth * plain[2], rel=1e-12)
    for p in range(3, 16):
        assert got[p] == pytest.approx(plain[p] / 8, rel=1e-12)
