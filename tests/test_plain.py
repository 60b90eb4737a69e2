"""The plain implementation itself, against hand-computed values (the values the
op tests of MythEclipse/llm pin, apps/engine/tests/ops.rs:5-93) and against the
properties its parts must have."""
import math

import pytest
import torch

import plain_llama as P
import plain_ops


def test_rms_norm_hand_value():
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    out = P.rms_norm(x, torch.tensor([1.0, 1.0, 2.0, 0.5]), 0.0)
    scale = 1.0 / math.sqrt(7.5)
    assert torch.allclose(out, torch.tensor([[1 * scale, 2 * scale, 6 * scale, 2 * scale]]))
    assert torch.allclose(P.rms_norm(torch.zeros(1, 4), torch.ones(4), 1e-6), torch.zeros(1, 4))


def test_silu_and_softmax_hand_values():
    assert P.silu(torch.tensor(1.0)).item() == pytest.approx(1 / (1 + math.exp(-1)))
    assert P.silu(torch.tensor(-1.0)).item() == pytest.approx(-1 / (1 + math.exp(1)))
    assert torch.allclose(P.softmax(torch.tensor([5.0, 5.0, 5.0, 5.0])), torch.full((4,), 0.25))
    assert torch.allclose(P.softmax(torch.tensor([0.0, math.log(3.0)])), torch.tensor([0.25, 0.75]))


@pytest.mark.parametrize("pairing", ["half", "interleaved"])
def test_rope_rotates_pairs_and_keeps_their_norm(pairing):
    inv_freq = P.rope_inverse_frequencies(4, 10000.0)
    assert inv_freq.tolist() == pytest.approx([1.0, 0.01])
    x = torch.zeros(1, 1, 4)
    if pairing == "half":
        x[0, 0, 0] = 1.0                     # pair 0 is (0, 2)
        out = P.rope_rotate(x, [1], inv_freq, pairing)
        assert out[0, 0].tolist() == pytest.approx([math.cos(1), 0, math.sin(1), 0], abs=1e-6)
    else:
        x[0, 0, 0] = 1.0                     # pair 0 is (0, 1)
        out = P.rope_rotate(x, [1], inv_freq, pairing)
        assert out[0, 0].tolist() == pytest.approx([math.cos(1), math.sin(1), 0, 0], abs=1e-6)
    y = torch.randn(5, 3, 8)
    turned = P.rope_rotate(y, [0, 1, 7, 100, 1000], P.rope_inverse_frequencies(8, 500000.0), pairing)
    assert torch.allclose(turned.norm(dim=-1), y.norm(dim=-1), atol=1e-5)
    assert torch.equal(turned[0], y[0])      # position 0 turns nothing


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    out = P.causal_attention(q, k, v, 0.3)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])   # first token sees itself
    k2, v2 = k.clone(), v.clone()
    k2[5], v2[5] = 9.0, 9.0                  # the future does not reach the past
    assert torch.allclose(P.causal_attention(q, k2, v2, 0.3)[:5], out[:5])
    windowed = P.causal_attention(q, k, v, 0.3, window=2)
    assert torch.allclose(windowed[:2], out[:2]) and not torch.allclose(windowed[5], out[5])
    scores = (k[4:6, 0] @ q[5, 0]) * 0.3
    assert torch.allclose(windowed[5, 0], P.softmax(scores) @ v[4:6, 0], atol=1e-6)


def test_argmax_first_maximum_and_xorshift():
    assert P.argmax_first(torch.tensor([1.0, 3.0, 3.0, 2.0])) == 1
    s = P.PlainSampler(0)                   # state seed | 1 = 1
    x = 1
    x ^= x >> 12; x ^= (x << 25) & P.MASK64; x ^= x >> 27
    expected = float(((x * 0x2545F4914F6CDD1D) & P.MASK64) >> 40) / float(1 << 24)
    assert s.next_uniform() == expected and 0.0 <= expected < 1.0


def test_sampler_chain_order_and_filters():
    logits = torch.tensor([2.0, 1.0, 0.5, -1.0, 3.0])
    s = P.PlainSampler(3)
    assert s.sample(logits, [], temperature=0.0, repeat_penalty=1.0) == 4
    assert s.sample(logits, [4, 4], temperature=0.0, repeat_penalty=2.0, repeat_last_n=64) == 0   # 3 / 2 / 2 < 2
    assert s.sample(logits, [4, 4], temperature=0.0, repeat_penalty=2.0, repeat_last_n=0) == 4
    assert s.sample(torch.tensor([-1.0, -2.0]), [0], temperature=0.0, repeat_penalty=3.0) == 1    # negative: multiplied
    for _ in range(20):                      # top_k 1 and a tiny top_p both leave only the best token
        assert s.sample(logits, [], temperature=1.0, top_k=1, top_p=1.0, min_p=0.0, repeat_penalty=1.0) == 4
        assert s.sample(logits, [], temperature=1.0, top_k=0, top_p=0.01, min_p=0.0, repeat_penalty=1.0) == 4
        assert s.sample(logits, [], temperature=1.0, top_k=0, top_p=1.0, min_p=0.9, repeat_penalty=1.0) == 4
    draws = {s.sample(logits, [], temperature=5.0, top_k=3, top_p=1.0, min_p=0.0, repeat_penalty=1.0)
             for _ in range(200)}
    assert draws == {4, 0, 1}                # only the three best are ever drawn


def test_plain_ops_sampler_equals_plain_sampler():
    """The per-kernel statement of the sampling chain and the sampler of the plain
    model are two writings of the same rule."""
    torch.manual_seed(1)
    for trial in range(30):
        logits = torch.randn(300) * 2
        recent = [int(t) for t in torch.randint(0, 300, (5,))]
        kwargs = dict(temperature=0.9, top_k=12, top_p=0.8, min_p=0.05, repeat_penalty=1.2, repeat_last_n=4)
        sampler = P.PlainSampler(trial)
        want = sampler.sample(logits, recent, **kwargs)
        params = torch.tensor([[0.9, 0.8, 0.05, 1.2]])
        iparams = torch.tensor([[12, 4]], dtype=torch.int32)
        window = torch.tensor([recent[-4:]], dtype=torch.int32)
        state = torch.tensor([(trial | 1)], dtype=torch.int64)
        out, status = torch.zeros(1, dtype=torch.int32), torch.zeros(1, dtype=torch.int32)
        plain_ops.sample_rows(logits[None].clone(), params, iparams, window,
                              torch.tensor([4], dtype=torch.int32), state, out, status)
        assert int(out[0]) == want and int(state[0]) == sampler.state
