"""The generation loop's decisions, on the CPU: batches, stop tokens, sequences that
end earlier, limits, slot release, the sampler's parameters. The engine's kernels
are replaced by their plain statements; the model is a tiny random Llama."""
import pytest
import torch

import plain_llama
from tiny import make_folder, random_tokens

from llm_b200.engine import Engine, GenerationRequest, generate, load_model, plan_batches
from llm_b200.errors import ContextFull, FormatError, Unsupported
from llm_b200.sampling import SamplingParams


def test_plan_batches_keeps_order_and_limits():
    fits = lambda lengths: sum((n + 63) // 64 for n in lengths) <= 4
    plan = plan_batches([(0, 64), (1, 64), (2, 130), (3, 10), (4, 10), (5, 200)], fits, max_batch=3)
    assert plan == [[0, 1], [2, 3], [4], [5]]
    assert plan_batches([(i, 1) for i in range(5)], lambda l: True, max_batch=2) == [[0, 1], [2, 3], [4]]
    with pytest.raises(ContextFull):
        plan_batches([(0, 1000)], fits, max_batch=3)


@pytest.fixture
def engine(tmp_path, plain_kernels):
    folder = make_folder(tmp_path, "A", torch.float32)
    model = load_model(folder, torch.float32, "cpu")
    config, weights = plain_llama.read_model_folder(folder)
    return Engine(model, max_tokens=64 * 3, max_seq_len=40, max_slots=3), config, weights


def test_unequal_batch_greedy_equals_plain_one_by_one(engine):
    eng, config, weights = engine
    prompts = [random_tokens(n, 256, 20 + n) for n in (5, 9, 17, 3, 11)]       # five requests, three slots
    requests = [GenerationRequest(p, max_tokens=3 + i, params=SamplingParams(temperature=0.0))
                for i, p in enumerate(prompts)]
    seen = []
    results = generate(eng, requests, on_token=lambda i, t: seen.append((i, t)))
    for i, (p, r) in enumerate(zip(prompts, results)):
        want, reason = plain_llama.generate(config, weights, p, 3 + i, temperature=0.0)
        assert r.tokens == want and r.stop_reason == reason == "max_tokens"
        assert r.prompt_tokens == len(p) and r.generated_tokens == len(want)
        assert [t for j, t in seen if j == i] == want
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and eng.cache.groups[0].pool.n_held == 0


def test_stop_token_is_neither_emitted_nor_fed(engine):
    eng, config, weights = engine
    prompt = random_tokens(8, 256, 1)
    free, _ = plain_llama.generate(config, weights, prompt, 6, temperature=0.0)
    stop = free[3]
    cut = free[:free.index(stop)]
    results = generate(eng, [GenerationRequest(prompt, 6, SamplingParams(temperature=0.0), (stop,)),
                             GenerationRequest(prompt, 6, SamplingParams(temperature=0.0), ())])
    assert results[0].tokens == cut and results[0].stop_reason == "eos"
    assert results[1].tokens == free and results[1].stop_reason == "max_tokens"   # its neighbour went on


def test_context_full_max_tokens_zero_and_cancel(engine):
    eng, config, weights = engine
    prompt = random_tokens(37, 256, 2)
    (r,) = generate(eng, [GenerationRequest(prompt, 50, SamplingParams(temperature=0.0))])
    want, reason = plain_llama.generate(config, weights, prompt, 50, context=40, temperature=0.0)
    assert r.tokens == want and r.stop_reason == reason == "context_full" and len(want) == 4
    (r,) = generate(eng, [GenerationRequest(prompt, 0)])
    assert r.tokens == [] and r.stop_reason == "max_tokens"
    calls = []
    def cancel():
        calls.append(1)
        return len(calls) > 2
    (r,) = generate(eng, [GenerationRequest(prompt[:5], 20, SamplingParams(temperature=0.0))], cancel=cancel)
    assert r.stop_reason == "cancelled" and len(r.tokens) == 2
    assert eng.cache.slots.n_held == 0


def test_requests_are_checked_before_anything_runs(engine):
    eng, _, _ = engine
    with pytest.raises(FormatError):
        generate(eng, [GenerationRequest([], 4)])
    with pytest.raises(ContextFull):
        generate(eng, [GenerationRequest(list(range(41)), 4)])
    with pytest.raises(FormatError):
        generate(eng, [GenerationRequest([1, 2, 999], 4)])
    assert eng.cache.slots.n_held == 0
    big = SamplingParams(temperature=1.0, top_k=0, top_p=0.9)
    big.check(256)                                        # a small vocabulary is ranked whole
    with pytest.raises(Unsupported):
        big.check(128256)
    with pytest.raises(Unsupported):
        SamplingParams(temperature=1.0, top_k=5000).check(128256)
    SamplingParams(temperature=0.0, top_k=5000).check(128256)        # greedy ignores the rest


def test_seeded_sampling_equals_the_plain_chain(engine):
    eng, config, weights = engine
    prompts = [random_tokens(n, 256, 40 + n) for n in (4, 12)]
    params = [SamplingParams(temperature=0.8, seed=1), SamplingParams(temperature=1.3, top_k=5,
                                                                       top_p=0.9, min_p=0.0,
                                                                       repeat_penalty=1.5,
                                                                       repeat_last_n=2, seed=7)]
    results = generate(eng, [GenerationRequest(p, 6, s) for p, s in zip(prompts, params)])
    for p, s, r in zip(prompts, params, results):
        want, _ = plain_llama.generate(config, weights, p, 6, seed=s.seed, temperature=s.temperature,
                                       top_k=s.top_k, top_p=s.top_p, min_p=s.min_p,
                                       repeat_penalty=s.repeat_penalty, repeat_last_n=s.repeat_last_n)
        assert r.tokens == want
