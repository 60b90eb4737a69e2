"""Host-side logic of the engine on the CPU: the kernels are replaced by their
plain PyTorch statements, and the result is compared with the plain whole-
sequence implementation. What is under test is packing, positions, pages,
slots, chunked passes and the order of the returned rows."""
import pytest
import torch

import plain_llama
from tiny import make_folder, random_tokens

from llm_b200.engine import Engine, Entry, load_model


def _setup(tmp_path, which, **engine_options):
    folder = make_folder(tmp_path, which, torch.float32)
    config, weights = plain_llama.read_model_folder(folder)
    model = load_model(folder, torch.float32, "cpu")
    engine = Engine(model, **{"max_tokens": 1024, **engine_options})
    return config, weights, engine


@pytest.mark.parametrize("which", ["A", "B"])
def test_whole_prompt_matches_plain(tmp_path, plain_kernels, which):
    config, weights, engine = _setup(tmp_path, which)
    tokens = random_tokens(23, config["vocab_size"], 7)
    expected = plain_llama.forward(config, weights, tokens)
    (slot,) = engine.acquire()
    logits = engine.step([Entry(slot, tokens, list(range(len(tokens))))])
    assert torch.allclose(logits, expected, atol=2e-5, rtol=1e-5)
    engine.release([slot])
    engine.cache.check()


@pytest.mark.parametrize("which", ["A", "B"])
def test_token_by_token_and_unequal_batch(tmp_path, plain_kernels, which):
    config, weights, engine = _setup(tmp_path, which)
    lengths = [5, 9, 17, 70] if which == "A" else [1, 7, 33, 64]
    seqs = [random_tokens(n + 6, config["vocab_size"], 11 + i) for i, n in enumerate(lengths)]
    expected = [plain_llama.forward(config, weights, s) for s in seqs]
    slots = engine.acquire(len(seqs))
    # prompts together, wanting the last place of each
    logits = engine.step([Entry(s, seq[:n], [n - 1]) for s, seq, n in zip(slots, seqs, lengths)])
    for b, n in enumerate(lengths):
        assert torch.allclose(logits[b], expected[b][n - 1], atol=2e-5, rtol=1e-5)
    # then one token each; the two shortest end two steps early
    live = list(range(len(seqs)))
    for k in range(6):
        if k == 4:
            engine.release([slots[0], slots[1]])
            live = live[2:]
        logits = engine.step([Entry(slots[b], [seqs[b][lengths[b] + k]], [0]) for b in live])
        for row, b in enumerate(live):
            assert torch.allclose(logits[row], expected[b][lengths[b] + k], atol=2e-5, rtol=1e-5)
    engine.release([slots[b] for b in live])
    engine.cache.check()
    assert engine.cache.slots.n_held == 0


def test_chunked_passes_equal_one_pass(tmp_path, plain_kernels):
    config, weights, engine = _setup(tmp_path, "B", step_tokens=16)
    seqs = [random_tokens(n, config["vocab_size"], 3 + n) for n in (40, 5, 17)]
    wants = [[0, 15, 16, 39], [4], [16, 2]]
    slots = engine.acquire(3)
    logits = engine.step([Entry(s, q, w) for s, q, w in zip(slots, seqs, wants)])
    row = 0
    for q, w in zip(seqs, wants):
        expected = plain_llama.forward(config, weights, q)
        for place in w:
            assert torch.allclose(logits[row], expected[place], atol=2e-5, rtol=1e-5)
            row += 1
    assert row == logits.shape[0]


def test_a_token_budget_per_pass_changes_nothing(tmp_path, plain_kernels):
    """Five prompts, at most 40 tokens a pass and 16 of one sequence: the same logits, in
    the caller's order, as one pass would give."""
    config, weights, engine = _setup(tmp_path, "A", step_tokens=16, pass_tokens=40)
    seqs = [random_tokens(n, config["vocab_size"], 50 + n) for n in (33, 7, 20, 1, 45)]
    wants = [[32, 0], [6], [], [0], [44, 15, 16]]
    slots = engine.acquire(5)
    logits = engine.step([Entry(s, q, w) for s, q, w in zip(slots, seqs, wants)])
    row = 0
    for q, w in zip(seqs, wants):
        expected = plain_llama.forward(config, weights, q)
        for place in w:
            assert torch.allclose(logits[row], expected[place], atol=2e-5, rtol=1e-5)
            row += 1
    assert row == logits.shape[0]
    assert [engine.length(s) for s in slots] == [33, 7, 20, 1, 45]


def test_slots_are_reused_between_batches(tmp_path, plain_kernels):
    config, weights, engine = _setup(tmp_path, "A", max_tokens=192, max_slots=2)
    for round_index in range(3):
        seqs = [random_tokens(60 + 10 * i, config["vocab_size"], 100 * round_index + i) for i in range(2)]
        slots = engine.acquire(2)
        logits = engine.step([Entry(s, q, [len(q) - 1]) for s, q in zip(slots, seqs)])
        for b, q in enumerate(seqs):
            expected = plain_llama.forward(config, weights, q)
            assert torch.allclose(logits[b], expected[-1], atol=2e-5, rtol=1e-5)
        engine.release(slots)
        engine.cache.check()


def test_ids_that_are_still_on_the_device_follow_their_entries_into_every_pass(tmp_path, plain_kernels):
    """A decode step of five sequences with at most two tokens a pass, fed by a tensor of ids
    instead of host ids: every pass must take its own entries' ids (not placeholder zeros)."""
    config, weights, engine = _setup(tmp_path, "A", pass_tokens=2)
    seqs = [random_tokens(n, config["vocab_size"], 80 + n) for n in (9, 4, 12, 6, 3)]
    slots = engine.acquire(5)
    engine.step([Entry(s, q[:-1], []) for s, q in zip(slots, seqs)])
    feed = torch.tensor([q[-1] for q in seqs], dtype=torch.int32)
    logits = engine.step([Entry(s, [0], [0]) for s in slots], device_tokens=feed)
    for b, q in enumerate(seqs):
        expected = plain_llama.forward(config, weights, q)
        assert torch.allclose(logits[b], expected[-1], atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("which", ["A", "B"])
def test_folded_norms_change_nothing_beyond_rounding(tmp_path, plain_kernels, monkeypatch, which):
    """bfloat16 runs fold every layer's norms into the products behind them (the gain into the
    weights, the scale into the epilogue, the input left by the product before). With the plain
    kernels in the kernels' place: the folded and the unfolded model agree with each other and
    with the plain implementation to bfloat16 rounding, in a prefill and in decode steps."""
    import llm_b200.parts.block as block_module
    folder = make_folder(tmp_path, which, torch.bfloat16)
    config, weights = plain_llama.read_model_folder(folder)
    tokens = random_tokens(40, config["vocab_size"], 5)
    expected = plain_llama.forward(config, weights, tokens)
    results = []
    for fold in (True, False):
        monkeypatch.setattr(block_module, "FOLD_NORMS", fold)
        model = load_model(folder, torch.bfloat16, "cpu")
        assert all(b.folded_mixer == fold and b.folded_ffn == fold for b in model.blocks)
        engine = Engine(model, max_tokens=256)
        (slot,) = engine.acquire()
        rows = [engine.step([Entry(slot, tokens[:36], list(range(36)))])]
        rows += [engine.step([Entry(slot, [t], [0])]) for t in tokens[36:]]
        results.append(torch.cat(rows))
    scale = float(expected.abs().max())
    for got in results:
        assert float((got - expected).abs().max()) <= 0.04 * scale
    assert float((results[0] - results[1]).abs().max()) <= 0.04 * scale
