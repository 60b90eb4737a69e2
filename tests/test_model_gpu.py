"""The engine on the GPU against the plain implementation, in 32-bit and in
bfloat16: whole requests, the last 32 tokens one by one, batches of unequal
lengths whose shorter requests end earlier with slots reused by the next
batch, long decoding, the first tokens of a sequence, and greedy generation
through the entry point."""
import pytest
import torch

import plain_llama
from tiny import CONFIGS, make_folder, random_tokens

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def close(got, want, dtype):
    """32-bit: equal to the plain implementation up to summation order.
    bfloat16: activations are rounded to 8 bits of mantissa between kernels,
    so logits agree to about 1 % of their range."""
    got, want = got.float().cpu(), want.float()
    scale = float(want.abs().max())
    if dtype == torch.float32:
        return float((got - want).abs().max()) <= 5e-5 * max(scale, 1.0)
    error = (got - want).abs()
    return float(error.max()) <= 0.04 * scale and float(error.mean()) <= 0.008 * scale


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {which: make_folder(root, which, torch.bfloat16) for which in CONFIGS}


@pytest.fixture(scope="module")
def plain(folders):
    return {which: plain_llama.read_model_folder(folder) for which, folder in folders.items()}


def engine_for(folder, dtype, **options):
    from llm_b200.engine import Engine, load_model
    model = load_model(folder, dtype, DEV)
    return Engine(model, **{"max_tokens": 4096, **options})


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["A", "B", "D", "E"])
def test_whole_request(folders, plain, dtype, which):
    from llm_b200.engine import Entry
    config, weights = plain[which]
    engine = engine_for(folders[which], dtype)
    for n in (1, 2, 65, 100):
        tokens = random_tokens(n, config["vocab_size"], 100 + n)
        (slot,) = engine.acquire()
        logits = engine.step([Entry(slot, tokens, list(range(n)))])
        assert close(logits, plain_llama.forward(config, weights, tokens), dtype), n
        engine.release([slot])
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["A", "B", "D", "E", "F"])
def test_last_32_tokens_one_by_one(folders, plain, dtype, which):
    from llm_b200.engine import Entry
    config, weights = plain[which]
    engine = engine_for(folders[which], dtype)
    tokens = random_tokens(100, config["vocab_size"], 5)
    expected = plain_llama.forward(config, weights, tokens)
    (slot,) = engine.acquire()
    head = len(tokens) - 32
    rows = [engine.step([Entry(slot, tokens[:head], list(range(head)))])]
    for t in tokens[head:]:
        rows.append(engine.step([Entry(slot, [t], [0])]))
    assert close(torch.cat(rows), expected, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["A", "B", "D", "F"])
def test_unequal_batches_with_slot_reuse(folders, plain, dtype, which):
    """Two batches one after the other on a cache that holds only one of them:
    the second batch gets the first one's slots and pages back."""
    from llm_b200.engine import Entry
    config, weights = plain[which]
    lengths = [1, 7, 33, 64] if which == "B" else [5, 9, 17, 70]
    extra = [3, 10, 6, 10]
    engine = engine_for(folders[which], dtype, max_tokens=64 * 5, max_slots=4)
    for batch in range(2):
        seqs = [random_tokens(n + e, config["vocab_size"], 31 * batch + i)
                for i, (n, e) in enumerate(zip(lengths, extra))]
        expected = [plain_llama.forward(config, weights, s) for s in seqs]
        slots = engine.acquire(4)
        logits = engine.step([Entry(s, q[:n], list(range(n))) for s, q, n in zip(slots, seqs, lengths)])
        at = 0
        for b, n in enumerate(lengths):
            assert close(logits[at:at + n], expected[b][:n], dtype), (batch, b)
            at += n
        live = [0, 1, 2, 3]
        for k in range(max(extra)):
            ended = [b for b in live if k >= extra[b]]
            engine.release([slots[b] for b in ended])
            live = [b for b in live if b not in ended]
            logits = engine.step([Entry(slots[b], [seqs[b][lengths[b] + k]], [0]) for b in live])
            for row, b in enumerate(live):
                assert close(logits[row], expected[b][lengths[b] + k], dtype), (batch, b, k)
        engine.release([slots[b] for b in live])
        engine.cache.check()
        assert engine.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["C", "D", "F"])
def test_long_decoding(folders, plain, dtype, which):
    """300 decode steps after a 40-token prompt, across several pages, beside a
    second sequence that grows from 1 token."""
    from llm_b200.engine import Entry
    config, weights = plain[which]
    engine = engine_for(folders[which], dtype)
    a = random_tokens(340, config["vocab_size"], 1)
    b = random_tokens(301, config["vocab_size"], 2)
    expect_a = plain_llama.forward(config, weights, a)
    expect_b = plain_llama.forward(config, weights, b)
    sa, sb = engine.acquire(2)
    engine.step([Entry(sa, a[:40], []), Entry(sb, b[:1], [])])
    got_a, got_b = [], []
    for k in range(300):
        logits = engine.step([Entry(sa, [a[40 + k]], [0]), Entry(sb, [b[1 + k]], [0])])
        got_a.append(logits[0])
        got_b.append(logits[1])
    assert close(torch.stack(got_a), expect_a[40:], dtype)
    assert close(torch.stack(got_b), expect_b[1:], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_family_shaped_model_prefill_and_decode(folders, plain, dtype):
    """Head size 128 with four query heads per kv head, prompts long enough for the paired
    tcgen05 product (more than 128 tokens), for several key blocks of the tcgen05 attention
    and for the llama3 frequency bands; then the split decode attention one token at a time."""
    from llm_b200.engine import Entry
    from llm_b200.ops import tactics
    config, weights = plain["F"]
    if dtype == torch.bfloat16:
        assert tactics.choose_attention(False, dtype, 4, 1, 128, 0, True) == "attention_prefill_tc"
        assert tactics.choose_attention(True, dtype, 4, 1, 128, 0) == "attention_decode"
        assert tactics.choose_linear(330, 768, 512, dtype, dtype, 512) == "gemm_tc"
    engine = engine_for(folders["F"], dtype)
    seqs = [random_tokens(n, config["vocab_size"], 300 + n) for n in (330, 140, 1)]
    expected = [plain_llama.forward(config, weights, s) for s in seqs]
    slots = engine.acquire(3)
    heads = [322, 132, 1]
    wanted = [[0, 127, 128, 255, 321], [0, 131], [0]]
    logits = engine.step([Entry(sl, s[:n], w) for sl, s, n, w in zip(slots, seqs, heads, wanted)])
    row = 0
    for b in range(3):
        for w in wanted[b]:
            assert close(logits[row], expected[b][w], dtype), (b, w)
            row += 1
    for k in range(8):                       # the third request has ended
        step = engine.step([Entry(slots[b], [seqs[b][heads[b] + k]], [0]) for b in range(2)])
        for b in range(2):
            assert close(step[b], expected[b][heads[b] + k], dtype), (b, k)
    engine.release(slots)
    engine.cache.check()
    engine.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_batch_of_seventy_sequences(folders, plain, dtype):
    """More sequences than the decode products' 64-token orientation takes (their steps run the
    kernels that prefill uses, on one token per sequence), lengths from 1 to 90, sequences
    leaving along the way."""
    from llm_b200.engine import Entry
    config, weights = plain["F"]
    engine = engine_for(folders["F"], dtype, max_tokens=70 * 128)
    lengths = [1 + (7 * i) % 90 for i in range(70)]
    seqs = [random_tokens(n + 4, config["vocab_size"], 500 + i) for i, n in enumerate(lengths)]
    watch = [0, 13, 37, 69]
    expected = {b: plain_llama.forward(config, weights, seqs[b]) for b in watch}
    slots = engine.acquire(70)
    logits = engine.step([Entry(slots[b], seqs[b][:lengths[b]], [lengths[b] - 1]) for b in range(70)])
    for b in watch:
        assert close(logits[b], expected[b][lengths[b] - 1], dtype), b
    live = list(range(70))
    for k in range(4):
        logits = engine.step([Entry(slots[b], [seqs[b][lengths[b] + k]], [0]) for b in live])
        for row, b in enumerate(live):
            if b in watch:
                assert close(logits[row], expected[b][lengths[b] + k], dtype), (b, k)
        gone = [b for b in live if b % 4 == k and b not in watch]      # a quarter leaves after each step
        engine.release([slots[b] for b in gone])
        live = [b for b in live if b not in gone]
    engine.release([slots[b] for b in live])
    engine.cache.check()
    engine.check()
    assert engine.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence(folders, plain, dtype):
    """Positions 0, 1, 2 decoded one by one from an empty slot."""
    from llm_b200.engine import Entry
    config, weights = plain["B"]
    engine = engine_for(folders["B"], dtype)
    tokens = random_tokens(4, config["vocab_size"], 9)
    expected = plain_llama.forward(config, weights, tokens)
    (slot,) = engine.acquire()
    rows = [engine.step([Entry(slot, [t], [0])]) for t in tokens]
    assert close(torch.cat(rows), expected, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_padding_and_neighbours_change_nothing(folders, dtype):
    """A request's logits are the same alone and beside other requests (32-bit: bit-equal)."""
    from llm_b200.engine import Entry
    engine = engine_for(folders["A"], dtype)
    tokens = random_tokens(50, 256, 4)
    (s,) = engine.acquire()
    alone = engine.step([Entry(s, tokens, [49])])
    engine.release([s])
    others = [random_tokens(n, 256, 60 + n) for n in (3, 120)]
    slots = engine.acquire(3)
    beside = engine.step([Entry(slots[0], others[0], []), Entry(slots[1], tokens, [49]),
                          Entry(slots[2], others[1], [])])
    if dtype == torch.float32:
        assert torch.equal(alone, beside)
    else:
        assert torch.allclose(alone, beside, atol=2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B"])
def test_greedy_generation_through_the_entry_point(folders, plain, dtype, which):
    import llm_b200
    config, weights = plain[which]
    llm = llm_b200.LLM(str(folders[which]), dtype=dtype, device=DEV, context=128, batch=3)
    prompts = [random_tokens(n, config["vocab_size"], 70 + n) for n in (5, 9, 17, 2)]
    # 32-bit: the default chain (greedy after the repeat penalty) token for token;
    # bfloat16: no penalty, so that each token can be checked against the plain logits
    penalty = 1.1 if dtype == "float32" else 1.0
    got = llm.generate(prompts, max_tokens=8, temperature=0.0, stop_tokens=[],
                       repeat_penalty=penalty)
    for prompt, tokens in zip(prompts, got):
        if dtype == "float32":
            want, _ = plain_llama.generate(config, weights, prompt, 8, temperature=0.0)
            assert tokens == want
        else:
            # bfloat16 may break a near-tie differently: check that each token is a
            # maximum of the plain logits up to the rounding of the run
            sequence = list(prompt)
            for token in tokens:
                logits = plain_llama.forward(config, weights, sequence)[-1]
                assert logits[token] >= logits.max() - 0.04 * float(logits.abs().max())
                sequence.append(token)


def test_seeded_temperature_sampling_matches_plain(folders, plain):
    """32-bit run, temperature 0.8, seed 1: the same tokens as the plain chain
    with the same generator (tiny config B of the baseline's workload)."""
    import llm_b200
    config, weights = plain["B"]
    llm = llm_b200.LLM(str(folders["B"]), dtype="float32", device=DEV, context=256, batch=4)
    prompts = [random_tokens(n, config["vocab_size"], 80 + n) for n in (1, 7, 33, 64)]
    got = llm.generate(prompts, max_tokens=12, temperature=0.8, seed=1, stop_tokens=[])
    for i, (prompt, tokens) in enumerate(zip(prompts, got)):
        want, _ = plain_llama.generate(config, weights, prompt, 12, seed=1 + i, temperature=0.8)
        assert tokens == want, i


def test_stop_tokens_and_context_end_sequences(folders, plain):
    import llm_b200
    config, weights = plain["A"]
    llm = llm_b200.LLM(str(folders["A"]), dtype="float32", device=DEV, context=24, batch=2)
    prompt = random_tokens(20, 256, 3)
    free_run, _ = plain_llama.generate(config, weights, prompt, 4, temperature=0.0)
    stop = free_run[2]
    results = llm.generate([prompt, prompt], max_tokens=50, temperature=0.0, stop_tokens=[stop],
                           details=True)
    assert results[0].tokens == free_run[:free_run.index(stop)] and results[0].stop_reason == "eos"
    results = llm.generate([prompt], max_tokens=50, temperature=0.0, stop_tokens=[], details=True)
    want, reason = plain_llama.generate(config, weights, prompt, 50, context=24, temperature=0.0)
    assert results[0].tokens == want and results[0].stop_reason == reason == "context_full"
    llm.engine.cache.check()
    assert llm.engine.cache.slots.n_held == 0


def test_an_engine_refuses_a_model_no_kernel_serves(tmp_path):
    """A head size above the kernels' limit is refused when the engine is built, by name."""
    from llm_b200.config import config_from_dict
    from llm_b200.engine import Engine, load_model
    from llm_b200.errors import LlmError
    from llm_b200.weights import write_random_model
    raw = dict(CONFIGS["A"][0])
    raw["head_dim"] = 272
    folder = tmp_path / "wide_heads"
    write_random_model(folder, config_from_dict(raw), 0, torch.bfloat16)
    for dtype in DTYPES:
        with pytest.raises(LlmError, match="head_dim 272 exceeds 256"):
            Engine(load_model(folder, dtype, DEV), max_tokens=256)


def test_captured_steps_are_dropped_and_captured_again(folders, plain, monkeypatch):
    """With room for two captured shapes only, a batch that shrinks from four sequences to one
    (four shapes) and a second batch after it still decode right: a dropped shape runs plain again
    until it is captured anew."""
    from llm_b200.engine import Entry, step
    monkeypatch.setattr(step, "MAX_GRAPHS", 2)
    config, weights = plain["D"]
    engine = engine_for(folders["D"], torch.bfloat16, max_slots=4)
    for round_ in range(2):
        seqs = [random_tokens(6 + 8 * (b + 1), config["vocab_size"], 50 + 10 * round_ + b) for b in range(4)]
        expected = [plain_llama.forward(config, weights, s) for s in seqs]
        slots = engine.acquire(4)
        engine.step([Entry(s, q[:6], []) for s, q in zip(slots, seqs)])
        live = [0, 1, 2, 3]
        for k in range(6, max(len(s) for s in seqs)):
            ended = [b for b in live if k >= len(seqs[b])]
            engine.release([slots[b] for b in ended])
            live = [b for b in live if b not in ended]
            logits = engine.step([Entry(slots[b], [seqs[b][k]], [0]) for b in live])
            for row, b in enumerate(live):
                assert close(logits[row], expected[b][k], torch.bfloat16), (round_, b, k)
        engine.release([slots[b] for b in live])
        assert len(engine._graphs) <= 2
    engine.cache.check()


def test_a_context_of_a_power_of_two_ends_in_the_bucket_it_decodes_in(folders, plain):
    """Captured decode steps are keyed by the batch size and a bucket of pages (2^(k-1), 2^k]: a
    sequence that decodes from position 130 (three pages) to 256 (four pages, a whole power of two)
    is captured once, every later step is a replay, and the logits are right on both sides of the
    page edge."""
    from llm_b200.engine import Entry, step
    config, weights = plain["C"]
    engine = engine_for(folders["C"], torch.bfloat16, max_slots=1)
    tokens = random_tokens(256, config["vocab_size"], 77)
    expected = plain_llama.forward(config, weights, tokens)
    slot, = engine.acquire(1)
    engine.step([Entry(slot, tokens[:130], [])])
    for k in range(130, 256):
        logits = engine.step([Entry(slot, [tokens[k]], [0])])
        if k in (130, 191, 192, 193, 255):
            assert close(logits[0], expected[k], torch.bfloat16), k
    assert len(engine._graphs) == 1
    assert engine.graph_replays == 126 - step.GRAPH_AFTER_STEPS
    engine.release([slot])
    engine.cache.check()


def test_the_device_generator_equals_its_plain_statement_bit_for_bit():
    import numpy as np
    import plain_random
    from llm_b200.weights.random_init import normal_, tensor_key
    for seed, name, n in ((0, "model.embed_tokens.weight", 70001), (5, "w", 1 << 18)):
        key = tensor_key(seed, name)
        want = plain_random.normal(key, n, 0.0, 0.02)
        got = normal_(torch.empty(n, device=DEV), key, 0.0, 0.02).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        half = normal_(torch.empty(n, dtype=torch.bfloat16, device=DEV), key, 1.0, 0.02).cpu()
        host = normal_(torch.empty(n, dtype=torch.bfloat16), key, 1.0, 0.02)
        assert torch.equal(half.view(torch.int16), host.view(torch.int16))


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_model_made_on_the_device_equals_the_folder_of_the_same_seed(tmp_path, dtype):
    """The benchmarks run on `random_model`; it must be the model that `write_random_model`
    writes and `load_model` binds: equal logits to the last bit, through the same kernels."""
    from llm_b200.config import config_from_dict
    from llm_b200.engine import Engine, Entry, load_model, random_model
    from llm_b200.weights import write_random_model
    config = config_from_dict(dict(CONFIGS["D"][0]))
    folder = write_random_model(tmp_path / "m", config, seed=11, std=0.05)
    tokens = random_tokens(70, config.vocab_size, 3)
    logits = []
    for model in (load_model(folder, dtype, DEV), random_model(config, 11, dtype, DEV, std=0.05)):
        engine = Engine(model, max_tokens=256)
        (slot,) = engine.acquire()
        logits.append(engine.step([Entry(slot, tokens, list(range(70)))]))
    assert torch.equal(logits[0], logits[1])
    config_plain, weights = plain_llama.read_model_folder(folder)
    assert close(logits[1], plain_llama.forward(config_plain, weights, tokens), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["D", "F"])
@pytest.mark.parametrize("options", [dict(step_tokens=48), dict(pass_tokens=100), dict(step_tokens=130, pass_tokens=200)])
def test_prompts_cut_into_passes(folders, plain, dtype, which, options):
    """A batch of three prompts (300, 70 and 129 tokens) with at most 48 new tokens of a sequence
    a pass, or at most 100 tokens a pass in all: continued prompts run through the prefill
    attention kernels and the products at starts that are no multiples of a tile, and the logits
    of every place come back in the caller's order."""
    config, weights = plain[which]
    engine = engine_for(folders[which], dtype, **options)
    seqs = [random_tokens(n, config["vocab_size"], 300 + n) for n in (300, 70, 129)]
    wants = [list(range(0, 300, 7)) + [299], [69, 0, 47, 48], list(range(100, 129))]
    slots = engine.acquire(3)
    logits = engine.step([(s, t, w) for s, t, w in zip(slots, seqs, wants)])
    row = 0
    for t, w in zip(seqs, wants):
        expected = plain_llama.forward(config, weights, t)
        assert close(logits[row:row + len(w)], expected[w], dtype)
        row += len(w)
    assert row == logits.shape[0]
    engine.release(slots)
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["B", "D", "F"])
def test_a_mixed_step(folders, plain, dtype, which):
    """Two sequences bring one token while a third brings 70 tokens onto a slot that already holds
    50 (what the last pass of a cut batch looks like), then all three decode."""
    config, weights = plain[which]
    engine = engine_for(folders[which], dtype)
    seqs = [random_tokens(n, config["vocab_size"], 400 + n) for n in (83, 40, 122)]
    expected = [plain_llama.forward(config, weights, t) for t in seqs]
    slots = engine.acquire(3)
    first = engine.step([(slots[0], seqs[0][:81], [80]), (slots[1], seqs[1][:38], [37]),
                         (slots[2], seqs[2][:50], [49])])
    assert close(first, torch.stack([expected[0][80], expected[1][37], expected[2][49]]), dtype)
    mixed = engine.step([(slots[0], [seqs[0][81]], [0]), (slots[2], seqs[2][50:120], [0, 35, 69]),
                         (slots[1], [seqs[1][38]], [0])])
    assert close(mixed, torch.stack([expected[0][81], expected[2][50], expected[2][85], expected[2][119],
                                     expected[1][38]]), dtype)
    last = engine.step([(slots[0], [seqs[0][82]], [0]), (slots[1], [seqs[1][39]], [0]),
                        (slots[2], [seqs[2][120]], [0])])
    assert close(last, torch.stack([expected[0][82], expected[1][39], expected[2][120]]), dtype)
    engine.release(slots)
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_family_size_layers_against_the_plain_implementation(tmp_path, dtype):
    """The layer sizes of a Llama-3.1-8B (hidden 4096, 32 heads over 8 kv heads of 128,
    feed-forward 14336, vocabulary 128256, llama3 rope scaling), 2 of its 32 layers plus the head,
    with the weights the benchmark runs on (seed 0, N(0, 0.02)), written to a folder and read
    back: a 64-token prompt and 8 greedy decode steps. 32-bit: logits within 1e-3 of the plain
    implementation on the CPU and the same greedy tokens; bfloat16: the usual tolerance."""
    from llm_b200.config import config_from_dict
    from llm_b200.engine import Engine, Entry, load_model
    from llm_b200.shapes import shape
    from llm_b200.weights import write_random_model
    config = config_from_dict(shape("llama-3.1-8b", 2))
    folder = write_random_model(tmp_path / "family", config, seed=0)
    engine = Engine(load_model(folder, dtype, DEV), max_tokens=128)
    prompt = random_tokens(64, config.vocab_size, 17)
    (slot,) = engine.acquire()
    rows = [engine.step([Entry(slot, prompt, [63])])]
    tokens = list(prompt)
    for _ in range(8):
        tokens.append(int(rows[-1][0].argmax()))
        rows.append(engine.step([Entry(slot, [tokens[-1]], [0])]))
    got = torch.cat(rows).cpu()
    del engine
    torch.cuda.empty_cache()
    config_plain, weights = plain_llama.read_model_folder(folder)
    want = plain_llama.forward(config_plain, weights, tokens)[63:]
    if dtype == torch.float32:
        assert float((got - want).abs().max()) <= 1e-3
        assert [int(r.argmax()) for r in want[:-1]] == tokens[64:]
    else:
        assert close(got, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["B", "F"])
def test_passes_walked_from_their_record_equal_plain_passes(folders, plain, dtype, which):
    """The second pass of a shape is recorded, later ones are made again by the native host library
    from that record. Chunks of equal size of different prompts at different positions, on
    different slots and pages, through a record and without one: bit-equal logits, and equal to
    the plain implementation. A pass of another shape in between leaves the record valid."""
    config, weights = plain[which]
    recorded = engine_for(folders[which], dtype, step_tokens=40)
    direct = engine_for(folders[which], dtype, step_tokens=40, use_graphs=False)
    direct.use_records = False
    seqs = [random_tokens(160, config["vocab_size"], 500 + i) for i in range(3)]
    for round_index, tokens in enumerate(seqs):
        expected = plain_llama.forward(config, weights, tokens)
        if round_index == 1:
            filler = recorded.acquire(2)                 # other slots and pages for the next round
        (slot,), (other,) = recorded.acquire(), direct.acquire()
        want = list(range(0, 160, 3))
        got = recorded.step([(slot, tokens, want)])      # four passes of 40 tokens
        same = direct.step([(other, tokens, want)])
        assert torch.equal(got, same)
        assert close(got, expected[want], dtype)
        if round_index == 0:
            recorded.step([(slot, [tokens[0]] * 7, [6])])        # another shape in between
            direct.step([(other, [tokens[0]] * 7, [6])])
        recorded.release([slot])
        direct.release([other])
    assert recorded.records_run >= 8 and direct.records_run == 0
    recorded.cache.check()
