"""Each part of a layer alone (norm, position encoding, mixer, feed-forward, block),
built from a spec with sizes of its own and compared with the plain functions, in
32-bit and in bfloat16. The mixer runs a prompt step and then two decode steps on a
cache made for it alone."""
import math

import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def close(got, want, dtype, scale=None):
    scale = scale or max(1.0, float(want.abs().max()))
    limit = 2e-4 if dtype == torch.float32 else 0.03
    return float((got.float().cpu() - want).abs().max()) <= limit * scale


def tensors_for(part, seed, std=0.1):
    from llm_b200.weights import random_tensors
    return random_tensors(part.parameters(), seed, torch.bfloat16, std=std)


def make_context(cache, slots, counts, dtype):
    """What Engine builds for a step, for parts that run without an engine."""
    from llm_b200.parts import StepContext
    tok_pos, tok_seq, cu, lens, starts = [], [], [0], [], []
    for b, (slot, n) in enumerate(zip(slots, counts)):
        start = cache.length(slot)
        cache.reserve(slot, start + n)
        tok_pos += range(start, start + n)
        tok_seq += [b] * n
        cu.append(cu[-1] + n)
        lens.append(start + n)
        starts.append(start)
    as_dev = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    ctx = StepContext(
        n_tokens=len(tok_pos), n_seqs=len(slots), dtype=dtype, device=torch.device(DEV),
        tok_pos=as_dev(tok_pos), tok_seq=as_dev(tok_seq), cu_seqlens=as_dev(cu), seq_lens=as_dev(lens),
        slot_ids=as_dev(slots), cache=cache,
        block_tables=[cache.block_table_rows(g, slots).to(DEV) for g in range(len(cache.groups))],
        decode=all(n == 1 for n in counts), new_counts=list(counts), starts=starts, max_len=max(lens))
    for slot, n in zip(slots, lens):
        cache.set_length(slot, n)
    return ctx


@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_part(dtype):
    from llm_b200.parts import build_norm
    from llm_b200.parts.spec import NormSpec
    norm = build_norm(NormSpec(200, 3e-4, "n.weight"))
    w = tensors_for(norm, 1)
    norm.bind(dict(w), dtype, DEV)
    x = torch.randn(9, 200, generator=torch.Generator().manual_seed(2)) * 4
    want = P.rms_norm(x, w["n.weight"].float(), 3e-4)
    assert close(norm.forward(x.to(DEV), dtype), want, dtype)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    assert close(norm.forward(x.to(DEV), dtype, rows=rows), want[[8, 0, 3]], dtype)


@pytest.mark.parametrize("scaling", [None, {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                                            "high_freq_factor": 4.0,
                                            "original_max_position_embeddings": 32}])
def test_rope_table(scaling):
    from llm_b200.parts import build_position
    from llm_b200.parts.spec import PositionSpec
    spec = PositionSpec(head_dim=48, theta=12345.0, max_positions=300,
                        scaling=tuple(sorted(scaling.items())) if scaling else None)
    rope = build_position(spec)
    assert build_position(spec) is rope                      # equal specs share one table
    rope.prepare(200, DEV)
    inv_freq = P.rope_inverse_frequencies(48, 12345.0, scaling)
    angle = torch.arange(200, dtype=torch.float64)[:, None] * inv_freq[None, :]
    want = torch.cat([angle.cos(), angle.sin()], 1).float()
    assert rope.table.shape == (200, 48) and torch.allclose(rope.table.cpu(), want, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,hidden,bias", [(6, 2, 64, 72, True), (5, 5, 48, 100, False)])
def test_attention_mixer_alone(dtype, heads, kv_heads, dim, hidden, bias):
    from llm_b200.cache import PagedCache
    from llm_b200.parts import build_mixer
    from llm_b200.parts.spec import AttentionSpec, PositionSpec, names
    roles = {r: f"a.{r}.w" for r in "qkvo"}
    if bias:
        roles.update({f"{r}_bias": f"a.{r}.b" for r in "qkvo"})
    spec = AttentionSpec(hidden=hidden, n_heads=heads, n_kv_heads=kv_heads, head_dim=dim,
                         scale=0.7 / math.sqrt(dim), bias=bias, window=0,
                         position=PositionSpec(dim, 30000.0, 512), names=names(**roles))
    mixer = build_mixer(spec)
    w = tensors_for(mixer, 3)
    mixer.bind(dict(w), dtype, DEV)
    mixer.prepare(512, DEV)
    cache = PagedCache([mixer.kv_request()], [None], 1024, 512, 4, dtype, DEV)
    lengths = [70, 3]
    gen = torch.Generator().manual_seed(4)
    hs = [torch.randn(n + 2, hidden, generator=gen) for n in lengths]        # prompt + 2 decode steps

    def plain(h):
        n = h.shape[0]
        wf = {k: v.float() for k, v in w.items()}
        q = h @ wf["a.q.w"].T + (wf["a.q.b"] if bias else 0)
        k = h @ wf["a.k.w"].T + (wf["a.k.b"] if bias else 0)
        v = h @ wf["a.v.w"].T + (wf["a.v.b"] if bias else 0)
        inv_freq = P.rope_inverse_frequencies(dim, 30000.0)
        q = P.rope_rotate(q.view(n, heads, dim), list(range(n)), inv_freq)
        k = P.rope_rotate(k.view(n, kv_heads, dim), list(range(n)), inv_freq)
        a = P.causal_attention(q, k, v.view(n, kv_heads, dim), spec.scale).reshape(n, heads * dim)
        return a @ wf["a.o.w"].T + (wf["a.o.b"] if bias else 0)

    want = [plain(h.to(dtype).float()) for h in hs]
    slots = [cache.acquire(), cache.acquire()]
    ctx = make_context(cache, slots, lengths, dtype)
    h = torch.cat([x[:n] for x, n in zip(hs, lengths)]).to(DEV).to(dtype)
    residual = torch.zeros(sum(lengths), hidden, device=DEV)
    mixer.forward(h, ctx, 0, 0, residual)
    assert close(residual, torch.cat([wnt[:n] for wnt, n in zip(want, lengths)]), dtype)
    for k in range(2):
        ctx = make_context(cache, slots, [1, 1], dtype)
        h = torch.stack([x[n + k] for x, n in zip(hs, lengths)]).to(DEV).to(dtype)
        residual = torch.full((2, hidden), 5.0, device=DEV)                 # the part adds, never overwrites
        mixer.forward(h, ctx, 0, 0, residual)
        assert close(residual - 5.0, torch.stack([wnt[n + k] for wnt, n in zip(want, lengths)]), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,inter", [(72, 208), (100, 172)])
def test_gated_mlp_alone(dtype, hidden, inter):
    from llm_b200.parts import build_feed_forward
    from llm_b200.parts.spec import GatedMlpSpec, names
    ffn = build_feed_forward(GatedMlpSpec(hidden, inter, "silu", names(gate="f.g", up="f.u", down="f.d")))
    w = tensors_for(ffn, 5)
    ffn.bind(dict(w), dtype, DEV)
    assert ffn.fused == (dtype == torch.bfloat16 and inter % 16 == 0 and hidden % 8 == 0)
    for n in (1, 70, 200):
        h = torch.randn(n, hidden, generator=torch.Generator().manual_seed(n))
        want = P.gated_mlp(h.to(dtype).float(), w["f.g"].float(), w["f.u"].float(), w["f.d"].float())
        residual = torch.ones(n, hidden, device=DEV)
        from types import SimpleNamespace
        ffn.forward(h.to(DEV).to(dtype), SimpleNamespace(scratch=lambda name, shape=None, dtype=None: None, extras={}), residual)
        assert close(residual - 1.0, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_pre_norm_block_alone(dtype):
    from llm_b200.cache import PagedCache
    from llm_b200.parts import build_block
    from llm_b200.parts.spec import (AttentionSpec, BlockSpec, GatedMlpSpec, NormSpec, PositionSpec, names)
    hidden, heads, kv_heads, dim = 64, 4, 1, 32
    mixer = AttentionSpec(hidden, heads, kv_heads, dim, 1 / math.sqrt(dim), False, 0,
                          PositionSpec(dim, 10000.0, 256, pairing="interleaved"),
                          names(q="q", k="k", v="v", o="o"))
    spec = BlockSpec(NormSpec(hidden, 1e-5, "n1"), mixer, NormSpec(hidden, 1e-6, "n2"),
                     GatedMlpSpec(hidden, 96, "silu", names(gate="g", up="u", down="d")))
    block = build_block(spec)
    w = tensors_for(block, 6)
    block.bind(dict(w), dtype, DEV)
    block.prepare(256, DEV)
    cache = PagedCache([block.mixer.kv_request()], [None], 512, 256, 2, dtype, DEV)
    n = 90
    x = torch.randn(n, hidden, generator=torch.Generator().manual_seed(7))
    wf = {k: v.float() for k, v in w.items()}
    h = P.rms_norm(x, wf["n1"], 1e-5)
    inv_freq = P.rope_inverse_frequencies(dim, 10000.0)
    q = P.rope_rotate((h @ wf["q"].T).view(n, heads, dim), list(range(n)), inv_freq, "interleaved")
    k = P.rope_rotate((h @ wf["k"].T).view(n, kv_heads, dim), list(range(n)), inv_freq, "interleaved")
    a = P.causal_attention(q, k, (h @ wf["v"].T).view(n, kv_heads, dim), 1 / math.sqrt(dim))
    want = x + a.reshape(n, heads * dim) @ wf["o"].T
    want = want + P.gated_mlp(P.rms_norm(want, wf["n2"], 1e-6), wf["g"], wf["u"], wf["d"])
    ctx = make_context(cache, [cache.acquire()], [n], dtype)
    got = x.to(DEV).clone()
    block.forward(got, ctx, 0, 0)
    assert close(got, want, dtype)
