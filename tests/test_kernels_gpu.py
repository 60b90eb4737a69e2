"""Every CUDA kernel alone against its plain PyTorch statement (tests/plain_ops.py),
at sizes other than the tiny models': widths that are no power of two, head
sizes 16 to 256, group sizes 1 to 8, shuffled pages, a window, and inputs made
so that a wrong key, page or row shows."""
import math

import pytest
import torch

import plain_ops

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    import llm_b200.ops as o
    return o


def tol(dtype, scale=1.0):
    return dict(atol=(2e-5 if dtype == torch.float32 else 2e-2) * scale,
                rtol=1e-5 if dtype == torch.float32 else 2e-2)


def randn(*shape, dtype=torch.float32, seed=0, scale=1.0):
    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=gen) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(dtype):
    table = randn(301, 72, dtype=dtype)
    tokens = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    assert torch.equal(ops().embed(tokens, table), plain_ops.embed(tokens, table))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [64, 96, 1000, 4096])
def test_rmsnorm(dtype, hidden):
    x = randn(7, hidden, seed=1, scale=3.0)
    x[3] *= 1e-3                         # a row where eps matters
    gain = 1.0 + randn(hidden, seed=2, scale=0.1)
    rows = torch.tensor([6, 0, 3, 3], dtype=torch.int32, device=DEV)
    for r in (None, rows):
        got = ops().rmsnorm(x, gain, 1e-5, dtype, r)
        want = plain_ops.rmsnorm(x, gain, 1e-5, dtype, r)
        assert torch.allclose(got.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    gu = randn(5, 2 * 172, dtype=dtype, seed=3, scale=2.0)
    got = ops().swiglu(gu)
    assert torch.allclose(got.float(), plain_ops.swiglu(gu).float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 96, 64), (7, 172, 64), (65, 100, 172), (129, 384, 96),
                                   (193, 130, 250), (33, 1000, 80)])
def test_linear(dtype, m, n, k):
    a = randn(m, k, dtype=dtype, seed=4)
    w = randn(n, k, dtype=dtype, seed=5, scale=0.1)
    bias = randn(n, seed=6)
    got = ops().linear(a, w, bias)
    want = plain_ops.linear(a, w, bias)
    assert torch.allclose(got.float(), want.float(), **tol(dtype, math.sqrt(k) / 8))
    # 32-bit output (the head) and accumulation into the residual stream
    got32 = ops().linear(a, w, out_dtype=torch.float32)
    assert torch.allclose(got32, plain_ops.linear(a, w, out_dtype=torch.float32), **tol(torch.float32, math.sqrt(k)))
    residual = randn(m, n, seed=7)
    expect = plain_ops.linear(a, w, bias, residual=residual.clone())
    ops().linear(a, w, bias, residual=residual)
    assert torch.allclose(residual, expect, **tol(torch.float32, math.sqrt(k)))


@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (8, 6144, 4096), (8, 1000, 200), (5, 72, 1032),
                                   (16, 4096, 14336), (17, 100, 1024), (33, 520, 2048),
                                   (64, 4100, 4096)])
@pytest.mark.parametrize("variant", ["gemm_skinny", "gemm_tc"])
def test_linear_decode_kernel(m, n, k, variant):
    """The split-K decode products (mma.sync and tcgen05): sizes with one and many
    splits, tails in N, K and M, called twice so that the tile counters must have
    been left at zero."""
    from llm_b200.ops import tactics
    if variant == "gemm_skinny":
        tactics.disable("gemm_tc")
    try:
        assert tactics.choose_linear(m, n, k, torch.bfloat16, torch.bfloat16, k) == variant
        _check_decode_product(m, n, k)
        assert ops().tensor_core_status() == 0
    finally:
        tactics.enable("gemm_tc")


def _check_decode_product(m, n, k):
    a = randn(m, k, dtype=torch.bfloat16, seed=80)
    w = randn(n, k, dtype=torch.bfloat16, seed=81, scale=0.05)
    bias = randn(n, seed=82)
    want = plain_ops.linear(a, w, bias, out_dtype=torch.float32)
    scale = float(want.abs().max())
    for _ in range(2):
        got = ops().linear(a, w, bias, out_dtype=torch.float32)
        assert float((got - want).abs().max()) <= 2e-3 * scale
    got16 = ops().linear(a, w, bias)
    assert float((got16.float() - want).abs().max()) <= 1e-2 * scale
    residual = randn(m, n, seed=83)
    expect = residual + want
    ops().linear(a, w, bias, residual=residual)
    assert float((residual - expect).abs().max()) <= 2e-3 * scale
    # the same rows alone and in the batch: the same split and order, bit-equal
    alone = ops().linear(a[:1].contiguous(), w, bias, out_dtype=torch.float32)
    assert torch.equal(alone[0], got[0])


@pytest.mark.parametrize("m,n,k", [(65, 256, 64), (128, 128, 128), (129, 300, 200), (200, 1000, 520),
                                   (513, 6144, 4096), (2048, 4096, 1024), (70, 72, 72),
                                   (300, 4104, 2048), (256, 4096, 4096), (1000, 2304, 1536),
                                   (140, 19200, 128), (2500, 8192, 192)])
def test_linear_tensor_core_kernel(m, n, k):
    """tcgen05 product for more than 64 tokens: tile edges in M, N and K. Shapes with few output
    tiles run with the weights on the 128-row side, several token tiles and split K (513 x 6144,
    300 x 4104), the others as 256 x 256 tiles on pairs of SMs (2048 x 4096)."""
    from llm_b200.ops import tactics
    assert tactics.choose_linear(m, n, k, torch.bfloat16, torch.bfloat16, k) == "gemm_tc"
    a = randn(m, k, dtype=torch.bfloat16, seed=84)
    w = randn(n, k, dtype=torch.bfloat16, seed=85, scale=0.05)
    bias = randn(n, seed=86)
    want = plain_ops.linear(a, w, bias, out_dtype=torch.float32)
    scale = float(want.abs().max())
    got = ops().linear(a, w, bias, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert ops().tensor_core_status() == 0
    assert float((got - want).abs().max()) <= 2e-3 * scale
    got16 = ops().linear(a, w, bias)
    assert float((got16.float() - want).abs().max()) <= 1e-2 * scale
    residual = randn(m, n, seed=87)
    expect = residual + want
    ops().linear(a, w, bias, residual=residual)
    assert float((residual - expect).abs().max()) <= 2e-3 * scale
    # a strided view as input (the query part of a fused projection)
    wide = randn(m, k + 64, dtype=torch.bfloat16, seed=88)
    view = wide[:, :k]
    got = ops().linear(view, w, out_dtype=torch.float32)
    assert float((got - plain_ops.linear(view, w, out_dtype=torch.float32)).abs().max()) <= 2e-3 * scale


@pytest.mark.parametrize("m,f,k", [(1, 64, 64), (8, 14336, 4096), (5, 208, 72), (64, 320, 128),
                                   (70, 320, 128), (300, 1024, 520), (2048, 1024, 256),
                                   (8, 320, 1024), (40, 320, 1024), (512, 2048, 2048)])
def test_linear_with_gated_epilogue(m, f, k):
    """silu(gate) * up in the epilogue of the tensor-core product, both orientations,
    against the product followed by the plain activation. The last two shapes split K: the
    activation is then applied where the splits are summed (by the last block of a tile at 8
    tokens, by the sum kernel at 40)."""
    a = randn(m, k, dtype=torch.bfloat16, seed=96)
    gate = randn(f, k, dtype=torch.bfloat16, seed=97, scale=0.1)
    up = randn(f, k, dtype=torch.bfloat16, seed=98, scale=0.1)
    mixed = torch.stack([gate.view(-1, 16, k), up.view(-1, 16, k)], dim=1).reshape(2 * f, k).contiguous()
    assert ops().glu_fusable(2 * f, k, torch.bfloat16)
    got = ops().linear(a, mixed, glu=True)
    g, u = a.float() @ gate.float().T, a.float() @ up.float().T
    want = g / (1 + torch.exp(-g)) * u
    assert got.shape == (m, f)
    assert torch.allclose(got.float(), want, atol=2e-2 * float(want.abs().max()), rtol=2e-2)
    assert torch.allclose(plain_ops.linear(a, mixed, glu=True).float(), want, atol=1e-2 * float(want.abs().max()), rtol=2e-2)
    assert ops().tensor_core_status() == 0


def test_linear_rows_do_not_depend_on_the_batch():
    """32-bit: a row's product is bit-equal whether it is computed alone or among 200 rows."""
    a = randn(200, 172, seed=8)
    w = randn(300, 172, seed=9)
    whole = ops().linear(a, w)
    for row in (0, 63, 64, 199):
        assert torch.equal(ops().linear(a[row:row + 1].contiguous(), w)[0], whole[row])


def make_cache(n_seqs, lens, n_kv_heads, head_dim, dtype, seed, ring_pages=None):
    """A shuffled page pool, block tables, and keys/values written position by position."""
    width = ring_pages or max((n + 63) // 64 for n in lens) + 1
    n_pages = n_seqs * width + 3
    gen = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=gen)
    table = perm[:n_seqs * width].view(n_seqs, width).to(torch.int32).to(DEV)
    k_cache = torch.full((n_pages, n_kv_heads, 64, head_dim), 7.0, dtype=dtype, device=DEV)
    v_cache = torch.full((n_pages, n_kv_heads, 64, head_dim), -9.0, dtype=dtype, device=DEV)
    return table, width, k_cache, v_cache


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,interleaved", [(4, 2, 16, False), (3, 1, 32, True),
                                                            (8, 8, 64, False), (16, 2, 128, False),
                                                            (2, 1, 256, False), (6, 2, 48, False)])
def test_rope_cache_write(dtype, heads, kv_heads, dim, interleaved):
    starts, counts = [0, 70, 5], [9, 1, 130]
    lens = [s + c for s, c in zip(starts, counts)]
    table, width, k_cache, v_cache = make_cache(3, lens, kv_heads, dim, dtype, 10)
    tok_pos = torch.tensor([p for s, c in zip(starts, counts) for p in range(s, s + c)],
                           dtype=torch.int32, device=DEV)
    tok_seq = torch.tensor([b for b, c in enumerate(counts) for _ in range(c)],
                           dtype=torch.int32, device=DEV)
    n = tok_pos.numel()
    qkv = randn(n, (heads + 2 * kv_heads) * dim, dtype=dtype, seed=11)
    angle = torch.arange(256, dtype=torch.float64)[:, None] * (
        10000.0 ** (-2.0 * torch.arange(dim // 2, dtype=torch.float64) / dim))[None, :]
    rope = torch.cat([angle.cos(), angle.sin()], 1).float().to(DEV)
    expect_qkv, expect_k, expect_v = qkv.clone(), k_cache.clone(), v_cache.clone()
    plain_ops.rope_cache_write(expect_qkv, rope, tok_pos, tok_seq, table, width, expect_k,
                               expect_v, heads, kv_heads, dim, interleaved)
    ops().rope_cache_write(qkv, rope, tok_pos, tok_seq, table, width, k_cache, v_cache, heads,
                           kv_heads, dim, interleaved)
    t = tol(dtype)
    assert torch.allclose(qkv.float(), expect_qkv.float(), **t)
    assert torch.allclose(k_cache.float(), expect_k.float(), **t)     # untouched rows keep 7.0
    assert torch.allclose(v_cache.float(), expect_v.float(), **t)
    # without a table nothing turns; without write_cache the cache stays
    q2, k2, v2 = qkv.clone(), k_cache.clone(), v_cache.clone()
    ops().rope_cache_write(q2, None, tok_pos, tok_seq, table, width, k2, v2, heads, kv_heads, dim,
                           interleaved, write_cache=False)
    assert torch.equal(q2, qkv) and torch.equal(k2, k_cache) and torch.equal(v2, v_cache)


def fill_cache(table, width, k_cache, v_cache, lens, seed):
    """Random keys and values at every position < len of every sequence."""
    kv_heads, dim = k_cache.shape[1], k_cache.shape[3]
    keys, values = [], []
    for b, n in enumerate(lens):
        k = randn(n, kv_heads, dim, seed=seed + 2 * b)
        v = randn(n, kv_heads, dim, seed=seed + 2 * b + 1)
        pos = torch.arange(n, device=DEV)
        pages = table[b].long()[(pos // 64) % width]
        k_cache[pages, :, pos % 64, :] = k.to(k_cache.dtype)
        v_cache[pages, :, pos % 64, :] = v.to(v_cache.dtype)
        keys.append(k)
        values.append(v)
    return keys, values


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,window", [(4, 2, 16, 0), (3, 1, 32, 0), (8, 1, 64, 0),
                                                       (8, 2, 128, 0), (2, 2, 256, 0),
                                                       (6, 2, 48, 0), (4, 2, 32, 37)])
def test_attention_prefill_and_decode(dtype, heads, kv_heads, dim, window):
    lens = [130, 1, 77, 300]
    table, width, k_cache, v_cache = make_cache(4, lens, kv_heads, dim, dtype, 20)
    fill_cache(table, width, k_cache, v_cache, lens, 21)
    scale = 1.0 / math.sqrt(dim)
    # prefill: every position of every sequence is a query
    tok_pos = torch.tensor([p for n in lens for p in range(n)], dtype=torch.int32, device=DEV)
    tok_seq = torch.tensor([b for b, n in enumerate(lens) for _ in range(n)], dtype=torch.int32, device=DEV)
    qkv = randn(tok_pos.numel(), (heads + 2 * kv_heads) * dim, dtype=dtype, seed=22)
    got = ops().attention(qkv, k_cache, v_cache, table, width, tok_pos, tok_seq, heads, kv_heads,
                          dim, scale, window)
    want = plain_ops.attention(qkv, k_cache, v_cache, table, width, tok_pos, tok_seq, heads,
                               kv_heads, dim, scale, window)
    assert torch.allclose(got.float(), want.float(), **tol(dtype))
    # decode: one query per sequence at its last position
    last = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    seqs = torch.arange(4, dtype=torch.int32, device=DEV)
    q1 = randn(4, (heads + 2 * kv_heads) * dim, dtype=dtype, seed=23)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    got = ops().attention(q1, k_cache, v_cache, table, width, last, seqs, heads, kv_heads, dim,
                          scale, window, decode=True, seq_lens=seq_lens, max_len=max(lens))
    want = plain_ops.attention(q1, k_cache, v_cache, table, width, last, seqs, heads, kv_heads,
                               dim, scale, window)
    assert torch.allclose(got.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("heads,kv_heads,dim", [(32, 8, 128), (8, 1, 64), (6, 2, 96), (4, 4, 32),
                                                (3, 1, 128)])
@pytest.mark.parametrize("forced_slices", [0, 1, 2, 16])
def test_attention_decode_kernel_long_contexts(heads, kv_heads, dim, forced_slices, monkeypatch):
    """The split-KV decode kernel at lengths from 1 to 3000 in one batch (page edges,
    empty slices, many slices), twice in a row on the same scratch; with the library's own
    choice of slices and with forced counts (one slice writes the result without the
    combining kernel)."""
    if forced_slices:
        monkeypatch.setenv("LLMB_DECODE_SPLITS", str(forced_slices))
    from llm_b200.ops import tactics
    dtype = torch.bfloat16
    assert tactics.choose_attention(True, dtype, heads, kv_heads, dim, 0) == "attention_decode"
    lens = [3000, 1, 64, 65, 1000, 127]
    table, width, k_cache, v_cache = make_cache(len(lens), lens, kv_heads, dim, dtype, 90)
    fill_cache(table, width, k_cache, v_cache, lens, 91)
    last = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    seqs = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    q = randn(len(lens), (heads + 2 * kv_heads) * dim, dtype=dtype, seed=92)
    want = plain_ops.attention(q, k_cache, v_cache, table, width, last, seqs, heads, kv_heads, dim,
                               dim ** -0.5)
    longest_first = torch.tensor(sorted(range(len(lens)), key=lambda b: -lens[b]), dtype=torch.int32, device=DEV)
    for order in (None, longest_first):          # the second call also takes the sequences longest first
        got = ops().attention(q, k_cache, v_cache, table, width, last, seqs, heads, kv_heads, dim,
                              dim ** -0.5, 0, decode=True, seq_lens=seq_lens, max_len=max(lens),
                              seq_order=order)
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("heads,kv_heads,dim", [(8, 2, 128), (4, 1, 64), (6, 2, 96), (4, 4, 32),
                                                (3, 1, 128)])
@pytest.mark.parametrize("variant", ["attention_prefill", "attention_prefill_tc"])
def test_attention_prefill_kernel(heads, kv_heads, dim, variant):
    """The flash prefill kernels (mma.sync and tcgen05): sequences that start at position 0
    and sequences that continue (chunked prompts), lengths around tile and page edges."""
    from llm_b200.ops import tactics
    if variant == "attention_prefill_tc" and dim not in (64, 128):
        pytest.skip("the tcgen05 kernel serves head sizes 64 and 128")
    if variant == "attention_prefill":
        tactics.disable("attention_prefill_tc")
    try:
        assert tactics.choose_attention(False, torch.bfloat16, heads, kv_heads, dim, 0, True) == variant
        _check_prefill_attention(heads, kv_heads, dim)
        ops().check_device_status()
    finally:
        tactics.enable("attention_prefill_tc")


def _check_prefill_attention(heads, kv_heads, dim):
    dtype = torch.bfloat16
    starts, counts = [0, 0, 100, 64, 0, 300], [300, 1, 65, 64, 63, 130]
    lens = [s + c for s, c in zip(starts, counts)]
    table, width, k_cache, v_cache = make_cache(len(lens), lens, kv_heads, dim, dtype, 93)
    fill_cache(table, width, k_cache, v_cache, lens, 94)
    tok_pos = torch.tensor([p for s, c in zip(starts, counts) for p in range(s, s + c)],
                           dtype=torch.int32, device=DEV)
    tok_seq = torch.tensor([b for b, c in enumerate(counts) for _ in range(c)], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    q = randn(tok_pos.numel(), (heads + 2 * kv_heads) * dim, dtype=dtype, seed=95)
    want = plain_ops.attention(q, k_cache, v_cache, table, width, tok_pos, tok_seq, heads, kv_heads,
                               dim, dim ** -0.5)
    longest_first = torch.tensor(sorted(range(len(lens)), key=lambda b: -lens[b]), dtype=torch.int32, device=DEV)
    for order in (None, longest_first):
        got = ops().attention(q, k_cache, v_cache, table, width, tok_pos, tok_seq, heads, kv_heads, dim,
                              dim ** -0.5, 0, seq_lens=seq_lens, max_len=max(lens), cu_seqlens=cu,
                              max_new=max(counts), seq_order=order)
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        # and relative to each row's norm: random softmax outputs are small, a lost key must show
        g, w = got.float().view(-1, heads, dim), want.float().view(-1, heads, dim)
        relative = (g - w).norm(dim=-1) / w.norm(dim=-1).clamp_min(1e-3)
        assert float(relative.max()) < 0.03


@pytest.mark.parametrize("variant", ["attention_prefill", "attention_prefill_tc"])
@pytest.mark.parametrize("dim", [64, 128])
def test_attention_prefill_growing_scores(variant, dim):
    """Keys grow from one block of 128 to the next, first a little and then by much, so that a
    row's running maximum moves late in the sequence: by less than the kernel's threshold for
    rescaling (probabilities above one) and by far more (the accumulated output is rescaled)."""
    from llm_b200.ops import tactics
    heads, kv_heads, dtype, n = 4, 2, torch.bfloat16, 700
    if variant == "attention_prefill":
        tactics.disable("attention_prefill_tc")
    try:
        assert tactics.choose_attention(False, dtype, heads, kv_heads, dim, 0, True) == variant
        table, width, k_cache, v_cache = make_cache(1, [n], kv_heads, dim, dtype, 96)
        fill_cache(table, width, k_cache, v_cache, [n], 97)
        for block, factor in enumerate([0.3, 1.0, 1.4, 0.5, 6.0, 2.0]):
            for page in (2 * block, 2 * block + 1):
                if page < width:
                    k_cache[int(table[0, page])] *= factor
        tok_pos = torch.arange(n, dtype=torch.int32, device=DEV)
        tok_seq = torch.zeros(n, dtype=torch.int32, device=DEV)
        cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
        seq_lens = torch.tensor([n], dtype=torch.int32, device=DEV)
        q = randn(n, (heads + 2 * kv_heads) * dim, dtype=dtype, seed=98)
        want = plain_ops.attention(q, k_cache, v_cache, table, width, tok_pos, tok_seq, heads, kv_heads,
                                   dim, dim ** -0.5)
        got = ops().attention(q, k_cache, v_cache, table, width, tok_pos, tok_seq, heads, kv_heads, dim,
                              dim ** -0.5, 0, seq_lens=seq_lens, max_len=n, cu_seqlens=cu, max_new=n)
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        ops().check_device_status()
    finally:
        tactics.enable("attention_prefill_tc")


@pytest.mark.parametrize("variant", ["attention_prefill", "attention_prefill_tc"])
@pytest.mark.parametrize("start,count", [(173, 2), (173, 129), (100, 130), (0, 300)])
def test_prefill_attention_finds_planted_keys(variant, start, count):
    """Random scores over hundreds of keys hide one lost or wrongly masked key, so keys are
    planted: one early key (position 3), the key just before a continued chunk's first token,
    and the chunk's last key. A query that points at a planted key must return that key's value
    (a query in the chunk's last tile, a chunk that starts off the tile and page edges); the query
    one position before the last key must not see it."""
    from llm_b200.ops import tactics
    heads, kv_heads, dim, dtype = 4, 2, 128, torch.bfloat16
    n = start + count
    if variant == "attention_prefill":
        tactics.disable("attention_prefill_tc")
    try:
        assert tactics.choose_attention(False, dtype, heads, kv_heads, dim, 0, True) == variant
        direction = torch.zeros(dim, device=DEV)
        direction[5] = 40.0
        tok_pos = torch.arange(start, n, dtype=torch.int32, device=DEV)
        tok_seq = torch.zeros(count, dtype=torch.int32, device=DEV)
        cu = torch.tensor([0, count], dtype=torch.int32, device=DEV)
        seq_lens = torch.tensor([n], dtype=torch.int32, device=DEV)
        cases = [(3, n - 1, True), (n - 1, n - 1, True)]
        if start > 0:
            cases += [(start - 1, start, True), (start - 1, n - 1, True)]
        if count >= 2:
            cases += [(n - 1, n - 2, False)]
        for key_pos, query_pos, seen in cases:
            table, width, k_cache, v_cache = make_cache(1, [n], kv_heads, dim, dtype, 130)
            keys, values = fill_cache(table, width, k_cache, v_cache, [n], 131)
            k_cache[int(table[0, key_pos // 64]), :, key_pos % 64, :] = direction.to(dtype)
            q = randn(count, (heads + 2 * kv_heads) * dim, dtype=dtype, seed=132, scale=0.1)
            q[query_pos - start, :heads * dim] = direction.repeat(heads).to(dtype)
            got = ops().attention(q, k_cache, v_cache, table, width, tok_pos, tok_seq, heads, kv_heads, dim,
                                  dim ** -0.5, 0, seq_lens=seq_lens, max_len=n, cu_seqlens=cu, max_new=count)
            row = got[query_pos - start].float().view(heads, dim)
            for h in range(heads):
                expect = values[0][key_pos, h // 2].to(dtype).float()
                hit = torch.allclose(row[h], expect, atol=2e-2)
                assert hit == seen, (key_pos, query_pos, h)
        ops().check_device_status()
    finally:
        tactics.enable("attention_prefill_tc")


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key(dtype):
    """Among 500 keys one early key matches the query; the output must be its
    value, and with a window that excludes it, must not be."""
    heads, kv_heads, dim, n = 4, 2, 64, 500
    table, width, k_cache, v_cache = make_cache(1, [n], kv_heads, dim, dtype, 30)
    keys, values = fill_cache(table, width, k_cache, v_cache, [n], 31)
    far = 3
    direction = torch.zeros(dim, device=DEV)
    direction[5] = 40.0
    page = int(table[0, far // 64])
    k_cache[page, :, far % 64, :] = direction.to(dtype)
    qkv = torch.zeros(1, (heads + 2 * kv_heads) * dim, dtype=dtype, device=DEV)
    qkv[0, :heads * dim] = direction.repeat(heads).to(dtype)
    pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = ops().attention(qkv, k_cache, v_cache, table, width, pos, seq, heads, kv_heads, dim,
                          1.0 / math.sqrt(dim), 0, decode=True,
                          seq_lens=torch.tensor([n], dtype=torch.int32, device=DEV), max_len=n)
    got = got.float().view(heads, dim)
    for h in range(heads):
        expect = values[0][far, h // 2].to(dtype).float()
        assert torch.allclose(got[h], expect, atol=2e-2)
    windowed = ops().attention(qkv, k_cache, v_cache, table, width, pos, seq, heads, kv_heads,
                               dim, 1.0 / math.sqrt(dim), 100).float().view(heads, dim)
    assert not torch.allclose(windowed[0], values[0][far, 0].to(dtype).float(), atol=0.1)


def test_attention_window_edge():
    """The key at position p - window is out, the key at p - window + 1 is in."""
    heads, kv_heads, dim, n, window = 2, 1, 32, 200, 64
    dtype = torch.float32
    table, width, k_cache, v_cache = make_cache(1, [n], kv_heads, dim, dtype, 40)
    keys, values = fill_cache(table, width, k_cache, v_cache, [n], 41)
    direction = torch.zeros(dim, device=DEV)
    direction[0] = 50.0
    qkv = torch.zeros(1, (heads + 2) * dim, device=DEV)
    qkv[0, :heads * dim] = direction.repeat(heads)
    pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    for key_pos, inside in ((n - 1 - window, False), (n - window, True)):
        kc = k_cache.clone()
        kc[int(table[0, key_pos // 64]), :, key_pos % 64, :] = direction
        got = ops().attention(qkv, kc, v_cache, table, width, pos, seq, heads, kv_heads, dim,
                              1.0 / math.sqrt(dim), window).view(heads, dim)
        hit = torch.allclose(got[0], values[0][key_pos, 0], atol=1e-3)
        assert hit == inside


def test_argmax_first_maximum_wins():
    logits = randn(5, 1000, seed=50)
    logits[1, 700] = logits[1, 20] = 9.0
    logits[2] = 0.0
    got = ops().argmax_rows(logits)
    assert got.tolist() == plain_ops.argmax_rows(logits).tolist()
    assert got[1] == 20 and got[2] == 0


def _sampler_state(n, params, iparams, seeds, cap=8):
    f = torch.tensor(params, dtype=torch.float32, device=DEV)
    i = torch.tensor(iparams, dtype=torch.int32, device=DEV)
    rng = torch.tensor([(s | 1) - (1 << 64) if (s | 1) >= (1 << 63) else (s | 1) for s in seeds],
                       dtype=torch.int64, device=DEV)
    recent = torch.zeros((n, cap), dtype=torch.int32, device=DEV)
    recent_len = torch.zeros((n,), dtype=torch.int32, device=DEV)
    out = torch.zeros((n,), dtype=torch.int32, device=DEV)
    status = torch.zeros((n,), dtype=torch.int32, device=DEV)
    return f, i, recent, recent_len, rng, out, status


@pytest.mark.parametrize("vocab", [384, 5000, 50001])
def test_sample_rows_matches_plain_chain(vocab):
    """Greedy, temperature with top-k / top-p / min-p, penalty, and no top-k at all:
    the same tokens and generator states as the plain chain, over several draws. 50,001 entries:
    rows that are read four values a load, eight loads ahead, with a tail that is not."""
    params = [[0.0, 0.75, 0.25, 1.0], [0.8, 0.75, 0.25, 1.1], [1.5, 0.95, 0.0, 1.3],
              [1.0, 1.0, 0.0, 1.0], [0.7, 2.0, 0.05, 1.0]]
    iparams = [[40, 64], [40, 64], [7, 4], [0, 0], [0, 0]]
    seeds = [1, 1, 0x5EED1234ABCD0001, 99, 12345]
    n = len(params)
    state_gpu = _sampler_state(n, params, iparams, seeds)
    state_cpu = [t.cpu().clone() for t in state_gpu]
    state_gpu[2][:, :3] = torch.tensor([3, 3, 10], dtype=torch.int32)
    state_cpu[2][:, :3] = torch.tensor([3, 3, 10], dtype=torch.int32)
    state_gpu[3][:] = 3
    state_cpu[3][:] = 3
    for draw in range(6):
        logits = randn(n, vocab, seed=60 + draw, scale=2.5)
        logits[:, 3] = 4.0            # a penalised token that matters
        cpu_logits = logits.cpu().clone()
        ops().sample_rows(logits, *state_gpu)
        plain_ops.sample_rows(cpu_logits, *state_cpu)
        assert state_gpu[5].tolist() == state_cpu[5].tolist(), f"draw {draw}"
        assert state_gpu[4].tolist() == state_cpu[4].tolist()
        assert state_gpu[6].tolist() == [0] * n


def test_sample_rows_records_windows_and_finds_state_by_row():
    """Three logits rows that belong to sequences 4, 0 and 2 of a batch of five: the kernel takes each
    row's parameters, window and generator from its sequence's row, enters the drawn token into that
    window, and leaves the other sequences' state alone; three draws in a row against the plain chain."""
    vocab, n = 777, 5
    params = [[0.9, 0.9, 0.05, 1.2]] * n
    iparams = [[30, 6]] * n
    state_gpu = _sampler_state(n, params, iparams, [11, 12, 13, 14, 15], cap=6)
    state_cpu = [t.cpu().clone() for t in state_gpu]
    rows = torch.tensor([4, 0, 2], dtype=torch.int32)
    out_gpu, out_cpu = torch.zeros(3, dtype=torch.int32, device=DEV), torch.zeros(3, dtype=torch.int32)
    for draw in range(8):                               # more draws than the window holds
        logits = randn(3, vocab, seed=200 + draw, scale=2.0)
        cpu_logits = logits.cpu().clone()
        f, i, recent, recent_len, rng, _, status = state_gpu
        ops().sample_rows(logits, f, i, recent, recent_len, rng, out_gpu, status, record=True,
                          state_rows=rows.to(DEV))
        f, i, recent, recent_len, rng, _, status = state_cpu
        plain_ops.sample_rows(cpu_logits, f, i, recent, recent_len, rng, out_cpu, status, record=True,
                              state_rows=rows)
        assert out_gpu.tolist() == out_cpu.tolist(), draw
        for g, c in zip(state_gpu[2:5], state_cpu[2:5]):
            assert g.tolist() == c.tolist(), draw
    assert state_gpu[3].tolist() == [8, 0, 8, 0, 8]


def test_sample_rows_refuses_what_it_cannot_rank():
    f, i, recent, recent_len, rng, out, status = _sampler_state(
        2, [[1.0, 0.9, 0.0, 1.0], [1.0, 1.0, 0.0, 1.0]], [[0, 0], [2000, 0]], [1, 2])
    logits = randn(2, 5000, seed=70)
    ops().sample_rows(logits, f, i, recent, recent_len, rng, out, status)
    assert status.tolist() == [1, 1]


def test_a_refused_row_stays_flagged_over_later_steps():
    """4,096 equal logits at a top-k cut of 40 are more ties than the kernel ranks: the row is refused.
    The next launch, on logits it can rank, must not erase the flag (only the host clears it)."""
    f, i, recent, recent_len, rng, out, status = _sampler_state(
        2, [[1.0, 0.9, 0.0, 1.0], [1.0, 0.9, 0.0, 1.0]], [[40, 0], [40, 0]], [1, 2])
    logits = torch.zeros(2, 4096, device=DEV)
    logits[1] = randn(1, 4096, seed=71)[0]
    ops().sample_rows(logits, f, i, recent, recent_len, rng, out, status)
    assert status.tolist() == [1, 0] and out.tolist()[0] == 0
    ops().sample_rows(randn(2, 4096, seed=72), f, i, recent, recent_len, rng, out, status)
    assert status.tolist() == [1, 0]


# ----------------------------------------------------------------------------- what rides in a product's epilogue

def _sums_in_parts(x, parts, seed):
    """Sums of squares of the rows of x, spread over `parts` partial sums (as a producer would leave them)."""
    total = (x.float() * x.float()).sum(dim=-1)
    weights = torch.rand(x.shape[0], parts, generator=torch.Generator().manual_seed(seed)).to(DEV) + 0.1
    sums = torch.full((x.shape[0], ops().SUMSQ_LD), 1e30, device=DEV)      # unused parts must not be read
    sums[:, :parts] = total[:, None] * weights / weights.sum(dim=-1, keepdim=True)
    return sums


@pytest.mark.parametrize("m,n,k,parts", [(8, 6144, 4096, 32), (1, 256, 64, 1), (16, 384, 512, 3),
                                         (40, 320, 1024, 5), (128, 512, 256, 64), (300, 512, 256, 2),
                                         (2048, 1024, 256, 16), (700, 200, 72, 1)])
@pytest.mark.parametrize("bias", [False, True])
def test_linear_with_a_folded_norm(m, n, k, parts, bias):
    """The norm folded into the product: un-normalised bfloat16 rows, the gain in the weights, the rows
    of the result scaled by 1 / sqrt(mean square + eps) in the epilogue (every kernel shape: decode
    tiles summed by the last block or by the sum kernel, one split, tokens on the 128-row side, pairs
    of SMs), against normalising first with the plain norm."""
    x = randn(m, k, seed=140, scale=3.0)
    x[m // 2] *= 1e-3
    gain = 1.0 + randn(k, seed=141, scale=0.2)
    w = randn(n, k, dtype=torch.bfloat16, seed=142, scale=0.1)
    b = randn(n, seed=143) if bias else None
    eps = 1e-5
    folded = (w.float() * gain[None, :]).to(torch.bfloat16)
    norm = ops().FoldedNorm(x.to(torch.bfloat16), _sums_in_parts(x, parts, 144), parts, eps, k)
    got = ops().linear(norm.rows, folded, b, norm=norm)
    want = plain_ops.rmsnorm(x, gain, eps, torch.float32) @ w.float().T + (b if bias else 0.0)
    assert torch.allclose(got.float(), want, atol=3e-2 * float(want.abs().max()), rtol=3e-2)
    assert torch.allclose(plain_ops.linear(norm.rows, folded, b, norm=norm).float(), want,
                          atol=3e-2 * float(want.abs().max()), rtol=3e-2)
    assert ops().tensor_core_status() == 0


@pytest.mark.parametrize("m,f,k", [(8, 14336, 4096), (40, 320, 1024), (300, 1024, 520), (2048, 1024, 256)])
def test_gated_epilogue_with_a_folded_norm(m, f, k):
    x = randn(m, k, seed=150, scale=2.0)
    gain = 1.0 + randn(k, seed=151, scale=0.2)
    gate = randn(f, k, dtype=torch.bfloat16, seed=152, scale=0.05)
    up = randn(f, k, dtype=torch.bfloat16, seed=153, scale=0.05)
    mixed = torch.stack([gate.view(-1, 16, k), up.view(-1, 16, k)], dim=1).reshape(2 * f, k)
    folded = (mixed.float() * gain[None, :]).to(torch.bfloat16).contiguous()
    norm = ops().FoldedNorm(x.to(torch.bfloat16), _sums_in_parts(x, 7, 154), 7, 1e-6, k)
    got = ops().linear(norm.rows, folded, glu=True, norm=norm)
    h = plain_ops.rmsnorm(x, gain, 1e-6, torch.float32)
    g, u = h @ gate.float().T, h @ up.float().T
    want = g / (1 + torch.exp(-g)) * u
    assert torch.allclose(got.float(), want, atol=3e-2 * float(want.abs().max()), rtol=3e-2)


@pytest.mark.parametrize("m,n,k", [(8, 4096, 4096), (1, 4096, 14336), (16, 384, 512), (8, 200, 256),
                                   (40, 4096, 1024), (64, 520, 256), (300, 512, 256), (5, 64, 64)])
def test_linear_leaves_the_next_norms_input(m, n, k):
    """A product that adds into the residual also leaves the updated rows as bfloat16 and the sums of
    their squares in parts (by the tile's last block, by the sum kernel, or by a kernel behind the
    product where the shape's kernel has no such epilogue): twice in a row on the same buffers."""
    a = randn(m, k, dtype=torch.bfloat16, seed=160)
    w = randn(n, k, dtype=torch.bfloat16, seed=161, scale=0.1)
    b = randn(n, seed=162)
    residual = randn(m, n, seed=163, scale=2.0)
    want = residual.clone()
    emit = ops().Emit(torch.zeros(m, n, dtype=torch.bfloat16, device=DEV),
                      torch.full((m, ops().SUMSQ_LD), float("nan"), device=DEV))
    for _ in range(2):
        want = want + (a.float() @ w.float().T + b)
        ops().linear(a, w, b, residual=residual, emit=emit)
        scale = float(want.abs().max())
        assert torch.allclose(residual, want, atol=2e-2 * scale, rtol=2e-2)
        assert 1 <= emit.parts <= ops().SUMSQ_LD
        assert torch.equal(emit.rows, residual.to(torch.bfloat16))
        sums = emit.sumsq[:, :emit.parts].sum(dim=-1)
        assert torch.allclose(sums, (residual * residual).sum(dim=-1), rtol=1e-4)
    assert ops().tensor_core_status() == 0


@pytest.mark.parametrize("tokens", [1, 8, 16, 40, 128, 300, 1100])
@pytest.mark.parametrize("heads,kv_heads,dim,interleaved,bias", [(8, 2, 128, False, False), (4, 4, 64, False, True),
                                                                 (6, 2, 32, True, True), (3, 1, 128, True, False),
                                                                 (6, 2, 48, False, False)])
def test_qkv_product_rotates_and_writes_the_cache(tokens, heads, kv_heads, dim, interleaved, bias):
    """The q/k/v product with the rotation and the cache write in its epilogue (and a folded norm
    with it) against the product followed by the plain rope_cache_write: sequences at different
    positions and pages, head sizes that fit a tile and one that does not (48: a kernel of its own
    runs behind the product). 1,100 tokens run 256 x 256 tiles on pairs of SMs, which leave the
    rotation to the kernel behind them."""
    k = 256
    width = (heads + 2 * kv_heads) * dim
    counts = [tokens] if tokens < 3 else [tokens - 2, 1, 1]
    starts = [130, 63, 0][:len(counts)]
    lens = [s + c for s, c in zip(starts, counts)]
    table, pages_wide, k_cache, v_cache = make_cache(len(counts), lens, kv_heads, dim, torch.bfloat16, 170)
    tok_pos = torch.tensor([p for s, c in zip(starts, counts) for p in range(s, s + c)], dtype=torch.int32, device=DEV)
    tok_seq = torch.tensor([i for i, c in enumerate(counts) for _ in range(c)], dtype=torch.int32, device=DEV)
    x = randn(tokens, k, seed=171, scale=2.0)
    gain = 1.0 + randn(k, seed=172, scale=0.2)
    w = randn(width, k, dtype=torch.bfloat16, seed=173, scale=0.1)
    b = randn(width, seed=174) if bias else None
    folded = (w.float() * gain[None, :]).to(torch.bfloat16)
    norm = ops().FoldedNorm(x.to(torch.bfloat16), _sums_in_parts(x, 4, 175), 4, 1e-5, k)
    angle = torch.arange(max(lens) + 1, dtype=torch.float64)[:, None] * (
        10000.0 ** (-2.0 * torch.arange(dim // 2, dtype=torch.float64) / dim))[None, :]
    rope = torch.cat([angle.cos(), angle.sin()], 1).float().to(DEV)
    # plain: normalise, project, round as the unfused path does, rotate, write
    want_qkv = (plain_ops.rmsnorm(x, gain, 1e-5, torch.float32) @ w.float().T + (b if bias else 0.0)).to(torch.bfloat16)
    want_k, want_v = k_cache.clone(), v_cache.clone()
    plain_ops.rope_cache_write(want_qkv, rope, tok_pos, tok_seq, table, pages_wide, want_k, want_v, heads,
                               kv_heads, dim, interleaved)
    for write in (True, False):
        got_k, got_v = k_cache.clone(), v_cache.clone()
        got = ops().linear(norm.rows, folded, b, norm=norm, rope=ops().RopeWrite(
            rope, tok_pos, tok_seq, table, pages_wide, got_k, got_v, heads, kv_heads, dim, interleaved, write))
        q = heads * dim
        scale = float(want_qkv.float().abs().max())
        assert torch.allclose(got[:, :q].float(), want_qkv[:, :q].float(), atol=3e-2 * scale, rtol=3e-2)
        if write:
            assert torch.allclose(got_k.float(), want_k.float(), atol=3e-2 * scale, rtol=3e-2)    # other rows keep 7.0
            assert torch.allclose(got_v.float(), want_v.float(), atol=3e-2 * scale, rtol=3e-2)
        else:
            assert torch.equal(got_k, k_cache) and torch.equal(got_v, v_cache)
    assert ops().tensor_core_status() == 0


def test_cast_sumsq_and_embedding_leave_the_first_norms_input():
    x = randn(9, 1000, seed=180, scale=3.0)
    emit = ops().Emit(torch.empty(9, 1000, dtype=torch.bfloat16, device=DEV), torch.zeros(9, ops().SUMSQ_LD, device=DEV))
    ops().cast_sumsq(x, emit)
    assert emit.parts == 1 and torch.equal(emit.rows, x.to(torch.bfloat16))
    assert torch.allclose(emit.sumsq[:, 0], (x * x).sum(dim=-1), rtol=1e-5)
    table = randn(301, 72, dtype=torch.bfloat16, seed=181)
    tokens = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    emit = ops().Emit(torch.empty(5, 72, dtype=torch.bfloat16, device=DEV), torch.zeros(5, ops().SUMSQ_LD, device=DEV))
    got = ops().embed(tokens, table, scale=2.0, emit=emit)
    want = plain_ops.embed(tokens, table, scale=2.0)
    assert torch.equal(got, want) and torch.equal(emit.rows, want.to(torch.bfloat16))
    assert torch.allclose(emit.sumsq[:, 0], (want * want).sum(dim=-1), rtol=1e-5)
