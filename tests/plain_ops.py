"""Plain PyTorch statements of what every kernel of `llm_b200.ops` computes.

Each function has the signature of the op it restates and works on any
device in 32-bit arithmetic (results are rounded to the op's output dtype at
the end). The GPU tests compare every CUDA kernel with its function here;
the CPU tests put these functions in the kernels' place (`install`) to check
the host-side logic of the engine: packing, positions, pages, slots, chunked
steps. Nothing in the `llm_b200` package imports this file.
"""
from __future__ import annotations

import torch

PAGE = 64


def embed(tokens, table, out=None, scale=1.0, emit=None):
    x = table[tokens.long()].to(torch.float32) * scale
    if emit is not None:
        cast_sumsq(x, emit)
    return x


def cast_sumsq(x, emit):
    """The next norm's input: the rows as bfloat16 and their sums of squares (one part)."""
    emit.rows.copy_(x.to(torch.bfloat16))
    emit.sumsq[:, 0] = (x.float() * x.float()).sum(dim=-1)
    emit.parts = 1
    return emit


def scale_(x, scale):
    x *= scale
    return x


def rmsnorm(x, gain, eps, out_dtype, rows=None, out=None):
    if rows is not None:
        x = x[rows.long()]
    x = x.to(torch.float32)
    scale = 1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return (x * scale * gain.to(torch.float32)).to(out_dtype)


def swiglu(gate_up, out=None):
    width = gate_up.shape[1] // 2
    g = gate_up[:, :width].to(torch.float32)
    u = gate_up[:, width:].to(torch.float32)
    return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype)


def linear(a, w, bias=None, out_dtype=None, residual=None, out=None, glu=False, norm=None, emit=None,
           rope=None):
    product = a.to(torch.float32) @ w.to(torch.float32).T
    if norm is not None:
        # a folded norm: rows scaled by 1 / sqrt(mean square + eps) from the partial sums of squares
        mean_square = norm.sumsq[:, :norm.parts].sum(dim=-1, keepdim=True) / norm.width
        product = product / torch.sqrt(mean_square + norm.eps)
    if rope is not None:
        if bias is not None:
            product = product + bias.to(torch.float32)
        qkv = product.to(out_dtype or a.dtype)
        rope_cache_write(qkv, rope.table, rope.tok_pos, rope.tok_seq, rope.block_table, rope.ring_pages,
                         rope.k_cache, rope.v_cache, rope.n_heads, rope.n_kv_heads, rope.head_dim,
                         rope.interleaved, rope.write_cache)
        return qkv
    if glu:
        # rows of w alternate 16 gate rows, 16 up rows
        m = product.shape[0]
        blocks = product.view(m, -1, 2, 16)
        g, u = blocks[:, :, 0, :].reshape(m, -1), blocks[:, :, 1, :].reshape(m, -1)
        return (g / (1.0 + torch.exp(-g)) * u).to(a.dtype)
    if bias is not None:
        product = product + bias.to(torch.float32)
    if residual is not None:
        residual += product
        if emit is not None:
            cast_sumsq(residual, emit)
        return residual
    return product.to(out_dtype or a.dtype)


def _rotate(x, cos, sin, interleaved):
    """x [n, heads, D] float32; cos, sin [n, n_rot/2]: the first n_rot elements of a head rotate,
    the rest passes through."""
    half = cos.shape[-1]
    n_rot = 2 * half
    cos, sin = cos[:, None, :], sin[:, None, :]
    out = x.clone()
    if interleaved:
        low, high = x[..., 0:n_rot:2], x[..., 1:n_rot:2]
        out[..., 0:n_rot:2] = low * cos - high * sin
        out[..., 1:n_rot:2] = low * sin + high * cos
    else:
        low, high = x[..., :half], x[..., half:n_rot]
        out[..., :half] = low * cos - high * sin
        out[..., half:n_rot] = low * sin + high * cos
    return out


def rope_cache_write(qkv, rope_table, tok_pos, tok_seq, block_table, ring_pages, k_cache, v_cache,
                     n_heads, n_kv_heads, head_dim, interleaved=False, write_cache=True):
    n = qkv.shape[0]
    if n == 0:
        return
    qw, kw = n_heads * head_dim, n_kv_heads * head_dim
    pos = tok_pos.long()
    q = qkv[:, :qw].to(torch.float32).view(n, n_heads, head_dim)
    k = qkv[:, qw:qw + kw].to(torch.float32).view(n, n_kv_heads, head_dim)
    v = qkv[:, qw + kw:].view(n, n_kv_heads, head_dim)
    if rope_table is not None:
        half = rope_table.shape[1] // 2
        cos, sin = rope_table[pos, :half], rope_table[pos, half:]
        q = _rotate(q, cos, sin, interleaved)
        k = _rotate(k, cos, sin, interleaved)
    qkv[:, :qw] = q.reshape(n, qw).to(qkv.dtype)
    if not write_cache:
        return
    pages = block_table.long()[tok_seq.long(), (pos // PAGE) % ring_pages]
    rows = pos % PAGE
    k_cache[pages, :, rows, :] = k.to(k_cache.dtype)
    v_cache[pages, :, rows, :] = v.to(v_cache.dtype)


def attention(qkv, k_cache, v_cache, block_table, ring_pages, tok_pos, tok_seq, n_heads,
              n_kv_heads, head_dim, scale, window=0, out=None, decode=False, seq_lens=None,
              max_len=0, cu_seqlens=None, max_new=0, seq_order=None):
    n = qkv.shape[0]
    result = torch.zeros((n, n_heads * head_dim), dtype=torch.float32, device=qkv.device)
    group = n_heads // n_kv_heads
    table = block_table.long()
    for t in range(n):
        pos, b = int(tok_pos[t]), int(tok_seq[t])
        first = max(0, pos - window + 1) if window > 0 else 0
        js = torch.arange(first, pos + 1, device=qkv.device)
        pages = table[b, (js // PAGE) % ring_pages]
        keys = k_cache[pages, :, js % PAGE, :].to(torch.float32)        # [n_keys, Hkv, D]
        vals = v_cache[pages, :, js % PAGE, :].to(torch.float32)
        q = qkv[t, :n_heads * head_dim].to(torch.float32).view(n_heads, head_dim)
        for h in range(n_heads):
            scores = (keys[:, h // group, :] @ q[h]) * scale
            p = torch.softmax(scores, dim=0)
            result[t, h * head_dim:(h + 1) * head_dim] = p @ vals[:, h // group, :]
    return result.to(qkv.dtype)


def argmax_rows(logits, out=None):
    best = logits.max(dim=1, keepdim=True).values
    first = (logits == best).to(torch.int32).argmax(dim=1)
    return first.to(torch.int32)


MASK64 = (1 << 64) - 1


def _next_uniform(state):
    x = state & MASK64
    x ^= x >> 12
    x ^= (x << 25) & MASK64
    x ^= x >> 27
    value = (x * 0x2545F4914F6CDD1D) & MASK64
    return x, float(value >> 40) / float(1 << 24)


def _sample_rows(logits, params, iparams, recent, recent_len, rng_state, out, status):
    """Row by row, the chain of csrc/sampling.cu in 32-bit host arithmetic."""
    n, vocab = logits.shape
    f32 = torch.float32
    for r in range(n):
        temperature, top_p, min_p, penalty = (float(v) for v in params[r])
        top_k, last_n = (int(v) for v in iparams[r])
        row = logits[r]
        status[r] = 0
        if penalty != 1.0 and last_n > 0 and recent is not None:
            cap = recent.shape[1]
            total = int(recent_len[r])
            span = min(total, last_n, cap)
            pen = torch.tensor(penalty, dtype=f32)
            for i in range(total - span, total):
                token = int(recent[r, i % cap])
                if 0 <= token < vocab:
                    row[token] = row[token] / pen if row[token] > 0 else row[token] * pen
        if not temperature > 0.0:
            out[r] = int(argmax_rows(row[None])[0])
            continue
        row *= (torch.tensor(1.0, dtype=f32) / torch.tensor(temperature, dtype=f32))
        state = int(rng_state[r]) & MASK64
        if (top_k <= 0 or top_k >= vocab) and vocab > 1024:
            if top_k > 0 or 0.0 <= top_p < 1.0:
                status[r], out[r] = 1, 0
                continue
            p = torch.exp(row - row.max())
            p = torch.where(p >= max(min_p, 0.0), p, torch.zeros_like(p))
            state, u = _next_uniform(state)
            target = torch.tensor(u, dtype=f32) * p.sum()
            pick = int((torch.cumsum(p, 0) >= target).nonzero()[0])
        else:
            if top_k > 1024:
                status[r], out[r] = 1, 0
                continue
            k = vocab if top_k <= 0 or top_k >= vocab else top_k
            order = sorted(range(vocab), key=lambda i: (-float(row[i]), i))[:k]
            probs = torch.exp(row[order] - row[order[0]])
            total = torch.tensor(0.0, dtype=f32)
            for v in probs:
                total = total + v
            if total > 0:
                probs = probs / total
            kept = len(order)
            if 0.0 <= top_p < 1.0:
                cumulative = torch.tensor(0.0, dtype=f32)
                for i, v in enumerate(probs):
                    cumulative = cumulative + v
                    if cumulative > top_p:
                        kept = i + 1
                        break
            if min_p > 0.0:
                cut = probs[0] * torch.tensor(min_p, dtype=f32)
                keep = 0
                while keep < kept and probs[keep] >= cut:
                    keep += 1
                kept = keep
            total = torch.tensor(0.0, dtype=f32)
            for v in probs[:kept]:
                total = total + v
            pick = order[0]
            if total > 0:
                state, u = _next_uniform(state)
                target = torch.tensor(u, dtype=f32) * total
                for i in range(kept):
                    target = target - probs[i]
                    if target <= 0:
                        pick = order[i]
                        break
        rng_state[r] = state - (1 << 64) if state >= (1 << 63) else state
        out[r] = pick
    return out


def sample_rows(logits, params, iparams, recent, recent_len, rng_state, out, status, record=False,
                state_rows=None):
    """The chain for every row; with `record`, the drawn tokens then enter the rows' windows.
    `state_rows`: row i of the logits belongs to the sequence in row state_rows[i] of the state."""
    if state_rows is not None:
        index = state_rows.long()
        taken = [t[index].clone() if t is not None else None
                 for t in (params, iparams, recent, recent_len, rng_state, status)]
        sample_rows(logits, taken[0], taken[1], taken[2], taken[3], taken[4], out, taken[5], record)
        for whole, part in zip((recent, recent_len, rng_state, status), (taken[2], taken[3], taken[4], taken[5])):
            if whole is not None:
                whole[index] = part
        return out
    _sample_rows(logits, params, iparams, recent, recent_len, rng_state, out, status)
    if record and recent is not None:
        cap = recent.shape[1]
        for r in range(logits.shape[0]):
            recent[r, int(recent_len[r]) % cap] = int(out[r])
            recent_len[r] += 1
    return out



OPS = {"embed": embed, "scale_": scale_, "cast_sumsq": cast_sumsq, "rmsnorm": rmsnorm, "swiglu": swiglu, "linear": linear,
       "rope_cache_write": rope_cache_write, "attention": attention, "argmax_rows": argmax_rows,
       "sample_rows": sample_rows}


def install(monkeypatch):
    """Put the plain functions in the kernels' place (CPU tests of host logic)."""
    import llm_b200.ops as ops
    for name, fn in OPS.items():
        monkeypatch.setattr(ops, name, fn)
    monkeypatch.setattr(ops, "ensure_built", lambda names: None)
    monkeypatch.setattr(ops, "check_device_status", lambda: None)
    monkeypatch.setattr(ops, "glu_fusable", lambda n, k, dtype: dtype == torch.bfloat16 and n % 32 == 0)
