"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import torch

from .. import ops
from ..cache import KvRequest
from ..weights.loader import ParamSpec
from .base import Mixer, build_position, register_mixer, to_float32, to_run_dtype


class AttentionMixer(Mixer):
    """q, k, v projections as one matrix product, rotation of q and k fused with
    the cache write, attention of the new tokens over the cache, and the output
    projection added to the residual stream in its epilogue: the dense attention
    of MythEclipse/llm (apps/engine/src/model.rs:930-1040), with the sizes, the
    scale, the window, the biases and the position encoding as parameters."""
    graph_safe = True
    emits = True
    libraries = ("elementwise", "gemm_simt", "gemm_skinny", "gemm_tc", "attention_generic", "attention_decode", "attention_prefill", "attention_prefill_tc")

    def __init__(self, spec):
        self.spec = spec
        self.position = build_position(spec.position)
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    @property
    def q_width(self):
        return self.spec.n_heads * self.spec.head_dim

    @property
    def kv_width(self):
        return self.spec.n_kv_heads * self.spec.head_dim

    def parameters(self):
        s, t = self.spec, self.spec.tensor
        out = {t["q"]: ParamSpec((self.q_width, s.hidden)),
               t["k"]: ParamSpec((self.kv_width, s.hidden)),
               t["v"]: ParamSpec((self.kv_width, s.hidden)),
               t["o"]: ParamSpec((s.hidden, self.q_width))}
        if s.bias:
            out[t["q_bias"]] = ParamSpec((self.q_width,), "bias")
            out[t["k_bias"]] = ParamSpec((self.kv_width,), "bias")
            out[t["v_bias"]] = ParamSpec((self.kv_width,), "bias")
            out[t["o_bias"]] = ParamSpec((s.hidden,), "bias")
        return out

    def bind(self, tensors, dtype, device):
        t = self.spec.tensor
        self.w_qkv = torch.cat([to_run_dtype(tensors[t[r]], dtype, device) for r in ("q", "k", "v")])
        self.w_o = to_run_dtype(tensors[t["o"]], dtype, device)
        if self.spec.bias:
            self.b_qkv = torch.cat([to_float32(tensors[t[r + "_bias"]], device) for r in ("q", "k", "v")])
            self.b_o = to_float32(tensors[t["o_bias"]], device)

    def fold_input_norm(self, gain):
        """bfloat16 runs: the gain goes into the columns of the q/k/v matrix (in 32-bit, rounded
        once), and the product's epilogue applies the norm's scale (ops.linear with `norm`)."""
        if self.w_qkv.dtype != torch.bfloat16 or self.spec.hidden % 8:
            return False
        self.w_qkv = (self.w_qkv.float() * gain.to(self.w_qkv.device)[None, :]).to(torch.bfloat16).contiguous()
        return True

    def prepare(self, max_positions, device):
        if self.position is not None:
            self.position.prepare(max_positions, device)

    def scratch_requests(self, n_tokens, dtype):
        from ..engine.workspace import BufferRequest
        s = self.spec
        # phases: 0 projections, 1 rotation + cache write, 2 attention, 3 output projection
        return [BufferRequest("qkv", (n_tokens, self.q_width + 2 * self.kv_width), dtype, 0, 2),
                BufferRequest("mixed", (n_tokens, self.q_width), dtype, 2, 3)]

    def kernel_shapes(self, dtype, token_counts):
        s, out = self.spec, []
        width = self.q_width + 2 * self.kv_width
        for n in token_counts:
            out.append((f"qkv product, {n} tokens", "linear",
                        dict(m=n, n=width, k=s.hidden, in_dtype=dtype, out_dtype=dtype, lda=s.hidden, aligned=True)))
            out.append((f"output product, {n} tokens", "linear",
                        dict(m=n, n=s.hidden, k=self.q_width, in_dtype=dtype, out_dtype=torch.float32,
                             lda=self.q_width, aligned=True)))
        for decode in (True, False):
            out.append(("decode attention" if decode else "prefill attention", "attention",
                        dict(decode=decode, dtype=dtype, n_heads=s.n_heads, n_kv_heads=s.n_kv_heads,
                             head_dim=s.head_dim, window=s.window, packed=True, aligned=True)))
        return out

    def kv_request(self):
        return KvRequest(self.spec.n_kv_heads, self.spec.head_dim, self.spec.window)

    def replay_key(self, step):
        """The attention kernels size their grids by the most new tokens of a sequence (prefill) or
        by the slices of the longest sequence (decode); positions, lengths and pages come from
        device arrays."""
        if step.decode:
            return (True, ops.decode_splits(step.n_seqs, self.spec.n_kv_heads, step.max_len))
        return (False, max(step.new_counts))

    def forward(self, h, ctx, entry, cache_entry, residual, emit=None):
        s = self.spec
        group, keys, values = ctx.cache.layer_view(cache_entry)
        table = ctx.block_tables[group]
        ring = ctx.cache.table_width(group)
        norm = h if isinstance(h, ops.FoldedNorm) else None
        if norm is not None:
            h = norm.rows
        n = h.shape[0]
        angles = self.position.table if self.position is not None else None
        interleaved = self.position.interleaved if self.position is not None else False
        out = ctx.scratch("qkv", (n, self.q_width + 2 * self.kv_width), h.dtype)
        if h.dtype == torch.bfloat16 and (angles is None or angles.shape[1] == s.head_dim):
            # the rotation and the cache write ride in the product's epilogue where its kernel has them
            qkv = ops.linear(h, self.w_qkv, self.b_qkv, out=out, norm=norm, rope=ops.RopeWrite(
                angles, ctx.tok_pos, ctx.tok_seq, table, ring, keys, values, s.n_heads, s.n_kv_heads,
                s.head_dim, interleaved, entry == cache_entry))
        else:
            qkv = ops.linear(h, self.w_qkv, self.b_qkv, out=out, norm=norm)
            ops.rope_cache_write(qkv, angles, ctx.tok_pos, ctx.tok_seq, table, ring, keys, values, s.n_heads,
                                 s.n_kv_heads, s.head_dim, interleaved=interleaved,
                                 write_cache=(entry == cache_entry))
        mixed = ops.attention(qkv, keys, values, table, ring, ctx.tok_pos, ctx.tok_seq, s.n_heads,
                              s.n_kv_heads, s.head_dim, s.scale, s.window, out=ctx.scratch("mixed", (n, self.q_width), h.dtype),
                              decode=ctx.decode,
                              seq_lens=ctx.seq_lens, max_len=ctx.max_len,
                              cu_seqlens=ctx.cu_seqlens, max_new=max(ctx.new_counts),
                              seq_order=ctx.seq_order)
        ops.linear(mixed, self.w_o, self.b_o, residual=residual, emit=emit)


register_mixer("attention", AttentionMixer)
