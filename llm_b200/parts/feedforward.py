"""Dense gated feed-forward."""
from __future__ import annotations

import torch

from .. import ops
from ..errors import Unsupported
from ..weights.loader import ParamSpec
from .base import FeedForward, register_feed_forward, to_run_dtype


class GatedMlp(FeedForward):
    """down(silu(gate h) * (up h)) added to the residual stream, gate and up as
    one matrix product (apps/engine/src/model.rs:1180-1216 of MythEclipse/llm)."""
    graph_safe = True
    emits = True
    libraries = ("elementwise", "gemm_simt", "gemm_skinny", "gemm_tc")

    def __init__(self, spec):
        if spec.activation != "silu":
            raise Unsupported(f"activation '{spec.activation}' in a gated feed-forward")
        self.spec = spec
        self.w_gate_up = self.w_down = None
        self.fused = False

    def parameters(self):
        s, t = self.spec, self.spec.tensor
        return {t["gate"]: ParamSpec((s.intermediate, s.hidden)),
                t["up"]: ParamSpec((s.intermediate, s.hidden)),
                t["down"]: ParamSpec((s.hidden, s.intermediate))}

    def bind(self, tensors, dtype, device):
        t, s = self.spec.tensor, self.spec
        gate = to_run_dtype(tensors[t["gate"]], dtype, device)
        up = to_run_dtype(tensors[t["up"]], dtype, device)
        # where the tensor-core product can apply the activation in its epilogue, gate and up
        # rows alternate in blocks of 16; otherwise they are stacked [gate; up]
        self.fused = ops.glu_fusable(2 * s.intermediate, s.hidden, dtype)
        if self.fused:
            b = ops.GLU_BLOCK
            self.w_gate_up = torch.stack([gate.view(-1, b, s.hidden), up.view(-1, b, s.hidden)],
                                         dim=1).reshape(2 * s.intermediate, s.hidden).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up])
        self.w_down = to_run_dtype(tensors[t["down"]], dtype, device)

    def fold_input_norm(self, gain):
        """bfloat16 runs: the gain goes into the columns of the gate and up matrix."""
        if self.w_gate_up.dtype != torch.bfloat16 or self.spec.hidden % 8:
            return False
        self.w_gate_up = (self.w_gate_up.float() * gain.to(self.w_gate_up.device)[None, :]).to(torch.bfloat16).contiguous()
        return True

    def kernel_shapes(self, dtype, token_counts):
        s, out = self.spec, []
        for n in token_counts:
            out.append((f"gate and up product, {n} tokens", "linear",
                        dict(m=n, n=2 * s.intermediate, k=s.hidden, in_dtype=dtype, out_dtype=dtype, lda=s.hidden, aligned=True)))
            out.append((f"down product, {n} tokens", "linear",
                        dict(m=n, n=s.hidden, k=s.intermediate, in_dtype=dtype, out_dtype=torch.float32,
                             lda=s.intermediate, aligned=True)))
        return out

    def scratch_requests(self, n_tokens, dtype):
        from ..engine.workspace import BufferRequest
        s = self.spec
        # phases: 0 gate and up, 1 activation, 2 down projection
        act = BufferRequest("act", (n_tokens, s.intermediate), dtype, 0 if self.fused else 1, 2)
        if self.fused:
            return [act]
        return [BufferRequest("gate_up", (n_tokens, 2 * s.intermediate), dtype, 0, 1), act]

    def replay_key(self, step):
        return ()

    def forward(self, h, ctx, residual, emit=None):
        norm = h if isinstance(h, ops.FoldedNorm) else None
        if norm is not None:
            h = norm.rows
        n, width = h.shape[0], self.spec.intermediate
        if self.fused:
            act = ops.linear(h, self.w_gate_up, glu=True, out=ctx.scratch("act", (n, width), h.dtype), norm=norm)
        else:
            gate_up = ops.linear(h, self.w_gate_up, out=ctx.scratch("gate_up", (n, 2 * width), h.dtype), norm=norm)
            act = ops.swiglu(gate_up, out=ctx.scratch("act", (n, width), h.dtype))
        ops.linear(act, self.w_down, residual=residual, emit=emit)


register_feed_forward("gated_mlp", GatedMlp)
