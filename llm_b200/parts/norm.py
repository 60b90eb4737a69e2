"""RMSNorm."""
from __future__ import annotations

from .. import ops
from ..weights.loader import ParamSpec
from .base import Norm, register_norm, to_float32


class RmsNorm(Norm):
    """x / sqrt(mean(x^2) + eps) * weight, the norm of MythEclipse/llm
    (apps/engine/src/ops.rs:4-12). The weight is held in 32-bit."""
    graph_safe = True
    libraries = ("elementwise",)
    #: y = x / sqrt(mean(x^2) + eps) * gain: a part behind this norm may fold it (Part.fold_input_norm)
    foldable = True

    def __init__(self, spec):
        self.spec = spec
        self.gain = None

    def parameters(self):
        return {self.spec.weight: ParamSpec((self.spec.size,), "gain")}

    def bind(self, tensors, dtype, device):
        self.gain = to_float32(tensors[self.spec.weight], device)

    def replay_key(self, step):
        return ()

    def forward(self, x, out_dtype, rows=None, out=None):
        return ops.rmsnorm(x, self.gain, self.spec.eps, out_dtype, rows, out=out)


register_norm("rmsnorm", RmsNorm)
