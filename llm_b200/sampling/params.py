"""Sampling parameters with the names, meanings and defaults of MythEclipse/llm."""
from __future__ import annotations

from dataclasses import dataclass, replace

from ..errors import Unsupported

DEFAULT_SEED = 0x5EED_1234_ABCD_0001
MAX_TOP_K = 1024       # MAX_TOP_K of csrc/sampling.cu


@dataclass(frozen=True)
class SamplingParams:
    """apps/engine/src/sampler.rs:9-37: temperature <= 0 is greedy; top_k 0 means
    no top-k; top_p outside [0, 1) and min_p <= 0 switch those filters off;
    repeat_penalty 1 or repeat_last_n 0 switch the penalty off."""
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.75
    min_p: float = 0.25
    repeat_penalty: float = 1.1
    repeat_last_n: int = 64
    seed: int = DEFAULT_SEED

    def check(self, vocab: int) -> None:
        """Refuse what the device sampler cannot do, before anything runs."""
        if self.temperature <= 0.0 or vocab <= MAX_TOP_K:
            return
        if self.top_k > MAX_TOP_K and self.top_k < vocab:
            raise Unsupported(f"top_k {self.top_k} exceeds {MAX_TOP_K}")
        if (self.top_k <= 0 or self.top_k >= vocab) and 0.0 <= self.top_p < 1.0:
            raise Unsupported("top_p below 1 needs a top_k between 1 and "
                              f"{MAX_TOP_K} (the ranked chain holds that many candidates)")
        if self.top_k >= vocab:
            raise Unsupported(f"top_k {self.top_k} covers the whole vocabulary; use 0 for no top-k")

    @staticmethod
    def greedy() -> "SamplingParams":
        return SamplingParams(temperature=0.0, repeat_penalty=1.0)

    def with_seed(self, seed: int) -> "SamplingParams":
        return replace(self, seed=seed)
