"""The Python entry point.

Options carry the names, meanings and defaults of MythEclipse/llm's command
line and sampler (apps/cli/src/main.rs:20-22,55-76: --model, --context 4096,
--max-tokens 256, --temperature 0.7; apps/engine/src/sampler.rs:19-37 for the
rest). Prompts and results are token ids.
"""
from __future__ import annotations

import torch

from .cache import round_up
from .engine import Engine, GenerationRequest, generate as _generate, load_model
from .errors import FormatError
from .sampling import DEFAULT_SEED, SamplingParams

DEFAULT_CONTEXT = 4096
DEFAULT_MAX_TOKENS = 256

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(name):
    try:
        return _DTYPES[name]
    except KeyError:
        raise FormatError(f"dtype '{name}' (use bfloat16 or float32)") from None


class LLM:
    """A loaded model with its cache.

    model: a folder with config.json and model.safetensors, or a bound DecoderModel.
    context: most positions one sequence may hold (its prompt and what it generates).
    batch: most sequences generated together.
    """

    def __init__(self, model, dtype="bfloat16", device="cuda:0", context: int = DEFAULT_CONTEXT,
                 batch: int = 8, max_tokens_held: int | None = None):
        if isinstance(model, (str, bytes)) or hasattr(model, "__fspath__"):
            model = load_model(model, parse_dtype(dtype), device)
        self.model = model
        context = min(context, model.spec.max_positions)
        held = max_tokens_held or batch * round_up(context)
        self.engine = Engine(model, max_tokens=held, max_seq_len=context, max_slots=batch)
        self.default_stop_tokens = tuple(model.spec.stop_tokens)

    def generate(self, prompts, max_tokens: int = DEFAULT_MAX_TOKENS, temperature: float = 0.7,
                 top_k: int = 40, top_p: float = 0.75, min_p: float = 0.25,
                 repeat_penalty: float = 1.1, repeat_last_n: int = 64, seed: int = DEFAULT_SEED,
                 stop_tokens=None, on_token=None, details: bool = False):
        """Generate for every prompt (a list of token ids each). The i-th
        prompt samples with seed + i. `stop_tokens` defaults to the model's
        eos ids. Returns the generated ids per prompt, or GenerationResult
        objects with `details=True`."""
        if prompts and isinstance(prompts[0], int):
            prompts = [prompts]
        stops = tuple(self.default_stop_tokens if stop_tokens is None else stop_tokens)
        requests = [GenerationRequest(
            prompt=list(p), max_tokens=max_tokens, stop_tokens=stops,
            params=SamplingParams(temperature, top_k, top_p, min_p, repeat_penalty, repeat_last_n,
                                  (seed + i) & ((1 << 64) - 1)))
            for i, p in enumerate(prompts)]
        results = _generate(self.engine, requests, on_token=on_token)
        return results if details else [r.tokens for r in results]


def load(model, **options) -> LLM:
    return LLM(model, **options)


def generate(model, prompts, **options):
    """One call: load `model` (a folder) and generate. Options of `LLM` (dtype,
    device, context, batch) and of `LLM.generate` may both be given."""
    load_keys = ("dtype", "device", "context", "batch", "max_tokens_held")
    llm = LLM(model, **{k: options.pop(k) for k in load_keys if k in options})
    return llm.generate(prompts, **options)
