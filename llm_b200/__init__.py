"""llm_b200: a small Llama generation library for one B200 GPU."""
from . import errors
from .api import LLM, generate, load
from .config import LlamaConfig, load_config, register_architecture
from .engine import (DecoderModel, Engine, Entry, GenerationRequest, GenerationResult, load_model,
                     random_model)
from .sampling import SamplingParams
from .weights import write_random_model

__all__ = ["errors", "LLM", "generate", "load", "LlamaConfig", "load_config",
           "register_architecture", "DecoderModel", "Engine", "Entry", "GenerationRequest",
           "GenerationResult", "load_model", "random_model", "SamplingParams",
           "write_random_model"]
