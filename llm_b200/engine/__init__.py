from .generate import GenerationRequest, GenerationResult, generate, plan_batches
from .model import DecoderModel, declared_parameters, load_model, random_model
from .step import Engine, Entry

__all__ = ["GenerationRequest", "GenerationResult", "generate", "plan_batches", "DecoderModel",
           "declared_parameters", "load_model", "random_model", "Engine", "Entry"]
