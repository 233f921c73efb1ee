from .generate import GenerationError, GenerationResult, Request, generate, plan_batches
from .loading import load_model, parse_dtype
from .model import BuildOptions, DecoderModel, LayerCall
from .step import Engine, StepEntry, StepError

__all__ = ["GenerationError", "GenerationResult", "Request", "generate", "plan_batches", "load_model",
           "parse_dtype", "BuildOptions", "DecoderModel", "LayerCall", "Engine", "StepEntry", "StepError"]
