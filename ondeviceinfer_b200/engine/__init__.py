from .generate import GenerationResult, generate_requests, plan_batches
from .model import DecoderModel
from .step import StepContext, resolve_want, run_step

__all__ = ["GenerationResult", "generate_requests", "plan_batches", "DecoderModel", "StepContext",
           "resolve_want", "run_step"]
