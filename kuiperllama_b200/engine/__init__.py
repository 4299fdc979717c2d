"""Model, step function, generation loop."""
from .model import DecoderModel, ignorable_tensor_suffixes, model_manifest
from .step import Engine, SequenceInput, StepError
from .generate import (EngineBackend, GenerationStats, RequestResult, next_batch, run_requests, tokens_held)
from .loading import load_model, parse_dtype, random_model, write_random_model_folder

__all__ = ["DecoderModel", "ignorable_tensor_suffixes", "model_manifest", "Engine", "SequenceInput", "StepError",
           "EngineBackend", "GenerationStats", "RequestResult", "next_batch", "run_requests", "tokens_held",
           "load_model", "parse_dtype", "random_model", "write_random_model_folder"]
