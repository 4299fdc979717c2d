"""kuiperllama_b200: a small single-GPU inference library for the Llama 2/3 dense decoder on
NVIDIA B200 (sm_100a): configuration, safetensors weights, parts, a paged cache with slots, one
step function, a generation loop, samplers and hand-written CUDA kernels."""
from .api import Inference, LlamaInfer, load
from .config import ConfigError, LlamaConfig, config_from_folder
from .engine import Engine, SequenceInput, StepError, load_model, random_model, write_random_model_folder
from .sampling import Sampler, SamplingParams
from .weights import WeightsError

__version__ = "0.1.0"
__all__ = ["Inference", "LlamaInfer", "load", "ConfigError", "LlamaConfig", "config_from_folder", "Engine", "SequenceInput",
           "StepError", "load_model", "random_model", "write_random_model_folder", "Sampler", "SamplingParams",
           "WeightsError"]
