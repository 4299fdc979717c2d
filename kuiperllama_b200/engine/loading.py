"""From a folder (or a configuration and a seed) to a model on the device."""
from __future__ import annotations

from typing import Optional

import torch

from ..config import config_from_folder
from ..parts.base import Runtime
from ..weights.loader import load_tensors
from ..weights.random_init import RandomTensors, write_random_model
from .model import DecoderModel, ignorable_tensor_suffixes, model_manifest

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype {dtype!r} is not supported (bfloat16 or float32)") from None


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("kuiperllama_b200 runs on a CUDA device only; there is no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; kuiperllama_b200 has no CPU path")
    return device


def load_model(folder: str, dtype="bfloat16", device="cuda:0") -> DecoderModel:
    """The model that ``folder``'s config.json names, with the weights of its safetensors."""
    device = require_cuda(device)
    config = config_from_folder(folder)
    spec = config.to_model_spec()
    tensors = load_tensors(folder, model_manifest(spec), ignorable=ignorable_tensor_suffixes(spec))
    model = DecoderModel(spec, tensors, Runtime(device=device, dtype=parse_dtype(dtype)))
    model.config = config
    return model


def random_model(config, seed: int, dtype="bfloat16", device="cuda:0", std: float = 0.02, stored=None) -> DecoderModel:
    """A model with random weights made on the device (nothing is written).  ``stored``
    ("bfloat16"): the values a checkpoint of that dtype would hold, so that a float32 model and a
    bfloat16 model of one seed have the same weights."""
    device = require_cuda(device)
    spec = config.to_model_spec()
    dt = parse_dtype(dtype)
    tensors = RandomTensors(model_manifest(spec), seed, device, dt, std, stored=None if stored is None else parse_dtype(stored))
    model = DecoderModel(spec, tensors, Runtime(device=device, dtype=dt))
    model.config = config
    return model


def write_random_model_folder(folder: str, config, seed: int, std: float = 0.02) -> None:
    """Random-weights mode: write config.json and model.safetensors for ``config``."""
    write_random_model(folder, config, model_manifest(config.to_model_spec()), seed, std)
