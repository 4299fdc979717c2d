"""Random weights: a model folder (config.json, model.safetensors) from a configuration and a
seed, and a lazy on-device source of the same kind of tensors for measurements.

ExiledOfCode/KuiperLLama has no random-weights mode at run time; tools/model.py:241-247
initialises matrices N(0, 0.02) for training.  Here every matrix is N(0, std) and every norm
weight 1 + N(0, std), std = 0.02 unless told otherwise, each tensor from a generator seeded
by (seed, tensor name), stored as bfloat16.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, Mapping, Optional

import torch

from .loader import TensorDecl
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, decl: TensorDecl, seed: int, std: float, device="cpu",
                  dtype: torch.dtype = torch.bfloat16, stored: Optional[torch.dtype] = None) -> torch.Tensor:
    """The tensor ``name`` for ``seed`` in ``dtype``.  With ``stored`` the values are first rounded
    to that dtype, as a checkpoint of that dtype would hold them."""
    if decl.role == "int_table":
        raise ValueError(f"{name}: integer tables have no random initialisation")
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    t = torch.empty(decl.shape, dtype=torch.float32, device=device).normal_(0.0, std, generator=gen)
    if decl.init == "one_plus_normal":
        t += 1.0
    elif decl.init != "normal":
        raise ValueError(f"{name}: unknown initialisation {decl.init!r}")
    if stored is not None:
        t = t.to(stored)
    return t.to(dtype)


def write_random_model(folder: str, config, manifest: Mapping[str, TensorDecl], seed: int, std: float = 0.02) -> None:
    """Write ``config.json`` and ``model.safetensors`` (bfloat16) into ``folder``."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=2)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      ((name, random_tensor(name, decl, seed, std)) for name, decl in manifest.items()),
                      metadata={"format": "pt", "seed": str(seed), "std": str(std)})


class RandomTensors(Mapping):
    """``tensors[name]`` makes the tensor on ``device`` when it is asked for and keeps no
    copy: a model of any size can be built without a file."""

    def __init__(self, manifest: Mapping[str, TensorDecl], seed: int, device, dtype: torch.dtype, std: float = 0.02,
                 stored: Optional[torch.dtype] = None):
        self.manifest, self.seed, self.device, self.dtype, self.std, self.stored = manifest, seed, device, dtype, std, stored

    def __getitem__(self, name: str) -> torch.Tensor:
        decl = self.manifest[name]
        keep32 = decl.role == "vector"
        return random_tensor(name, decl, self.seed, self.std, device=self.device,
                             dtype=torch.float32 if keep32 else self.dtype, stored=self.stored)

    def __iter__(self) -> Iterator[str]:
        return iter(self.manifest)

    def __len__(self) -> int:
        return len(self.manifest)
