"""Fetch a model's tensors from safetensors by name and check them against what the
model's parts declare.  One error lists every missing tensor, every unexpected tensor and
every wrong shape or type.

Storage rule: bfloat16 stays bfloat16, float16 stays float16 on the host (the parts round it
once, to the run's compute dtype: exact in a float32 run), a tensor stored in 32 bits stays
float32, integer tables become int32.  (KuiperLLama has only float32 and finds tensors by offset,
kuiper/source/model/llama3.cpp:289-422, without a shape check, model.cpp:133-138.)
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Set, Tuple

import torch

from .safetensors_io import SafetensorsFile, SafetensorsFormatError


@dataclass(frozen=True)
class TensorDecl:
    """What a part expects of one tensor.

    role  "matrix": an operand of a matrix product, held in the run's compute dtype;
          "vector": a small per-channel tensor, always held in float32 on the device;
          "int_table": integers, held as int32.
    init  how random-weights mode fills it: "normal" N(0, std) or "one_plus_normal" 1 + N(0, std).
    """
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"


class WeightsError(ValueError):
    """The checkpoint does not fit the model.  ``missing``, ``unexpected`` and ``wrong``
    hold the details that the message lists."""

    def __init__(self, folder: str, missing: List[str], unexpected: List[str], wrong: List[str],
                 other: List[str] = ()):
        self.missing, self.unexpected, self.wrong, self.other = list(missing), list(unexpected), list(wrong), list(other)
        lines = [f"weights in {folder!r} do not fit the model:"]
        if self.other:
            lines += [f"  {o}" for o in self.other]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong:
            lines.append(f"  wrong shape or type ({len(self.wrong)}):")
            lines += [f"    {w}" for w in self.wrong]
        super().__init__("\n".join(lines))


def _open_files(folder: str) -> Dict[str, Tuple[SafetensorsFile, str]]:
    """name -> (file, name) over ``model.safetensors`` or the shards an index names."""
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    paths: List[str]
    if os.path.isfile(single):
        paths = [single]
    elif os.path.isfile(index):
        with open(index) as f:
            weight_map = json.load(f).get("weight_map", {})
        paths = [os.path.join(folder, p) for p in sorted(set(weight_map.values()))]
    else:
        raise WeightsError(folder, [], [], [], [f"neither model.safetensors nor model.safetensors.index.json exists"])
    table: Dict[str, Tuple[SafetensorsFile, str]] = {}
    for p in paths:
        try:
            sf = SafetensorsFile(p)
        except (OSError, SafetensorsFormatError) as e:
            raise WeightsError(folder, [], [], [], [str(e)]) from None
        for name in sf.names():
            table[name] = (sf, name)
    return table


_FLOATS = (torch.float32, torch.float16, torch.bfloat16, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def stored_dtype(file_dtype: torch.dtype, role: str) -> Optional[torch.dtype]:
    """The dtype a tensor is kept in on the host after loading, or None if its type does
    not fit its role."""
    if role == "int_table":
        return torch.int32 if file_dtype in _INTS else None
    if file_dtype not in _FLOATS:
        return None
    if file_dtype in (torch.float16, torch.bfloat16):
        return file_dtype              # kept as stored; the parts convert once to the compute dtype
    return torch.float32


def load_tensors(folder: str, manifest: Dict[str, TensorDecl],
                 ignorable: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """All tensors of ``manifest`` as CPU tensors.  Names in the checkpoint that the
    manifest lacks are an error unless they end with one of ``ignorable``."""
    table = _open_files(folder)
    ignorable = tuple(ignorable)
    missing = [n for n in manifest if n not in table]
    unexpected = [n for n in table if n not in manifest and not (ignorable and n.endswith(ignorable))]
    wrong: List[str] = []
    for name, decl in manifest.items():
        if name not in table:
            continue
        sf, _ = table[name]
        e = sf.entries[name]
        if tuple(e.shape) != tuple(decl.shape):
            wrong.append(f"{name}: shape {list(e.shape)}, expected {list(decl.shape)}")
        elif stored_dtype(e.dtype, decl.role) is None:
            wrong.append(f"{name}: dtype {e.dtype} does not fit a {decl.role}")
    if missing or unexpected or wrong:
        raise WeightsError(folder, sorted(missing), sorted(unexpected), wrong)
    out: Dict[str, torch.Tensor] = {}
    for name, decl in manifest.items():
        sf, _ = table[name]
        t = sf.tensor(name)
        out[name] = t.to(stored_dtype(t.dtype, decl.role))   # a view when the dtype already fits
    return out
