"""Reading and writing the safetensors container: an 8-byte little-endian header length,
a JSON header ``{name: {dtype, shape, data_offsets}}`` and the raw tensor bytes.

Tensors are found by name.  (KuiperLLama finds them by byte offset in a flat export,
kuiper/source/model/llama3.cpp:289-422; this reader replaces that export step.)
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFormatError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int            # byte offsets relative to the start of the data section
    end: int


class SafetensorsFile:
    """A memory-mapped safetensors file.  ``entries`` is known after construction;
    ``tensor(name)`` returns a CPU tensor that views the mapping (copy it to keep it)."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsFormatError(f"{path}: shorter than the 8-byte header length")
        self._file = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._file.read(8))
        if 8 + hlen > size:
            raise SafetensorsFormatError(f"{path}: header length {hlen} exceeds the file size {size}")
        try:
            header = json.loads(self._file.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsFormatError(f"{path}: the header is not JSON: {e}") from None
        self._data_start = 8 + hlen
        data_size = size - self._data_start
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                dtype, width = _DTYPES[info["dtype"]]
                shape = tuple(int(s) for s in info["shape"])
                begin, end = (int(o) for o in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise SafetensorsFormatError(f"{path}: bad header entry for {name!r}: {info!r}") from None
            count = 1
            for s in shape:
                count *= s
            if end - begin != count * width or begin < 0 or end > data_size:
                raise SafetensorsFormatError(
                    f"{path}: tensor {name!r} claims bytes [{begin}, {end}) for shape {list(shape)} "
                    f"{info['dtype']} in a data section of {data_size} bytes (truncated file?)")
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end)
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        count = 1
        for s in e.shape:
            count *= s
        if count == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # the mapping is read-only; nothing writes through the view
            t = torch.frombuffer(self._map, dtype=e.dtype, count=count, offset=self._data_start + e.begin)
        return t.view(e.shape)

    def close(self) -> None:
        # Tensors that still view the mapping keep it alive; closing the file is enough.
        self._file.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata: Dict[str, str] = None) -> None:
    """Write ``(name, tensor)`` pairs in the order given.  The data section starts on an
    8-byte boundary, as the format asks."""
    items = [(n, t.detach().cpu().contiguous()) for n, t in tensors]
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsFormatError(f"cannot store dtype {t.dtype} ({name})")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
