"""The parts a layer is put together from, their interfaces and their registries.

A part is built from a ``PartSpec`` (its sizes and constants), a tensor-name prefix, the
loaded tensors and the run's ``Runtime`` (device and compute dtype).  It never sees the
model's configuration, so no part knows which model it is in.  A new part is a class with
the interface below, registered under a name with ``register_mixer`` / ``register_feed_forward``
/ ``register_norm`` / ``register_position`` / ``register_arrangement``; a ``LayerSpec`` then
names it.

ExiledOfCode/KuiperLLama's counterpart is its op layer (kuiper/include/op/layer.h:25-188):
layers with stored inputs and outputs wired by the model class, with eps, theta and head
counts partly compiled in.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch

from ..cache import CacheView, KVRequest, StateRequest
from ..config.spec import PartSpec
from ..weights.loader import TensorDecl


@dataclass(frozen=True)
class Runtime:
    """Where and in which precision a model runs.  ``dtype`` is float32 (everything in true
    32-bit arithmetic) or bfloat16 (serving: bfloat16 storage, 32-bit accumulation)."""
    device: torch.device
    dtype: torch.dtype


@dataclass
class StepContext:
    """One step's batch as the parts see it: packed tokens of several sequences.

    ``n_tokens`` rows are real; tensors may be longer (padding rows have token_slot -1 and
    write nothing).  All tensors are int32 on the device."""
    n_tokens: int                 # rows the kernels run (real tokens plus padding rows)
    n_seqs: int
    token_ids: torch.Tensor       # [n_tokens]
    positions: torch.Tensor       # [n_tokens] absolute position of each token in its sequence
    token_slot: torch.Tensor      # [n_tokens] cache slot of each token's sequence, -1 for padding
    seq_slots: torch.Tensor       # [n_seqs]
    seq_starts: torch.Tensor      # [n_seqs] tokens the sequence held before this step
    seq_new: torch.Tensor         # [n_seqs] tokens of the sequence in this step
    cu_tokens: torch.Tensor       # [n_seqs + 1] first row of each sequence in the packed batch
    is_decode: bool               # every sequence brings exactly one token
    max_new: int                  # host copy: longest run of new tokens
    max_context: int              # host copy: longest sequence after this step
    host_slots: List[int]         # host copies for parts that plan their launches
    host_starts: List[int]
    host_new: List[int]
    # The engine's class of max_context (0 up to 16 cache pages, then one per doubling).  A captured
    # decode step is replayed for steps of its class only, so a decode launch may be planned by this
    # number; a plan made from max_context itself would go stale inside a graph.
    context_class: int = 0
    # Set by the block around a call of a mixer or feed-forward that says it ``may_accumulate``:
    # the float32 residual stream its result is to be added to, with the norm that will read the
    # stream next.  Such a part may add the result itself (inside its last product) and return
    # ``Accumulated`` instead of a tensor.
    residual_sink: Optional["StreamSink"] = None
    # Set by the model before a block runs: the norm that will receive the block's pending result
    # (the next scheduled block's first norm, or the final norm), and whether this step may fold
    # the residual stream into the products at all.
    next_norm: Optional["Norm"] = None
    allow_stream_fusion: bool = False


@dataclass
class StreamSink:
    residual: torch.Tensor        # float32 [n_tokens, hidden], updated in place
    norm: "Norm"                  # the norm that reads it next; it has ``weight`` (float32 [hidden]) and ``eps``


@dataclass
class Accumulated:
    """A part's result that is already in the residual stream.  ``ss`` holds, in pieces
    [pieces, 64], the sum of squares of every row of the stream after the addition, and
    ``scaled`` the new rows times the weight of ``norm`` in the compute dtype: together what
    that norm needs to hand normalised rows on without a pass of its own."""
    ss: torch.Tensor
    scaled: torch.Tensor
    norm: "Norm"


@dataclass
class NormedLazy:
    """Rows that a norm has not finished: y = scaled * rsqrt(sum(x^2) / width + eps), with
    ``scaled`` = weight * x in the compute dtype and sum(x^2) known in pieces.  A product of few
    tokens multiplies by the factor in its epilogue (it is one number per row, so it commutes
    with the product); everything else calls ``dense()``."""
    residual: torch.Tensor
    weight: torch.Tensor
    eps: float
    ss: torch.Tensor
    scaled: torch.Tensor
    dtype: torch.dtype

    @property
    def shape(self):
        return self.residual.shape

    @property
    def device(self):
        return self.residual.device

    def dense(self) -> torch.Tensor:
        from ..csrc import ops
        out = torch.empty(self.residual.shape, dtype=self.dtype, device=self.residual.device)
        ops.add_rmsnorm(self.residual, None, self.weight, out, self.eps)
        return out


class Part:
    """Base of all parts."""

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        """The tensors the part reads: name -> shape, role and random initialisation."""
        return {}

    def __init__(self, spec: PartSpec, prefix: str, tensors: Dict[str, torch.Tensor], runtime: Runtime):
        self.spec = spec
        self.prefix = prefix
        self.runtime = runtime


class Norm(Part):
    """``forward(residual, delta, n_rows, rows)``: adds ``delta`` (None, [n, hidden] in the
    compute dtype, or float32 partial sums [S, n, hidden]) to the float32 residual stream in
    place and returns the normalised rows in the compute dtype.  With ``rows`` only those rows
    are produced and the residual is left unchanged.

    A norm that sets ``accepts_accumulated`` also takes ``Accumulated`` as delta (the sum is in
    the stream already) and may then return ``NormedLazy`` for the part that follows."""

    accepts_accumulated = False

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], n_rows: int,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """A position encoding either rotates queries and keys inside the mixer (``rotary()``
    returns the inverse frequencies and the rotated width) or changes the embeddings before
    the first layer (``add_to_embeddings``), or both."""

    def rotary(self) -> Optional[tuple]:
        return None

    def add_to_embeddings(self, residual: torch.Tensor, step: StepContext) -> None:
        return None


class Mixer(Part):
    """Mixes information between the tokens of a sequence.  ``kv_request`` / ``state_request``
    say what the cache must hold for one execution; ``forward`` gets the normalised rows
    [n_tokens, hidden], the step and its view of the cache, and returns [n_tokens, hidden]
    in the compute dtype (the block adds it to the residual stream).  It may instead return
    float32 partial sums [S, n_tokens, hidden] whose sum over S is that result; the norm
    that follows adds them in ascending order."""

    # A part that sets these takes ``NormedLazy`` as input, and may add its result into
    # ``step.residual_sink`` itself and return ``Accumulated``.
    accepts_lazy_norm = False
    may_accumulate = False

    def __init__(self, spec, prefix, tensors, runtime, position: Optional[PositionEncoding] = None):
        super().__init__(spec, prefix, tensors, runtime)
        self.position = position

    def kv_request(self) -> Optional[KVRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    def forward(self, x: torch.Tensor, step: StepContext, cache: CacheView) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    """``forward(x, step)``: [n_tokens, hidden] -> [n_tokens, hidden], token by token (or
    float32 partial sums [S, n_tokens, hidden], as a mixer may)."""

    accepts_lazy_norm = False
    may_accumulate = False

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        raise NotImplementedError


# ----------------------------------------------------------------------------- registries

_REGISTRIES: Dict[str, Dict[str, type]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position": {},
                                           "arrangement": {}}


def _register(family: str, name: str) -> Callable[[type], type]:
    def deco(cls: type) -> type:
        _REGISTRIES[family][name] = cls
        return cls
    return deco


def register_mixer(name: str): return _register("mixer", name)
def register_feed_forward(name: str): return _register("feed_forward", name)
def register_norm(name: str): return _register("norm", name)
def register_position(name: str): return _register("position", name)
def register_arrangement(name: str): return _register("arrangement", name)


def part_class(family: str, name: str) -> type:
    try:
        return _REGISTRIES[family][name]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[family])) or "(none)"
        raise KeyError(f"no {family} is registered as {name!r}; registered: {known}") from None
