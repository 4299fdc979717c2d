"""Architecture-neutral description of a decoder: what the engine builds a model from.

An architecture's typed configuration (for instance ``LlamaConfig``) turns itself into a
``ModelSpec``.  Everything below the configuration (weights, parts, cache, step function)
reads only the ``ModelSpec``; none of it knows which architecture it came from.

* ``PartSpec``    one part (a mixer, a feed-forward, a norm, a position encoding): the
                  name it is registered under and its sizes and constants.
* ``LayerSpec``   one layer: the arrangement of its parts in a block, the parts, and the
                  prefix of its tensor names.
* ``ScheduleEntry`` one execution of a layer.  The order in which layers run is the list
                  ``ModelSpec.schedule``; it may name a layer twice (weights are shared,
                  each execution has a cache of its own) or let an execution read the cache
                  that an earlier execution wrote (``cache_from``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    prefix: str                      # tensor-name prefix, e.g. "model.layers.3."
    arrangement: str                 # registered block arrangement, e.g. "pre_norm"
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    position: Optional[PartSpec]     # position encoding handed to the mixer (None: none)


@dataclass(frozen=True)
class ScheduleEntry:
    layer: int                       # index into ModelSpec.layers
    cache_from: Optional[int] = None # index of an EARLIER schedule entry whose cache is read


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    embedding_name: str              # [vocab, hidden]
    final_norm: PartSpec
    final_norm_prefix: str
    lm_head_name: Optional[str]      # None: tied to the embedding table
    stop_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    # Tensor-name endings a checkpoint of this architecture may hold without the model reading them.
    ignorable_suffixes: Tuple[str, ...] = ()
    # Options that some decoders have around the layers; None leaves the step out.
    embedding_multiplier: Optional[float] = None     # x = multiplier * E[token]
    logit_scale: Optional[float] = None              # logits = scale * (W_cls x)
    logit_softcap: Optional[float] = None            # logits = cap * tanh(logits / cap), after the scale

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ValueError(f"logit_softcap must be positive, got {self.logit_softcap}")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule[{i}] names layer {e.layer}, but there are {len(self.layers)} layers")
            if e.cache_from is not None and not 0 <= e.cache_from < i:
                raise ValueError(f"schedule[{i}].cache_from={e.cache_from} must name an earlier schedule entry")
            if e.cache_from is not None and self.schedule[e.cache_from].cache_from is not None:
                raise ValueError(f"schedule[{i}].cache_from={e.cache_from} names an entry that owns no cache")


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(layer=i) for i in range(n_layers))
