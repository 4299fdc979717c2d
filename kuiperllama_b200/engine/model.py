"""A decoder put together from a ``ModelSpec``: embedding, a schedule of layer executions,
final norm and classifier.  It is architecture-neutral: the Llama configuration produces a
``ModelSpec`` and nothing here asks which architecture that was.

Forward of one step (ExiledOfCode/KuiperLLama kuiper/source/model/llama3.cpp:146-166,
721-730, for one token of one sequence there): x = E[token]; every scheduled layer in
order; final RMSNorm and logits = W_cls x at the wanted rows only.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Tuple

import torch

from ..cache import KVRequest, SequenceCache, StateRequest
from ..config.spec import LayerSpec, ModelSpec
from ..csrc import ops
from ..parts.base import Runtime, StepContext, part_class
from ..parts.linear import Linear
from ..weights.loader import TensorDecl


def model_manifest(spec: ModelSpec) -> Dict[str, TensorDecl]:
    """Every tensor the model reads, gathered from its parts."""
    m: Dict[str, TensorDecl] = {spec.embedding_name: TensorDecl((spec.vocab_size, spec.hidden_size))}
    for layer in spec.layers:
        for family, ps in (("norm", layer.mixer_norm), ("mixer", layer.mixer),
                           ("norm", layer.feed_forward_norm), ("feed_forward", layer.feed_forward)):
            m.update(part_class(family, ps.kind).manifest(ps, layer.prefix))
        if layer.position is not None:
            m.update(part_class("position", layer.position.kind).manifest(layer.position, layer.prefix))
    m.update(part_class("norm", spec.final_norm.kind).manifest(spec.final_norm, spec.final_norm_prefix))
    if spec.lm_head_name is not None:
        m[spec.lm_head_name] = TensorDecl((spec.vocab_size, spec.hidden_size))
    return m


def ignorable_tensor_suffixes(spec: ModelSpec) -> Tuple[str, ...]:
    """Name endings a checkpoint may hold without the model reading them; the architecture's
    configuration lists them in its ``ModelSpec``."""
    return tuple(spec.ignorable_suffixes)


class DecoderModel:
    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        spec.validate()
        self.spec = spec
        self.runtime = runtime
        dev, dt = runtime.device, runtime.dtype
        self.embedding = tensors[spec.embedding_name].to(device=dev, dtype=dt).contiguous()
        self.blocks = [self._build_layer(layer, tensors) for layer in spec.layers]
        self.final_norm = part_class("norm", spec.final_norm.kind)(spec.final_norm, spec.final_norm_prefix, tensors, runtime)
        if spec.lm_head_name is None:
            self.lm_head = Linear(self.embedding, runtime)    # tied: the same storage, no copy
        else:
            self.lm_head = Linear(tensors[spec.lm_head_name], runtime)
        self.error_flag = ops.error_word(dev)               # shared per device; read with the status word in one copy
        # Option (bfloat16 decode steps of a few tokens): a block lets its products add into the residual
        # stream themselves and finish the norms in their epilogues (see parts/block.py).  It rounds
        # the normalised rows differently from the norm kernel (bf16(x * w) * r instead of
        # bf16(x * r * w)), so results would change in the last bit with the number of rows of a step,
        # padding rows included; it is therefore off unless asked for.
        self.stream_fusion = False

    def _build_layer(self, layer: LayerSpec, tensors):
        rt = self.runtime
        position = None
        if layer.position is not None:
            position = part_class("position", layer.position.kind)(layer.position, layer.prefix, tensors, rt)
        mixer = part_class("mixer", layer.mixer.kind)(layer.mixer, layer.prefix, tensors, rt, position)
        ffn = part_class("feed_forward", layer.feed_forward.kind)(layer.feed_forward, layer.prefix, tensors, rt)
        n1 = part_class("norm", layer.mixer_norm.kind)(layer.mixer_norm, layer.prefix, tensors, rt)
        n2 = part_class("norm", layer.feed_forward_norm.kind)(layer.feed_forward_norm, layer.prefix, tensors, rt)
        block = part_class("arrangement", layer.arrangement)(n1, mixer, n2, ffn)
        block.position = position
        return block

    # ------------------------------------------------------------------ cache
    def cache_requests(self) -> Tuple[List[Optional[KVRequest]], List[Optional[StateRequest]], List[Optional[int]]]:
        kv, st, src = [], [], []
        for e in self.spec.schedule:
            mixer = self.blocks[e.layer].mixer
            kv.append(mixer.kv_request())
            st.append(mixer.state_request())
            src.append(e.cache_from)
        return kv, st, src

    def new_cache(self, max_tokens: int, max_seq_len: Optional[int] = None, max_slots: Optional[int] = None,
                  window_step_tokens: Optional[int] = None) -> SequenceCache:
        kv, st, src = self.cache_requests()
        return SequenceCache(kv, st, src, max_tokens=max_tokens,
                             max_seq_len=max_seq_len or self.spec.max_positions,
                             dtype=self.runtime.dtype, device=self.runtime.device, max_slots=max_slots,
                             window_step_tokens=window_step_tokens)

    def cache_bytes_per_token(self) -> int:
        """Bytes of keys and values one token of one sequence takes over all executions that own
        storage (per-slot state of fixed size is not counted)."""
        kv, _, src = self.cache_requests()
        esize = torch.empty(0, dtype=self.runtime.dtype).element_size()
        return sum(2 * r.kv_heads * r.head_dim * esize for r, s in zip(kv, src) if r is not None and s is None)

    # ------------------------------------------------------------------ forward
    def hidden_states(self, step: StepContext, cache: SequenceCache) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """Run embedding and all scheduled layers: the float32 residual stream and the last
        feed-forward's output that is still to be added to it."""
        step.allow_stream_fusion = self.stream_fusion and step.is_decode
        residual = torch.empty((step.n_tokens, self.spec.hidden_size), dtype=torch.float32, device=self.runtime.device)
        ops.embedding(step.token_ids[:step.n_tokens], self.embedding, residual, self.error_flag,
                      scale=1.0 if self.spec.embedding_multiplier is None else float(self.spec.embedding_multiplier))
        first = self.blocks[self.spec.schedule[0].layer]
        if getattr(first, "position", None) is not None:
            first.position.add_to_embeddings(residual, step)
        pending = None
        schedule = self.spec.schedule
        for i, entry in enumerate(schedule):
            following = self.blocks[schedule[i + 1].layer] if i + 1 < len(schedule) else None
            step.next_norm = getattr(following, "mixer_norm", None) if following is not None else self.final_norm
            residual, pending = self.blocks[entry.layer].forward(residual, pending, step, cache.view(i))
        step.next_norm = None
        return residual, pending

    def logits(self, residual: torch.Tensor, pending: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [len(rows), vocab] of the given rows of the step."""
        x = self.final_norm.forward(residual, pending, rows.numel(), rows)
        out = self.lm_head.forward(x, out_dtype=torch.float32)
        if self.spec.logit_scale is not None or self.spec.logit_softcap is not None:
            ops.logit_transform(out, 1.0 if self.spec.logit_scale is None else float(self.spec.logit_scale),
                                float(self.spec.logit_softcap or 0.0))
        return out

    def forward(self, step: StepContext, cache: SequenceCache, rows: torch.Tensor) -> torch.Tensor:
        residual, pending = self.hidden_states(step, cache)
        return self.logits(residual, pending, rows)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for t in self._weights():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def _weights(self):
        yield self.embedding
        yield self.lm_head.weight
        for b in self.blocks:
            for part in (b.mixer_norm, b.mixer, b.feed_forward_norm, b.feed_forward):
                for v in vars(part).values():
                    if isinstance(v, torch.Tensor):
                        yield v
                    elif isinstance(v, Linear):
                        yield v.weight
