"""Grouped-query attention over the paged cache: the mixer of the Llama decoder."""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..cache import CacheView, KVRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import Mixer, PositionEncoding, Runtime, StepContext, register_mixer
from .linear import Linear


@register_mixer("attention")
class AttentionMixer(Mixer):
    """q = Wq n, k = Wk n, v = Wv n (no bias); rotate q and k by position; append k, v to the
    cache; per head softmax((q . K) * scale) V over the keys up to the token's own position,
    head h reading kv head h // (H / KV); out = Wo o
    (ExiledOfCode/KuiperLLama kuiper/source/model/llama3.cpp:610-639, 651-675;
    mha_kernel.cu:61,74-106).

    Spec: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``window`` (None:
    every earlier key), ``scale`` (default head_dim ** -0.5, what KuiperLLama fixes,
    mha_kernel.cu:61) and ``names`` of the four projection tensors.  The three input
    projections are stacked into one matrix at load so that one product makes q, k and v.
    """

    accepts_lazy_norm = True      # the q/k/v product can normalise the stream's rows itself
    may_accumulate = True         # the output product can add into the stream itself

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        hid, H, KV, hd = spec["hidden_size"], spec["num_heads"], spec["num_kv_heads"], spec["head_dim"]
        n = spec["names"]
        return {prefix + n["q"]: TensorDecl((H * hd, hid)), prefix + n["k"]: TensorDecl((KV * hd, hid)),
                prefix + n["v"]: TensorDecl((KV * hd, hid)), prefix + n["o"]: TensorDecl((hid, H * hd))}

    def __init__(self, spec, prefix, tensors, runtime: Runtime, position: Optional[PositionEncoding] = None):
        super().__init__(spec, prefix, tensors, runtime, position)
        self.hidden = int(spec["hidden_size"])
        self.H, self.KV, self.hd = int(spec["num_heads"]), int(spec["num_kv_heads"]), int(spec["head_dim"])
        if self.H % self.KV:
            raise ValueError(f"{self.H} heads are not a multiple of {self.KV} kv heads")
        if self.hd % 16 or self.hd > 256:
            raise ValueError(f"head_dim {self.hd} is not supported by the attention kernels "
                             "(multiples of 16 up to 256)")
        self.window = spec.get("window")
        self.scale = float(spec.get("scale") or 1.0 / math.sqrt(float(self.hd)))
        n = spec["names"]
        dev, dt = runtime.device, runtime.dtype
        stacked = torch.cat([tensors[prefix + n[k]].to(device=dev, dtype=dt) for k in ("q", "k", "v")], dim=0)
        self.qkv = Linear(stacked, runtime)
        self.o = Linear(tensors[prefix + n["o"]], runtime)
        rot = position.rotary() if position is not None else None
        self.inv_freq, self.rotary_dim = rot if rot is not None else (None, 0)

    def kv_request(self) -> Optional[KVRequest]:
        return KVRequest(kv_heads=self.KV, head_dim=self.hd, kind="full", window=self.window)

    def forward(self, x: torch.Tensor, step: StepContext, cache: CacheView) -> torch.Tensor:
        n = step.n_tokens
        qkv = self.qkv.forward(x, allow_partials=True)
        if (step.is_decode and cache.writable and n == step.n_seqs and self.inv_freq is not None
                and ops.decode_fusable(self.runtime.dtype, self.hd, self.rotary_dim, self.H, self.KV)):
            # a decode step: rotation, cache write, attention and the merge of the splits in one kernel
            attn = torch.empty((n, self.H * self.hd), dtype=self.runtime.dtype, device=x.device)
            ops.attention_decode_fused(qkv, self.inv_freq, attn, cache.k, cache.v, cache.block_table, step, self.H, self.KV,
                                       self.hd, self.scale, int(self.window or 0))
            return self.o.forward(attn, allow_partials=True, sink=step.residual_sink)
        parts = None
        if qkv.dim() == 3:                                         # pieces of the product: the rotary kernel adds them
            parts, qkv = qkv, torch.empty(qkv.shape[1:], dtype=self.runtime.dtype, device=x.device)
        ops.rope_kv_write(qkv, self.inv_freq, self.rotary_dim, step.positions, step.token_slot, cache.block_table,
                          cache.k if cache.writable else None, cache.v if cache.writable else None,
                          self.H, self.KV, self.hd, partials=parts)
        attn = torch.empty((n, self.H * self.hd), dtype=self.runtime.dtype, device=x.device)
        ops.attention(qkv, qkv.shape[1], attn, cache.k, cache.v, cache.block_table, step, self.H, self.KV, self.hd,
                      self.scale, int(self.window or 0))
        return self.o.forward(attn, allow_partials=True, sink=step.residual_sink)
