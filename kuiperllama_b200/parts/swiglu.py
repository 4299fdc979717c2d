"""The dense SwiGLU feed-forward."""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import FeedForward, NormedLazy, Runtime, StepContext, register_feed_forward
from .linear import Linear


@register_feed_forward("swiglu")
class SwiGLUFeedForward(FeedForward):
    """f = W_down (silu(W_gate n) * W_up n), silu(g) = g / (1 + exp(-g)), no bias
    (ExiledOfCode/KuiperLLama kuiper/source/model/llama3.cpp:692-718, swiglu_kernel.cu:18-21;
    gate = w1, up = w3, down = w2, tools/export_llama3.py:583-585).  Gate and up are stacked
    into one matrix at load (and the activation is applied in that product's epilogue where the
    tensor-core kernel runs).  Spec: ``hidden_size``, ``intermediate_size``, ``names``."""

    accepts_lazy_norm = True
    may_accumulate = True

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        hid, inter, n = spec["hidden_size"], spec["intermediate_size"], spec["names"]
        return {prefix + n["gate"]: TensorDecl((inter, hid)), prefix + n["up"]: TensorDecl((inter, hid)),
                prefix + n["down"]: TensorDecl((hid, inter))}

    def __init__(self, spec, prefix, tensors, runtime: Runtime):
        super().__init__(spec, prefix, tensors, runtime)
        self.hidden, self.inter = int(spec["hidden_size"]), int(spec["intermediate_size"])
        n = spec["names"]
        dev, dt = runtime.device, runtime.dtype
        gate, up = (tensors[prefix + n[k]].to(device=dev, dtype=dt) for k in ("gate", "up"))
        # One product for gate and up.  Where the tensor-core kernel can apply the activation in
        # its epilogue, the rows are stored as alternating blocks of 64 gate and 64 up rows.
        self.fused = ops.swiglu_fusable(self.hidden, self.inter, dt)
        self.gate_up = Linear(ops.interleave_gate_up(gate, up) if self.fused else torch.cat([gate, up], dim=0), runtime)
        del gate, up
        self.down = Linear(tensors[prefix + n["down"]], runtime)

    def forward(self, x, step: StepContext):
        if isinstance(x, NormedLazy):
            if self.fused and ops.stream_fusable(x.shape[0], self.gate_up.weight):
                # gate, up and the activation in one kernel that also finishes the norm before them
                act = ops.gemm_skinny_stream(self.gate_up.weight, x.scaled, row_scale=(x.ss, x.eps), swiglu=True)
                return self.down.forward(act, allow_partials=True, sink=getattr(step, "residual_sink", None))
            x = x.dense()
        act = torch.empty((x.shape[0], self.inter), dtype=self.runtime.dtype, device=x.device)
        if self.fused:
            ops.matmul_swiglu(x, self.gate_up.weight, act)
        else:
            ops.swiglu(self.gate_up.forward(x), act)
        return self.down.forward(act, allow_partials=True, sink=getattr(step, "residual_sink", None))
