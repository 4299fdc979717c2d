"""RMSNorm fused with the residual add."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import Accumulated, Norm, NormedLazy, Runtime, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """out = w * x * rsqrt(mean(x^2) + eps) on x = residual + delta, statistics in 32 bits
    (ExiledOfCode/KuiperLLama rmsnorm_kernel.cu:70-106; the add is its add_kernel.cu:4-12,
    fused here).  ``size``, ``eps`` and the tensor's ``name`` come from the spec."""

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        return {prefix + spec["name"]: TensorDecl((spec["size"],), role="vector", init="one_plus_normal")}

    def __init__(self, spec, prefix, tensors, runtime: Runtime):
        super().__init__(spec, prefix, tensors, runtime)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = tensors[prefix + spec["name"]].to(device=runtime.device, dtype=torch.float32).contiguous()

    accepts_accumulated = True

    def forward(self, residual: torch.Tensor, delta, n_rows: int, rows: Optional[torch.Tensor] = None):
        if isinstance(delta, Accumulated):
            # the stream holds the sum already; if the rows times this norm's weight came with it,
            # the product that follows only has to apply 1 / rms
            if rows is None and delta.norm is self and delta.scaled is not None:
                return NormedLazy(residual, self.weight, self.eps, delta.ss, delta.scaled, self.runtime.dtype)
            delta = None
        n_out = rows.numel() if rows is not None else residual.shape[0]
        out = torch.empty((n_out, self.size), dtype=self.runtime.dtype, device=residual.device)
        ops.add_rmsnorm(residual, delta, self.weight, out, self.eps, rows)
        return out
