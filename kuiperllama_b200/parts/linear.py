"""y = x W^T: the one place that picks a matrix-product kernel.

Weights are [out, in] row-major without bias, as in ExiledOfCode/KuiperLLama
(kuiper/source/op/kernels/cuda/matmul_kernel.cu:6-54, MatmulLayer has_bias=false,
kuiper/include/op/matmul.h:12-13).  In a float32 run every product uses the plain 32-bit
kernel.  In a bfloat16 run the kernel is picked by shape; each of them accumulates in
32 bits.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from .base import Runtime


class Linear:
    def __init__(self, weight: torch.Tensor, runtime: Runtime):
        assert weight.dim() == 2
        self.weight = weight.to(device=runtime.device, dtype=runtime.dtype).contiguous()
        self.out_features, self.in_features = self.weight.shape
        self.runtime = runtime

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
                out: Optional[torch.Tensor] = None, allow_partials: bool = False) -> torch.Tensor:
        """[m, in] -> [m, out].  With ``allow_partials`` the result may instead be float32
        partial sums [S, m, out] (a product of few tokens whose K range was cut over CTAs);
        the norm and the rotary kernel add such pieces themselves, which saves a pass."""
        m = x.shape[0]
        if allow_partials and out is None:
            parts = ops.gemm_skinny_partials(x, self.weight)
            if parts is not None:
                return parts
        if out is None:
            out = torch.empty((m, self.out_features), dtype=out_dtype or self.runtime.dtype, device=x.device)
        ops.matmul(x, self.weight, out)
        return out
