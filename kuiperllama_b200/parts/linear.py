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
from .base import Accumulated, NormedLazy, Runtime


class Linear:
    def __init__(self, weight: torch.Tensor, runtime: Runtime):
        assert weight.dim() == 2
        self.weight = weight.to(device=runtime.device, dtype=runtime.dtype).contiguous()
        self.out_features, self.in_features = self.weight.shape
        self.runtime = runtime

    def forward(self, x, out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
                allow_partials: bool = False, sink=None):
        """[m, in] -> [m, out].  With ``allow_partials`` the result may instead be float32
        partial sums [S, m, out] (a product of few tokens whose K range was cut over CTAs);
        the norm and the rotary kernel add such pieces themselves, which saves a pass.

        ``x`` may be ``NormedLazy`` (rows of the residual stream times a norm's weight, 1 / rms
        still to be applied): a product of few tokens applies it in its epilogue, anything else
        asks for the dense rows.  With ``sink`` (the float32 residual stream and the norm that
        reads it next) such a product adds its result into the stream itself and returns
        ``Accumulated``."""
        m = x.shape[0]
        if sink is not None and m > ops.STREAM_SINK_MAX_ROWS:
            sink = None
        if allow_partials and out is None and ops.stream_fusable(m, self.weight) and (
                isinstance(x, NormedLazy) or sink is not None):
            lazy = isinstance(x, NormedLazy)
            got = ops.gemm_skinny_stream(self.weight, x.scaled if lazy else x, row_scale=(x.ss, x.eps) if lazy else None,
                                         sink=(sink.residual, sink.norm.weight) if sink is not None else None)
            return Accumulated(got[0], got[1], sink.norm) if sink is not None else got
        if isinstance(x, NormedLazy):
            x = x.dense()
        if allow_partials and out is None:
            parts = ops.gemm_skinny_partials(x, self.weight)
            if parts is not None:
                return parts
        if out is None:
            out = torch.empty((m, self.out_features), dtype=out_dtype or self.runtime.dtype, device=x.device)
        ops.matmul(x, self.weight, out)
        return out
