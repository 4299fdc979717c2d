"""Where a step's time goes, without a profiler: per-kernel CUDA-event timing and NVTX ranges.

ExiledOfCode/KuiperLLama's Llama path has only unused TICK/TOCK wall-clock macros
(kuiper/include/base/tick.h:7-12); its Qwen2 model sums per-op times into an ``OpProfileStat``
(kuiper/include/model/qwen2.h:13-18).  This is that idea for the kernels of this package:

    from kuiperllama_b200 import profiling
    with profiling.kernel_timing() as times:        # every entry point of csrc/ops.py between two events
        model.generate(...)
    print(times.report())

Timing puts an event pair around every call and reads them at the end, so kernels no longer
overlap their neighbours' tails the way they do in a normal run (compare shares, not sums), and
steps replayed from CUDA graphs are one launch and show up as nothing: use it with
``use_graphs=False``.  ``KL_NVTX=1`` in the environment wraps every entry point in an NVTX range
named after it, for a system profiler's timeline.
"""
from __future__ import annotations

import contextlib
import functools
import os
from collections import defaultdict
from typing import Dict, List, Tuple

import torch

from .csrc import ops

# The entry points of csrc/ops.py that launch kernels.
KERNEL_ENTRY_POINTS = ("embedding", "add_rmsnorm", "swiglu", "rope_kv_write", "attention_simt", "gemm_simt", "argmax_rows",
                       "sample_rows", "token_logprob", "logit_transform", "gemm_tcgen05", "gemm_skinny_stream",
                       "gemm_skinny_partials", "gemm_skinny", "attention_decode", "attention_mma", "attention_tcgen05",
                       "attention_decode_fused")


class KernelTimes:
    def __init__(self):
        self.pairs: List[Tuple[str, "torch.cuda.Event", "torch.cuda.Event"]] = []

    def totals(self) -> Dict[str, Tuple[int, float]]:
        """name -> (calls, milliseconds); synchronises."""
        torch.cuda.synchronize()
        out: Dict[str, List[float]] = defaultdict(lambda: [0, 0.0])
        for name, a, b in self.pairs:
            out[name][0] += 1
            out[name][1] += a.elapsed_time(b)
        return {k: (int(v[0]), float(v[1])) for k, v in out.items()}

    def report(self) -> str:
        t = self.totals()
        whole = sum(ms for _, ms in t.values()) or 1.0
        lines = [f"{ms:10.3f} ms {100 * ms / whole:5.1f} %  x{n:<6d} {name}"
                 for name, (n, ms) in sorted(t.items(), key=lambda kv: -kv[1][1])]
        return "\n".join(lines + [f"{whole:10.3f} ms total over {sum(n for n, _ in t.values())} calls"])


def _wrap(module, names, make):
    saved = {}
    for name in names:
        fn = getattr(module, name)
        saved[name] = fn
        setattr(module, name, make(name, fn))
    return saved


@contextlib.contextmanager
def kernel_timing():
    """Time every kernel entry point of ``csrc/ops.py`` called inside the block."""
    times = KernelTimes()

    def make(name, fn):
        @functools.wraps(fn)
        def timed(*args, **kwargs):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            try:
                return fn(*args, **kwargs)
            finally:
                b.record()
                times.pairs.append((name, a, b))
        return timed

    saved = _wrap(ops, KERNEL_ENTRY_POINTS, make)
    try:
        yield times
    finally:
        for name, fn in saved.items():
            setattr(ops, name, fn)


def enable_nvtx() -> None:
    """Wrap every kernel entry point in an NVTX range (until the process ends)."""
    def make(name, fn):
        @functools.wraps(fn)
        def ranged(*args, **kwargs):
            torch.cuda.nvtx.range_push(f"kl.{name}")
            try:
                return fn(*args, **kwargs)
            finally:
                torch.cuda.nvtx.range_pop()
        return ranged

    if not getattr(ops, "_nvtx_enabled", False):
        _wrap(ops, KERNEL_ENTRY_POINTS, make)
        ops._nvtx_enabled = True


if os.environ.get("KL_NVTX", "") not in ("", "0"):
    enable_nvtx()
