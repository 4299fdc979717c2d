"""The decode-attention entry point that allocates nothing, called through its exported C
symbol (``kl_attention_decode_noalloc`` in the attention_decode library), against the regular
entry point, on two calls in a row.

It exists for programs that cannot call cudaMalloc when they need attention (all device
memory already handed to a pool of their own, or a loop that cannot afford an allocation):
the scratch for the split-KV partial results is a fixed 4 MiB array inside the library
instead of a buffer from the caller.  This file is collected last, so a run that stops at the
first failure has already run every other test.
"""
from __future__ import annotations

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


def _problem(seed, rows, H, KV, hd, max_len):
    """Queries, a scattered paged cache with random lengths, and the index arrays."""
    g = torch.Generator().manual_seed(seed)
    blocks = (max_len + PAGE - 1) // PAGE
    n_pages = rows * blocks + 2
    table = torch.randperm(n_pages, generator=g)[: rows * blocks].view(rows, blocks).to(torch.int32).to(DEV)
    k = torch.randn(n_pages, KV, PAGE, hd, generator=g).bfloat16().to(DEV)
    v = torch.randn(n_pages, KV, PAGE, hd, generator=g).bfloat16().to(DEV)
    q = torch.randn(rows, H * hd, generator=g).bfloat16().to(DEV)
    pos = torch.randint(0, max_len, (rows,), generator=g).to(torch.int32).to(DEV)
    slot = torch.arange(rows, dtype=torch.int32, device=DEV)
    return q, k, v, table, pos, slot


def _float64_attention(q, k, v, table, pos, H, KV, hd):
    """softmax(q . K / sqrt(hd)) V per row and head over the row's keys 0..pos, in float64."""
    rows = q.shape[0]
    out = torch.zeros(rows, H * hd, dtype=torch.float64)
    qd, kd, vd, tb = q.double().cpu().view(rows, H, hd), k.double().cpu(), v.double().cpu(), table.cpu()
    for r in range(rows):
        n = int(pos[r]) + 1
        pages = tb[r, : (n + PAGE - 1) // PAGE].long()
        for h in range(H):
            g = h // (H // KV)
            keys = kd[pages, g].reshape(-1, hd)[:n]
            vals = vd[pages, g].reshape(-1, hd)[:n]
            p = torch.softmax(keys @ qd[r, h] / math.sqrt(hd), dim=0)
            out[r, h * hd:(h + 1) * hd] = p @ vals
    return out


def _call_noalloc(lib, q, k, v, table, pos, slot, out, rows, H, KV, hd, splits):
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    return lib.kl_attention_decode_noalloc(
        ptr(q), q.shape[1], ptr(out), ptr(k), ptr(v), ptr(table), table.shape[1], ptr(pos), ptr(slot), rows, H, KV, hd,
        ctypes.c_float(1.0 / math.sqrt(hd)), 0, splits, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_entry_point_without_allocation_matches_the_regular_one():
    from kuiperllama_b200.csrc import build, ops
    lib = ctypes.CDLL(build.ensure_built("attention_decode"))      # the exported C symbol, not the Python wrapper
    rows, H, KV, hd, splits = 6, 8, 2, 128, 5
    for call, seed in enumerate((21, 22)):                          # two calls in a row share the built-in scratch
        q, k, v, table, pos, slot = _problem(seed, rows, H, KV, hd, max_len=700)
        want = torch.empty(rows, H * hd, device=DEV, dtype=torch.bfloat16)
        ops.attention_decode(q, q.shape[1], want, k, v, table, pos, slot, rows, H, KV, hd, 1.0 / math.sqrt(hd), 0, splits)
        got = torch.full_like(want, 9.0)
        before = torch.cuda.memory_allocated()
        rc = _call_noalloc(lib, q, k, v, table, pos, slot, got, rows, H, KV, hd, splits)
        torch.cuda.synchronize()
        assert rc == 0, f"call {call} returned {rc}"
        assert torch.cuda.memory_allocated() == before, "the entry point allocated through torch"
        # the same kernels with the same cuts: not a bit may differ (a wrong place for one cut's
        # running maximum and sum in the built-in scratch would show here)
        assert torch.equal(got, want), f"call {call}: max abs difference {float((got.float() - want.float()).abs().max())}"
        # and against float64 arithmetic on the host, within bfloat16's rounding of the output
        ref = _float64_attention(q, k, v, table, pos, H, KV, hd)
        err = float((got.double().cpu() - ref).abs().max())
        assert err <= 2.0 ** -8 * float(ref.abs().max()) + 1e-3, f"call {call}: {err} from the float64 result"
    # a request beyond the built-in scratch is refused, and nothing is written
    big_rows, big_splits = 64, 32
    q, k, v, table, pos, slot = _problem(23, big_rows, H, KV, hd, max_len=64)
    out = torch.full((big_rows, H * hd), 9.0, device=DEV, dtype=torch.bfloat16)
    assert big_rows * H * big_splits * (hd + 2) > (1 << 20)
    assert _call_noalloc(lib, q, k, v, table, pos, slot, out, big_rows, H, KV, hd, big_splits) == -2
    torch.cuda.synchronize()
    assert float((out.float() - 9.0).abs().max()) == 0.0
