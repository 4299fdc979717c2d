"""Time one kernel of the package alone on synthetic operands (CUDA events, median of
repeats, a buffer larger than L2 written between repeats), and print the achieved rate.

    python microbench.py gemm_skinny --m 8 --n 28672 --k 4096 [--swiglu]
    python microbench.py gemm_tcgen05 --m 2048 --n 6144 --k 4096
    python microbench.py attention_prefill --tokens 2048 --heads 32 --kv-heads 8 --head-dim 128 [--mma]
    python microbench.py attention_decode --batch 64 --context 640 --heads 32 --kv-heads 8 --head-dim 128
    python microbench.py attention_decode --batch 8 --context 516 --fused     (the decode step's form)
    python microbench.py decode_step --shape 8b --layers 4 --batch 32 --context 8300 [--splits 2]
        (decode steps of a few layers of one of bench.py's shapes, replayed from a CUDA graph; --splits
        fixes the number of pieces the decode attention cuts a sequence into, else the package's rule)
    python microbench.py prefill_step --shape 8b --layers 2 --tokens 2048
        (one prompt through a few layers, launched kernel by kernel: the case for a launch list)

It is also the small case that profiler captures of single kernels are taken on.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from kuiperllama_b200.csrc import ops  # noqa: E402

DEV = torch.device("cuda:0")


def _time(fn, repeats: int, flush: bool = True) -> float:
    scratch = torch.empty(192 << 20, dtype=torch.uint8, device=DEV) if flush else None
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(repeats):
        if scratch is not None:
            scratch.zero_()                                    # evict L2 (126 MB)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e-3)
    times.sort()
    return times[len(times) // 2]


def _paged(n_seqs: int, length: int, kv: int, hd: int):
    blocks = (length + ops.PAGE - 1) // ops.PAGE
    pages = n_seqs * blocks
    table = torch.randperm(pages).view(n_seqs, blocks).to(torch.int32).to(DEV)
    k = torch.randn(pages, kv, ops.PAGE, hd, device=DEV).bfloat16()
    v = torch.randn(pages, kv, ops.PAGE, hd, device=DEV).bfloat16()
    return table, k, v


def _decode_step(args) -> int:
    import bench
    import kuiperllama_b200 as kl
    from kuiperllama_b200.config import config_from_dict
    from kuiperllama_b200.engine import Engine, SequenceInput
    from kuiperllama_b200.engine.step import context_class
    base = {"8b": bench.LLAMA31_8B, "7b": bench.LLAMA2_7B, "1b": bench.LLAMA32_1B, "70b": bench.LLAMA3_70B}[args.shape]
    B, N, L = args.batch, args.context, args.layers
    cfg = dict(base, num_hidden_layers=L, max_position_embeddings=max(base["max_position_embeddings"], N + args.steps + 16))
    model = kl.random_model(config_from_dict(cfg), seed=0)
    rule = ops.decode_attention_splits
    if args.splits:
        ops.decode_attention_splits = lambda n_seqs, kv, hd=128, cls=0: args.splits
    g = torch.Generator().manual_seed(1)
    room = N + args.steps + 16
    eng = Engine(model, model.new_cache(max_tokens=B * (room + ops.PAGE), max_seq_len=room), use_graphs=True)
    with torch.inference_mode():
        slots = [eng.alloc_slot() for _ in range(B)]
        for s in slots:                                   # one prompt per step keeps the prefill's activations small
            eng.step([SequenceInput(s, torch.randint(0, cfg["vocab_size"], (N,), generator=g).tolist(), [])])
        tok = [1] * B
        for _ in range(6):
            eng.decode_step(slots, tok)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            eng.decode_step(slots, tok)
        b.record()
        torch.cuda.synchronize()
    eng.check_device_errors()
    us = a.elapsed_time(b) / args.steps * 1e3
    pieces = args.splits or rule(B, cfg["num_key_value_heads"], cfg["hidden_size"] // cfg["num_attention_heads"], context_class(N + 6))
    print(json.dumps({"kernel": "decode_step", "shape": args.shape, "layers": L, "batch": B, "context": N, "pieces": pieces,
                      "us_per_step": round(us, 1), "us_per_layer": round(us / L, 1)}))
    return 0


def _prefill_step(args) -> int:
    import bench
    import kuiperllama_b200 as kl
    from kuiperllama_b200.config import config_from_dict
    from kuiperllama_b200.engine import Engine, SequenceInput
    base = {"8b": bench.LLAMA31_8B, "7b": bench.LLAMA2_7B, "1b": bench.LLAMA32_1B, "70b": bench.LLAMA3_70B}[args.shape]
    T, L = args.tokens, args.layers
    cfg = dict(base, num_hidden_layers=L, max_position_embeddings=max(base["max_position_embeddings"], T))
    model = kl.random_model(config_from_dict(cfg), seed=0)
    eng = Engine(model, model.new_cache(max_tokens=T + ops.PAGE, max_seq_len=T), use_graphs=False)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg["vocab_size"], (T,), generator=g).tolist()
    times = []
    with torch.inference_mode():
        for _ in range(3 + args.repeats):
            slot = eng.alloc_slot()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            eng.step([SequenceInput(slot, prompt, [T - 1])])
            b.record()
            torch.cuda.synchronize()
            eng.free_slot(slot)
            times.append(a.elapsed_time(b))
    eng.check_device_errors()
    times = sorted(times[3:])
    ms = times[len(times) // 2]
    print(json.dumps({"kernel": "prefill_step", "shape": args.shape, "layers": L, "tokens": T, "ms": round(ms, 3),
                      "us_per_layer": round(ms * 1e3 / L, 1)}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="microbench")
    ap.add_argument("kernel", choices=["gemm_skinny", "gemm_tcgen05", "attention_prefill", "attention_decode", "decode_step",
                                           "prefill_step"])
    ap.add_argument("--shape", default="8b", choices=["8b", "7b", "1b", "70b"], help="decode_step: which of bench.py's shapes")
    ap.add_argument("--layers", type=int, default=4, help="decode_step: layers of the model")
    ap.add_argument("--steps", type=int, default=150, help="decode_step: timed steps")
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--splits", type=int, default=None)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=640)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--repeats", type=int, default=20)
    ap.add_argument("--simt", action="store_true", help="attention_decode: the split-KV SIMT kernel instead of the tensor-core one")
    ap.add_argument("--mma", action="store_true", help="attention_prefill: the mma.sync kernel instead of the tcgen05 one")
    ap.add_argument("--fused", action="store_true", help="attention_decode: the form of a decode step (sums six pieces of "
                    "the q/k/v product, rotates, writes the token into the cache, attends, merges the splits)")
    args = ap.parse_args(argv)
    torch.manual_seed(0)
    out = {"kernel": args.kernel}
    if args.kernel == "decode_step":
        return _decode_step(args)
    if args.kernel == "prefill_step":
        return _prefill_step(args)
    if args.kernel in ("gemm_skinny", "gemm_tcgen05"):
        a = torch.randn(args.m, args.k, device=DEV).bfloat16()
        w = torch.randn(args.n, args.k, device=DEV).bfloat16()
        c = torch.empty(args.m, args.n // 2 if args.swiglu else args.n, device=DEV, dtype=torch.bfloat16)
        if args.kernel == "gemm_skinny":
            fn = lambda: ops.gemm_skinny(a, w, c, args.splits, swiglu=args.swiglu)
        else:
            fn = lambda: ops.gemm_tcgen05(a, w, c, swiglu=args.swiglu)
        t = _time(fn, args.repeats)
        flops = 2.0 * args.m * args.n * args.k
        byts = 2.0 * (args.n * args.k + args.m * args.k + c.numel())
        out.update(m=args.m, n=args.n, k=args.k, swiglu=args.swiglu, us=round(t * 1e6, 2), tflops=round(flops / t / 1e12, 1),
                   gbs=round(byts / t / 1e9, 1))
    else:
        H, KV, hd = args.heads, args.kv_heads, args.head_dim
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        scale = 1.0 / math.sqrt(hd)
        if args.kernel == "attention_prefill":
            T = args.tokens
            table, k, v = _paged(1, T, KV, hd)
            q = torch.randn(T, (H + 2 * KV) * hd, device=DEV).bfloat16()
            o = torch.empty(T, H * hd, device=DEV, dtype=torch.bfloat16)
            cu, sl, st, nw = i32([0, T]), i32([0]), i32([0]), i32([T])
            if args.mma or hd not in (64, 128):
                fn = lambda: ops.attention_mma(q, q.shape[1], o, k, v, table, cu, sl, st, nw, 1, T, T, H, KV, hd, scale, 0, 1, False)
            else:
                fn = lambda: ops.attention_tcgen05(q, q.shape[1], o, k, v, table, cu, sl, st, nw, 1, T, T, H, KV, hd, scale)
            t = _time(fn, args.repeats)
            flops = 4.0 * H * hd * T * (T + 1) / 2
            out.update(tokens=T, heads=H, kv_heads=KV, head_dim=hd, us=round(t * 1e6, 2), tflops=round(flops / t / 1e12, 1))
        else:
            B, N = args.batch, args.context
            table, k, v = _paged(B, N, KV, hd)
            q = torch.randn(B, (H + 2 * KV) * hd, device=DEV).bfloat16()
            o = torch.empty(B, H * hd, device=DEV, dtype=torch.bfloat16)
            pos, slots = i32([N - 1] * B), i32(list(range(B)))
            cu, st, nw = i32(list(range(B + 1))), i32([N - 1] * B), i32([1] * B)
            splits = args.splits or ops.decode_attention_splits(B, KV, hd)
            if args.fused:
                from types import SimpleNamespace
                step = SimpleNamespace(n_seqs=B, n_tokens=B, is_decode=True, cu_tokens=cu, seq_slots=slots, seq_starts=st, seq_new=nw)
                pieces = torch.randn(6, B, (H + 2 * KV) * hd, device=DEV)
                inv_freq = (500000.0 ** (-torch.arange(0, hd, 2, dtype=torch.float64) / hd)).float().to(DEV)
                splits = args.splits
                fn = lambda: ops.attention_decode_fused(pieces, inv_freq, o, k, v, table, step, H, KV, hd, scale, 0, args.splits)
            elif args.simt:
                fn = lambda: ops.attention_decode(q, q.shape[1], o, k, v, table, pos, slots, B, H, KV, hd, scale, 0, args.splits)
            else:
                fn = lambda: ops.attention_mma(q, q.shape[1], o, k, v, table, cu, slots, st, nw, B, 1, B, H, KV, hd, scale, 0, splits, True)
            t = _time(fn, args.repeats)
            byts = 2.0 * 2 * B * N * KV * hd
            out.update(batch=B, context=N, heads=H, kv_heads=KV, head_dim=hd, splits=splits, us=round(t * 1e6, 2),
                       gbs=round(byts / t / 1e9, 1))
    ops.check_status(DEV)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
