#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama-3.1-8B-shaped model with random weights on one
B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--impl reference]

A "step" is one decode step of a batch (default 8 sequences that each hold a 512-token
prompt, context limit 4096).  One JSON line is printed:

* ``value``     decoded tokens a second over K device-timed steps (CUDA events); a step's token
                ids stay on the device for the next step and are read on the host one step later;
* ``e2e``       the same through the Python entry point ``LlamaInfer.generate`` with host
                token lists in and out (every step copies its token ids to the device from
                pinned memory and reads the sampled ids back);
* ``prefill``   one 2,048-token prompt in one step: tokens a second, and the step's flops over
                its time over the bf16 peak;
* ``roofline``  for the decode step: the bytes it has to read (every weight once, and the
                keys and values of the live sequences) over its time, against the HBM peak;
* ``points``    decode tokens a second at batch 1 and 64.

Peaks come from MEASURED_PEAKS.json beside this file when the driver wrote it, else from the
fallback figures of this pool (6.65 TB/s, 1.59 PFLOP/s).  Each decode step streams 15 GB of
weights, far more than the 126 MB L2, so no extra flush runs between timed steps.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Llama-3.1-8B layer sizes (the third configuration of BASELINE.json)
LLAMA31_8B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "intermediate_size": 14336,
    "num_hidden_layers": 32, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "vocab_size": 128256, "max_position_embeddings": 4096, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False, "hidden_act": "silu",
}
PROMPT_LEN = 512
PREFILL_LEN = 2048
CONTEXT = 4096


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                    "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
        except (OSError, KeyError, ValueError):
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                mhz.append(int(parts[0]))
                mx = int(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def decode_bytes(cfg, n_layers, batch, mean_context, dtype_bytes=2):
    """Bytes one decode step must read: every weight it uses once (the embedding table is
    only gathered from; the classifier is read whole) and the live sequences' keys and values."""
    d, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    h, kv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (h * hd * d + 2 * kv * hd * d + d * h * hd + 3 * d * i) * dtype_bytes + 2 * d * 4
    weights = n_layers * per_layer + v * d * dtype_bytes + d * 4
    cache = batch * mean_context * n_layers * 2 * kv * hd * dtype_bytes
    return weights + cache, weights, cache


def prefill_flops(cfg, n_layers, tokens):
    d, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    h, kv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = 2 * tokens * (h * hd * d + 2 * kv * hd * d + d * h * hd + 3 * d * i)
    attention = 4 * h * hd * tokens * (tokens + 1) // 2        # causal: QK^T and PV over t(t+1)/2 pairs
    return n_layers * (linear + attention) + 2 * v * d          # the classifier on the last row only


def time_decode(infer, batch, steps, warmup, seed):
    """K device-timed decode steps of ``batch`` sequences after 512-token prompts.  Returns
    (seconds, mean context over the timed steps, kernel launches in the timed region)."""
    import torch
    from kuiperllama_b200.csrc import ops
    from kuiperllama_b200.engine import SequenceInput
    from kuiperllama_b200.sampling import Sampler, SamplingParams
    eng = infer.engine
    g = torch.Generator().manual_seed(seed)
    vocab = infer.model.spec.vocab_size
    prompts = torch.randint(0, vocab, (batch, PROMPT_LEN), generator=g).tolist()
    from kuiperllama_b200.engine.generate import _Tokens
    sampler = Sampler(SamplingParams())
    empty = torch.empty(0, dtype=torch.int32, device=eng.device)

    def one_step(prev):
        """Start the step that follows `prev` from its tokens on the device, then read `prev`'s
        tokens on the host: the way the generation loop runs (one step ahead of the host)."""
        nxt = _Tokens(sampler.sample(eng.decode_step(slots, prev.device_tokens), empty, empty))
        prev.read()
        return nxt

    with torch.inference_mode():
        slots = [eng.alloc_slot() for _ in range(batch)]
        logits = eng.step([SequenceInput(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        tokens = _Tokens(sampler.sample(logits, empty, empty))
        for _ in range(warmup):
            tokens = one_step(tokens)
        tokens.read()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = ops.launch_count
        ctx0 = eng.cache.lengths[slots[0]]
        start.record()
        for _ in range(steps):
            tokens = one_step(tokens)
        tokens.read()
        stop.record()
        torch.cuda.synchronize()
        seconds = start.elapsed_time(stop) / 1e3
        launches = ops.launch_count - launches0
        mean_ctx = ctx0 + (steps + 1) / 2.0
        for s in slots:
            eng.free_slot(s)
    return seconds, mean_ctx, launches


def time_prefill(infer, warmup, repeats, seed):
    import torch
    from kuiperllama_b200.engine import SequenceInput
    eng = infer.engine
    g = torch.Generator().manual_seed(seed)
    prompt = torch.randint(0, infer.model.spec.vocab_size, (PREFILL_LEN,), generator=g).tolist()
    times = []
    with torch.inference_mode():
        for it in range(warmup + repeats):
            slot = eng.alloc_slot()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            eng.step([SequenceInput(slot, prompt, [PREFILL_LEN - 1])])
            b.record()
            torch.cuda.synchronize()
            if it >= warmup:
                times.append(a.elapsed_time(b) / 1e3)
            eng.free_slot(slot)
    times.sort()
    return times[len(times) // 2]


def time_e2e(infer, batch, steps, seed):
    """Through the public entry point: host token lists in, host token lists out."""
    import torch
    g = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, infer.model.spec.vocab_size, (batch, PROMPT_LEN), generator=g).tolist()
    infer.generate(prompts, max_new_tokens=4, stop_ids=[])                 # warm-up
    torch.cuda.synchronize()
    out = infer.generate(prompts, max_new_tokens=steps + 1, stop_ids=[])
    torch.cuda.synchronize()
    st = infer.last_stats
    assert all(len(o) == steps + 1 for o in out)
    return st.decode_tokens / st.decode_seconds, st


def reference_arm(args):
    """ExiledOfCode/KuiperLLama is a CMake C++ project without a Python package definition, and
    its build fetches glog, armadillo, sentencepiece and gtest over the network; it cannot be
    installed offline: `pip install --no-index` answers that the directory has neither
    setup.py nor pyproject.toml."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "KuiperLLama has no setup.py/pyproject.toml (pip install fails) and its CMake build needs "
                      "glog, armadillo, sentencepiece and gtest fetched from the network"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=32, help="fewer layers than the configuration's 32 (both are reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points and the prefill")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library has no multi-GPU path (--gpus {args.gpus} refused)")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import kuiperllama_b200 as kl
    from kuiperllama_b200.config import config_from_dict

    cfg = dict(LLAMA31_8B, num_hidden_layers=args.layers)
    pk = peaks()
    max_batch = max(args.batch, 1 if args.no_points else 64)
    model = kl.random_model(config_from_dict(cfg), seed=0, dtype=args.dtype, device="cuda:0")
    infer = kl.LlamaInfer(model, max_tokens=max_batch * CONTEXT, max_batch=max_batch, max_seq_len=CONTEXT)
    esize = 2 if args.dtype == "bfloat16" else 4

    clocks = ClockSampler()
    clocks.start()
    seconds, mean_ctx, launches = time_decode(infer, args.batch, args.steps, args.warmup, seed=1)
    clock_record = clocks.stop()
    ms_per_step = seconds / args.steps * 1e3
    value = args.batch * args.steps / seconds
    total_bytes, weight_bytes, cache_bytes = decode_bytes(cfg, args.layers, args.batch, mean_ctx, esize)
    achieved = total_bytes / (seconds / args.steps) / 1e9

    e2e_value, st = time_e2e(infer, args.batch, args.steps, seed=1)
    h2d = (3 * args.batch + 3 * args.batch + args.batch + 1 + args.batch) * 4      # the step's packed integer inputs
    d2h = args.batch * 4                                                          # the sampled token ids

    line = {
        "metric": "decode tok/s, Llama-3.1-8B shape bf16, batch 8 (also batch 1/64 and prefill tok/s at 2048 tokens)",
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic: random weights N(0, 0.02), uniform random token ids",
        "config": {
            "model": "Llama-3.1-8B shape", "layers": args.layers, "layers_of_configuration": 32,
            "hidden_size": cfg["hidden_size"], "intermediate_size": cfg["intermediate_size"],
            "num_attention_heads": cfg["num_attention_heads"], "num_key_value_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "vocab_size": cfg["vocab_size"], "rope_theta": cfg["rope_theta"],
            "rope_scaling": "llama3 factor 8 low 1 high 4 original 8192", "rms_norm_eps": cfg["rms_norm_eps"],
            "global_batch": args.batch, "prompt_len": PROMPT_LEN, "seq_len": CONTEXT, "prefill_len": PREFILL_LEN,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (15 GB of weights per step), no flush",
            "peaks": pk["source"],
        },
        "clocks": clock_record,
        "e2e": {"value": round(e2e_value, 2), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "weight_gb": round(weight_bytes / 1e9, 3),
                     "cache_gb": round(cache_bytes / 1e9, 3)},
        "impl": "ours",
    }
    if not args.no_points:
        t = time_prefill(infer, warmup=3, repeats=5, seed=2)
        flops = prefill_flops(cfg, args.layers, PREFILL_LEN)
        line["prefill"] = {"value": round(PREFILL_LEN / t, 1), "tokens": PREFILL_LEN, "ms": round(t * 1e3, 3),
                           "frac": round(flops / t / (pk["bf16_tflops"] * 1e12), 4),
                           "frac_of_sustained": round(flops / t / (pk["bf16_tflops_sustained"] * 1e12), 4),
                           "tflop": round(flops / 1e12, 3)}
        points = {}
        for b in (1, 64):
            s, _, _ = time_decode(infer, b, max(16, args.steps // 2), args.warmup, seed=3 + b)
            points[f"decode_b{b}"] = round(b * max(16, args.steps // 2) / s, 2)
        line["points"] = points
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
