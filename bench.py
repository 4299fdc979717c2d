#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama-3.1-8B-shaped model with random weights on one
B200, and the two other workloads of the same family (Llama-2-7B shape with ragged prompts,
Llama-3.2-1B shape with temperature sampling).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--impl reference] [--no-points]

A "step" is one decode step of a batch (default 8 sequences that each hold a 512-token
prompt, context limit 4096).  One JSON line is printed:

* ``value``     decoded tokens a second over K device-timed steps (CUDA events); a step's token
                ids stay on the device for the next step and are read on the host one step later;
* ``e2e``       the same through the Python entry point ``Inference.generate`` with host
                token lists in and out (every step copies its token ids to the device from
                pinned memory and reads the sampled ids back);
* ``prefill``   one 2,048-token prompt in one step: tokens a second, and the step's flops over
                its time over the bf16 peak;
* ``roofline``  for the decode step: the bytes it has to read (every weight once, and the
                keys and values of the live sequences) over its time, against the HBM peak;
* ``points``    decode tokens a second at batch 1, 64 and 128 with their roofline fractions, the
                headline's batch again after 40 warm-up steps (``decode_b8_settled``: the SM clock
                needs some 14 steps to recover from the prefill's time under the power cap), and the
                rates of the two other workloads; ``workloads`` has their sizes, bytes and flops,
                and their decode rates with CUDA graphs on and off;
* ``checks``    what was verified beside the clock: after every timed region the device's report
                words were read (a kernel that gave up a bounded wait would otherwise make the
                run *faster*), the last logits were finite, and a decode step replayed from its
                CUDA graph gave the same logits as the same step launched kernel by kernel.  A
                failed check ends the run with an error instead of a number.

Peaks come from MEASURED_PEAKS.json beside this file when the driver wrote it, else from the
fallback figures of this pool (6.65 TB/s, 1.59 PFLOP/s).  Each decode step streams gigabytes of
weights, far more than the 126 MB L2, so no extra flush runs between timed steps.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

_LLAMA3_ROPE = {"rope_type": "llama3", "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}
# The layer sizes of the three workloads: Llama-3.1-8B, Llama-2-7B and Llama-3.2-1B.
LLAMA31_8B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "intermediate_size": 14336,
    "num_hidden_layers": 32, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "vocab_size": 128256, "max_position_embeddings": 4096, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": dict(_LLAMA3_ROPE, factor=8.0), "tie_word_embeddings": False, "hidden_act": "silu",
}
LLAMA2_7B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "intermediate_size": 11008,
    "num_hidden_layers": 32, "num_attention_heads": 32, "num_key_value_heads": 32, "head_dim": 128,
    "vocab_size": 32000, "max_position_embeddings": 4096, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "rope_scaling": None, "tie_word_embeddings": False, "hidden_act": "silu",
}
LLAMA32_1B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 2048, "intermediate_size": 8192,
    "num_hidden_layers": 16, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "vocab_size": 128256, "max_position_embeddings": 4096, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": dict(_LLAMA3_ROPE, factor=32.0), "tie_word_embeddings": True, "hidden_act": "silu",
}
# Not one of the bench's workloads: the largest Llama shape whose weights fit one B200 in bfloat16 (141 GB),
# for `microbench.py decode_step / prefill_step --shape 70b` on a few of its layers.
LLAMA3_70B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 8192, "intermediate_size": 28672,
    "num_hidden_layers": 80, "num_attention_heads": 64, "num_key_value_heads": 8, "head_dim": 128,
    "vocab_size": 128256, "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": dict(_LLAMA3_ROPE, factor=8.0), "tie_word_embeddings": False, "hidden_act": "silu",
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
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,utilization.gpu")

    def __init__(self):
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
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
        mhz, busy_mhz, mx, reasons = [], [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 7:
                continue
            try:
                mhz.append(int(parts[0]))
                mx = int(parts[1])
                if int(parts[6]) >= 50:
                    busy_mhz.append(int(parts[0]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        under_load = sorted(busy_mhz or mhz)
        return {"sm_mhz": under_load[len(under_load) // 2] if under_load else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(mhz), "samples_under_load": len(busy_mhz)}


# ---------------------------------------------------------------------------------------------- bytes and flops

def layer_params(cfg):
    d, i = cfg["hidden_size"], cfg["intermediate_size"]
    h, kv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    return h * hd * d + 2 * kv * hd * d + d * h * hd + 3 * d * i


def decode_bytes(cfg, n_layers, total_context, dtype_bytes=2):
    """Bytes one decode step must read: every weight it uses once (the embedding table is only
    gathered from; the classifier, which a tied model shares with it, is read whole) and the keys
    and values of the live sequences (``total_context`` tokens over all of them)."""
    d, v = cfg["hidden_size"], cfg["vocab_size"]
    kv, hd = cfg["num_key_value_heads"], cfg["head_dim"]
    weights = n_layers * (layer_params(cfg) * dtype_bytes + 2 * d * 4) + v * d * dtype_bytes + d * 4
    cache = total_context * n_layers * 2 * kv * hd * dtype_bytes
    return weights + cache, weights, cache


def prefill_flops(cfg, n_layers, lengths):
    """Flops of one step that brings whole prompts of the given lengths and asks for the logits at
    each prompt's last token: products, causal attention (QK^T and PV over t (t + 1) / 2 pairs) and
    one classifier row per prompt."""
    d, v = cfg["hidden_size"], cfg["vocab_size"]
    h, hd = cfg["num_attention_heads"], cfg["head_dim"]
    tokens = sum(lengths)
    linear = 2 * tokens * layer_params(cfg)
    attention = sum(4 * h * hd * t * (t + 1) // 2 for t in lengths)
    return n_layers * (linear + attention) + len(lengths) * 2 * v * d


# ---------------------------------------------------------------------------------------------- checks

class BenchCheckError(RuntimeError):
    pass


def check_after(infer, logits, what, checks):
    """After a timed region: the device's report words (raises if a kernel gave up a wait or met a
    bad token id) and the last logits."""
    import torch
    infer.engine.check_device_errors()
    if logits is not None and not bool(torch.isfinite(logits).all()):
        raise BenchCheckError(f"{what}: the logits are not finite")
    checks["device_words_read"] = checks.get("device_words_read", 0) + 1
    checks["logits_finite"] = True


def verify_graph_replay(eng, slots, tokens):
    """One decode step twice from the same state: launched kernel by kernel (the first step of a
    batch size, which also captures the graph), then replayed from the graph after the lengths
    were set back.  Both write the same keys and values to the same places.  Returns the largest
    difference between the two steps' logits (0 expected: the same kernels on the same data)."""
    import torch
    n = len(slots)
    assert n not in eng.graph_sizes(), "the graph of this batch size exists already"
    before = [eng.cache.lengths[s] for s in slots]
    eager = eng.decode_step(slots, tokens).clone()
    assert n in eng.graph_sizes()
    for s, b in zip(slots, before):
        eng.cache.lengths[s] = b
    replayed = eng.decode_step(slots, tokens)
    if not torch.equal(eager.argmax(dim=1), replayed.argmax(dim=1)):
        raise BenchCheckError(f"batch {n}: the step replayed from its CUDA graph chose other tokens than the same step without a graph")
    return float((eager - replayed).abs().max())


# ---------------------------------------------------------------------------------------------- timed regions

def time_decode(infer, batch, steps, warmup, seed, checks):
    """K device-timed decode steps of ``batch`` sequences after 512-token prompts.  Returns
    (seconds, mean context over the timed steps, kernel launches in the timed region)."""
    import torch
    from kuiperllama_b200.csrc import ops
    from kuiperllama_b200.engine import SequenceInput
    from kuiperllama_b200.engine.generate import _Tokens
    from kuiperllama_b200.sampling import Sampler, SamplingParams
    eng = infer.engine
    g = torch.Generator().manual_seed(seed)
    vocab = infer.model.spec.vocab_size
    prompts = torch.randint(0, vocab, (batch, PROMPT_LEN), generator=g).tolist()
    sampler = Sampler(SamplingParams())
    empty = torch.empty(0, dtype=torch.int32, device=eng.device)
    last = {}

    def one_step(prev):
        """Start the step that follows `prev` from its tokens on the device, then read `prev`'s
        tokens on the host: the way the generation loop runs (one step ahead of the host)."""
        last["logits"] = eng.decode_step(slots, prev.device_tokens)
        nxt = _Tokens(sampler.sample(last["logits"], empty, empty))
        prev.read()
        return nxt

    with torch.inference_mode():
        slots = [eng.alloc_slot() for _ in range(batch)]
        logits = eng.step([SequenceInput(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        tokens = _Tokens(sampler.sample(logits, empty, empty))
        if eng.use_graphs and batch not in eng.graph_sizes():
            diff = verify_graph_replay(eng, slots, tokens.read())
            checks[f"graph_replay_b{batch}_max_logit_diff"] = diff
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
        check_after(infer, last.get("logits"), f"decode at batch {batch}", checks)
        for s in slots:
            eng.free_slot(s)
    return seconds, mean_ctx, launches


def time_prefill(infer, warmup, repeats, seed, checks):
    import torch
    from kuiperllama_b200.engine import SequenceInput
    eng = infer.engine
    g = torch.Generator().manual_seed(seed)
    prompt = torch.randint(0, infer.model.spec.vocab_size, (PREFILL_LEN,), generator=g).tolist()
    times = []
    logits = None
    with torch.inference_mode():
        for it in range(warmup + repeats):
            slot = eng.alloc_slot()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            logits = eng.step([SequenceInput(slot, prompt, [PREFILL_LEN - 1])])
            b.record()
            torch.cuda.synchronize()
            if it >= warmup:
                times.append(a.elapsed_time(b) / 1e3)
            eng.free_slot(slot)
        check_after(infer, logits, "prefill", checks)
    times.sort()
    return times[len(times) // 2]


def time_e2e(infer, batch, steps, seed):
    """Through the public entry point: host token lists in, host token lists out."""
    import torch
    g = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, infer.model.spec.vocab_size, (batch, PROMPT_LEN), generator=g).tolist()
    infer.generate(prompts, max_new_tokens=4, stop_ids=[])                 # warm-up
    torch.cuda.synchronize()
    out = infer.generate(prompts, max_new_tokens=steps + 1, stop_ids=[])   # reads the device's report words itself
    torch.cuda.synchronize()
    st = infer.last_stats
    assert all(len(o) == steps + 1 for o in out)
    return st.decode_tokens / st.decode_seconds, st


def run_workload(kl, cfg, name, n_seqs, lo, hi, new_tokens, temperature, pk, seed):
    """One of the ragged workloads through ``Inference.generate``: ``n_seqs`` prompts with lengths
    uniform in [lo, hi], then ``new_tokens - 1`` decode steps; with CUDA graphs and without."""
    import torch
    from kuiperllama_b200.config import config_from_dict
    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(lo, hi + 1, (n_seqs,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]
    held = sum((n + new_tokens + 63) // 64 * 64 for n in lengths)
    model = kl.random_model(config_from_dict(cfg), seed=0, dtype="bfloat16", device="cuda:0")
    layers = cfg["num_hidden_layers"]
    out = {"sequences": n_seqs, "prompt_tokens": sum(lengths), "prompt_len_min": min(lengths), "prompt_len_max": max(lengths),
           "decode_steps": new_tokens - 1, "temperature": temperature}
    for graphs in (True, False):
        infer = kl.Inference(model, max_tokens=held, max_batch=n_seqs, max_seq_len=hi + new_tokens, use_graphs=graphs)
        # warm-up: the whole run once, so that the decode step is captured for every class of context lengths it passes through
        infer.generate(prompts, max_new_tokens=new_tokens, temperature=temperature, seed=1, stop_ids=[])
        torch.cuda.synchronize()
        res = infer.generate(prompts, max_new_tokens=new_tokens, temperature=temperature, seed=1, stop_ids=[])
        torch.cuda.synchronize()
        assert all(len(r) == new_tokens for r in res)
        st = infer.last_stats
        decode_rate = st.decode_tokens / st.decode_seconds
        if graphs:
            steps = st.decode_steps
            mean_total_ctx = sum(lengths) + n_seqs * (new_tokens + 1) / 2.0
            byts, wb, cb = decode_bytes(cfg, layers, mean_total_ctx)
            sec_per_step = st.decode_seconds / steps
            flops = prefill_flops(cfg, layers, lengths)
            out.update({
                "prefill_tokens_per_s": round(st.prefill_tokens / st.prefill_seconds, 1),
                "prefill_ms": round(st.prefill_seconds * 1e3, 2), "prefill_tflop": round(flops / 1e12, 2),
                "prefill_frac": round(flops / st.prefill_seconds / (pk["bf16_tflops"] * 1e12), 4),
                "decode_tokens_per_s": round(decode_rate, 1), "decode_ms_per_step": round(sec_per_step * 1e3, 4),
                "decode_gb_per_step": round(byts / 1e9, 3), "decode_weight_gb": round(wb / 1e9, 3), "decode_cache_gb": round(cb / 1e9, 3),
                "decode_frac": round(byts / sec_per_step / 1e9 / pk["hbm_gbs"], 4)})
        else:
            out["decode_tokens_per_s_without_graphs"] = round(decode_rate, 1)
        del infer
    del model
    torch.cuda.empty_cache()
    return out


def reference_arm(args):
    """ExiledOfCode/KuiperLLama is a CMake C++ project without a Python package definition, and
    its build fetches glog, armadillo, sentencepiece and gtest over the network; it cannot be
    installed offline: `pip install --no-index` answers that the directory has neither
    setup.py nor pyproject.toml.  Even built, its stock path is float32 only, one sequence, and
    feeds the prompt token by token (demo/main.cpp:18-41, kuiper/include/base/base.h:42-47), so it
    could not run this metric's configuration (bfloat16, batches, whole prompts in one step)."""
    print(json.dumps({"impl": "reference", "unavailable":
                      "KuiperLLama has no setup.py/pyproject.toml (pip install fails) and its CMake build needs glog, "
                      "armadillo, sentencepiece and gtest fetched from the network; its engine is float32-only, batch 1 and "
                      "feeds prompts token by token, so no same-configuration ratio could exist"}))
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
    ap.add_argument("--no-points", action="store_true",
                    help="only the headline: skip the prefill, the batch 1, 64 and 128 points and the two other workloads")
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
    checks = {}
    max_batch = max(args.batch, 1 if args.no_points else 128)
    model = kl.random_model(config_from_dict(cfg), seed=0, dtype=args.dtype, device="cuda:0")
    infer = kl.Inference(model, max_tokens=max_batch * CONTEXT, max_batch=max_batch, max_seq_len=CONTEXT)
    esize = 2 if args.dtype == "bfloat16" else 4

    clocks = ClockSampler()
    clocks.start()
    seconds, mean_ctx, launches = time_decode(infer, args.batch, args.steps, args.warmup, seed=1, checks=checks)
    ms_per_step = seconds / args.steps * 1e3
    value = args.batch * args.steps / seconds
    total_bytes, weight_bytes, cache_bytes = decode_bytes(cfg, args.layers, args.batch * mean_ctx, esize)
    achieved = total_bytes / (seconds / args.steps) / 1e9

    e2e_value, st = time_e2e(infer, args.batch, args.steps, seed=1)
    checks["device_words_read"] += 2                                               # generate() reads them before it returns
    h2d = (3 * args.batch + 3 * args.batch + args.batch + 1 + args.batch) * 4      # the step's packed integer inputs
    d2h = args.batch * 4                                                          # the sampled token ids

    line = {
        "metric": "decode tok/s, Llama-3.1-8B shape bf16, batch 8 (also batch 1/64/128 and prefill tok/s at 2048 tokens)",
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
        "e2e": {"value": round(e2e_value, 2), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "weight_gb": round(weight_bytes / 1e9, 3),
                     "cache_gb": round(cache_bytes / 1e9, 3)},
        "impl": "ours",
    }
    if not args.no_points:
        t = time_prefill(infer, warmup=3, repeats=5, seed=2, checks=checks)
        flops = prefill_flops(cfg, args.layers, [PREFILL_LEN])
        line["prefill"] = {"value": round(PREFILL_LEN / t, 1), "tokens": PREFILL_LEN, "ms": round(t * 1e3, 3),
                           "frac": round(flops / t / (pk["bf16_tflops"] * 1e12), 4),
                           "frac_of_sustained": round(flops / t / (pk["bf16_tflops_sustained"] * 1e12), 4),
                           "tflop": round(flops / 1e12, 3)}
        points = {}
        # The headline's batch again with 40 warm-up steps: for the 14 steps after a 4,096-token prefill the SM
        # clock is still 1.4 GHz under the power cap's after-effect (then 1.85 GHz), and a decode step follows it.
        k = max(16, args.steps // 2)
        s, ctx, _ = time_decode(infer, args.batch, k, 40, seed=2, checks=checks)
        byts, _, _ = decode_bytes(cfg, args.layers, args.batch * ctx, esize)
        points[f"decode_b{args.batch}_settled"] = round(args.batch * k / s, 2)
        points[f"decode_b{args.batch}_settled_frac"] = round(byts / (s / k) / 1e9 / pk["hbm_gbs"], 4)
        for b in (1, 64, 128):        # 128 sequences: beyond the 64-token tiles of the decode products
            k = max(16, args.steps // 2)
            s, ctx, _ = time_decode(infer, b, k, max(args.warmup, 40), seed=3 + b, checks=checks)     # settled, as above
            byts, _, _ = decode_bytes(cfg, args.layers, b * ctx, esize)
            points[f"decode_b{b}"] = round(b * k / s, 2)
            points[f"decode_b{b}_frac"] = round(byts / (s / k) / 1e9 / pk["hbm_gbs"], 4)
        del infer, model
        torch.cuda.empty_cache()
        workloads = {}
        if args.dtype == "bfloat16" and args.layers == 32:
            workloads["llama2_7b_ragged"] = run_workload(kl, LLAMA2_7B, "llama2_7b", 16, 16, 1024, 129, 0.0, pk, seed=7)
            workloads["llama32_1b_sampled"] = run_workload(kl, LLAMA32_1B, "llama32_1b", 64, 1, 2048, 257, 1.0, pk, seed=8)
            checks["device_words_read"] += 8
            for name, w in workloads.items():
                points[f"{name}_prefill"] = w["prefill_tokens_per_s"]
                points[f"{name}_decode"] = w["decode_tokens_per_s"]
                points[f"{name}_decode_frac"] = w["decode_frac"]
            line["workloads"] = workloads
        line["points"] = points
    line["clocks"] = clocks.stop()
    line["checks"] = checks
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
