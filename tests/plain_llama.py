"""Plain, slow Llama 2/3 decoder on the CPU in float32: the oracle of the test-suite.

Whole sequences, no cache, one function for each part.  It shares no code with the
package under test: it reads ``config.json`` as a plain dict and the weights as a
plain ``{name: tensor}`` dict.  Every function cites the place in
ExiledOfCode/KuiperLLama whose arithmetic it restates (paths are relative to that
project's root).  ``tests/golden/make_golden.py`` compares this file once with
KuiperLLama's own ``tools/model.py`` on a tiny random model.

The Llama-3 frequency scaling rule has no counterpart in KuiperLLama (its Llama-3
build uses the unscaled theta, kuiper/source/op/kernels/cuda/rope_kernel.cu:38-49);
``rope_inverse_frequencies`` restates the published definition of
``rope_type: "llama3"`` from the keys of config.json alone.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


# ----------------------------------------------------------------------------- config

def read_config(folder: str) -> dict:
    """config.json as a dict with the defaults KuiperLLama's exporter assumes
    (tools/export_llama3.py:547-554: n_kv_heads defaults to n_heads; head size is
    dim / n_heads, kuiper/source/model/model.cpp:123)."""
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    if c.get("head_dim") is None:
        c["head_dim"] = c["hidden_size"] // c["num_attention_heads"]
    c.setdefault("rms_norm_eps", 1e-5)
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("rope_scaling", None)
    c.setdefault("tie_word_embeddings", False)
    return c


def read_weights(folder: str) -> Dict[str, torch.Tensor]:
    """All tensors of model.safetensors as float32 (through the safetensors package,
    so the package's own reader and writer are checked against an independent one)."""
    from safetensors.torch import load_file

    return {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


# ----------------------------------------------------------------------------- parts

def embedding(table: torch.Tensor, token_ids: Sequence[int]) -> torch.Tensor:
    """x_t = E[tok_t, :], no scaling (kuiper/source/op/kernels/cuda/emb_kernel.cu:15-20)."""
    return table[torch.as_tensor(list(token_ids), dtype=torch.long)].clone()


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """out = w * x * rsqrt(mean(x^2) + eps); eps inside the root, weight after
    (kuiper/source/op/kernels/cpu/rmsnorm_kernel.cpp:27-32, tools/model.py:33-38)."""
    mean_sq = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return weight * (x * torch.rsqrt(mean_sq + eps))


def rope_inverse_frequencies(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """freq_j = theta^(-2j/head_dim), j in [0, head_dim/2)
    (kuiper/source/op/kernels/cpu/rope_kernel.cpp:6-8, tools/model.py:42), computed in
    float64 and rounded once to float32.  With rope_type "llama3": wavelengths shorter
    than original/high_freq_factor keep their frequency, those longer than
    original/low_freq_factor are divided by factor, those between are interpolated."""
    j = torch.arange(0, head_dim, 2, dtype=torch.float64)
    freq = 1.0 / (float(theta) ** (j / head_dim))
    if scaling is not None:
        kind = scaling.get("rope_type", scaling.get("type"))
        assert kind == "llama3", kind
        factor = float(scaling["factor"])
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        orig = float(scaling["original_max_position_embeddings"])
        out = []
        for f in freq.tolist():
            wavelen = 2.0 * math.pi / f
            if wavelen < orig / high:
                out.append(f)
            elif wavelen > orig / low:
                out.append(f / factor)
            else:
                s = (orig / wavelen - low) / (high - low)
                out.append((1.0 - s) * f / factor + s * f)
        freq = torch.tensor(out, dtype=torch.float64)
    return freq.float()


def rope_rotate(v: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """v: [T, heads, head_dim].  Half-split pairs (j, j + head_dim/2):
    v[j] <- a cos - b sin, v[j+hd/2] <- a sin + b cos with angle = float(pos) * freq_j
    (kuiper/source/op/kernels/cpu/rope_kernel.cpp:25-41, Llama-3 build, which works on
    HF-layout weights without permuting them, tools/export_llama3.py:578-579)."""
    half = v.shape[-1] // 2
    angle = positions.float()[:, None] * inv_freq[None, :]          # [T, half], float32
    cos = torch.cos(angle)[:, None, :]
    sin = torch.sin(angle)[:, None, :]
    a, b = v[..., :half], v[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


def attention_scores_softmax_values(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """q: [T, H, hd], k/v: [T, KV, hd] of one whole sequence starting at position 0.
    Head h reads kv head h // (H / KV); s_t = (q . k_t) / sqrt(hd) for t <= pos; softmax
    with the maximum subtracted; o = sum_t p_t v_t
    (kuiper/source/op/kernels/cuda/mha_kernel.cu:61,74-106; cpu/mha_kernel.cpp:11,28-59)."""
    T, H, hd = q.shape
    KV = k.shape[1]
    group = H // KV
    scale = 1.0 / math.sqrt(float(hd))
    out = torch.empty_like(q)
    for h in range(H):
        g = h // group
        for pos in range(T):
            s = (k[: pos + 1, g, :] @ q[pos, h, :]) * scale
            e = torch.exp(s - s.max())
            p = e / e.sum()
            out[pos, h, :] = p @ v[: pos + 1, g, :]
    return out


def attention_mixer(n: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, c: dict,
                    inv_freq: torch.Tensor) -> torch.Tensor:
    """q, k, v projections without bias, rope on q and k (not v), attention, output
    projection (kuiper/source/model/llama3.cpp:610-639, 651-675)."""
    T = n.shape[0]
    H, KV, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    q = (n @ w[prefix + "self_attn.q_proj.weight"].T).view(T, H, hd)
    k = (n @ w[prefix + "self_attn.k_proj.weight"].T).view(T, KV, hd)
    v = (n @ w[prefix + "self_attn.v_proj.weight"].T).view(T, KV, hd)
    positions = torch.arange(T)
    q = rope_rotate(q, positions, inv_freq)
    k = rope_rotate(k, positions, inv_freq)
    o = attention_scores_softmax_values(q, k, v).reshape(T, H * hd)
    return o @ w[prefix + "self_attn.o_proj.weight"].T


def swiglu_feed_forward(n: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """f = W2 (silu(W1 n) * W3 n), silu(g) = g / (1 + exp(-g)); gate=W1, up=W3, down=W2
    (kuiper/source/model/llama3.cpp:692-718, kuiper/source/op/kernels/cpu/swiglu_kernel.cpp:21-22,
    tools/export_llama3.py:583-585)."""
    g = n @ w[prefix + "mlp.gate_proj.weight"].T
    u = n @ w[prefix + "mlp.up_proj.weight"].T
    m = g * (1.0 / (1.0 + torch.exp(-g))) * u
    return m @ w[prefix + "mlp.down_proj.weight"].T


def decoder_block(x: torch.Tensor, w: Dict[str, torch.Tensor], layer: int, c: dict,
                  inv_freq: torch.Tensor) -> torch.Tensor:
    """x += Attn(norm1(x)); x += FFN(norm2(x)) (kuiper/source/model/llama3.cpp:155-164,
    tools/model.py:200-203)."""
    p = f"model.layers.{layer}."
    eps = c["rms_norm_eps"]
    x = x + attention_mixer(rmsnorm(x, w[p + "input_layernorm.weight"], eps), w, p, c, inv_freq)
    x = x + swiglu_feed_forward(rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps), w, p)
    return x


def output_logits(x: torch.Tensor, w: Dict[str, torch.Tensor], c: dict) -> torch.Tensor:
    """Final RMSNorm, then the classifier; tied embeddings reuse the embedding table
    (kuiper/source/model/llama3.cpp:721-730, 369-378)."""
    x = rmsnorm(x, w["model.norm.weight"], c["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if c["tie_word_embeddings"] else w["lm_head.weight"]
    return x @ head.T


def forward_logits(w: Dict[str, torch.Tensor], c: dict, token_ids: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] at every position of one whole sequence."""
    inv_freq = rope_inverse_frequencies(c["head_dim"], c["rope_theta"], c["rope_scaling"])
    x = embedding(w["model.embed_tokens.weight"], token_ids)
    for layer in range(c["num_hidden_layers"]):
        x = decoder_block(x, w, layer, c, inv_freq)
    return output_logits(x, w, c)


# ----------------------------------------------------------------------------- sampling and generation

def argmax_token(logits: torch.Tensor) -> int:
    """Index of the largest logit, the lowest index among equals
    (kuiper/source/sampler/argmax_sampler.cpp:5-13, argmax_kernel.cu:13-18)."""
    best, best_i = -math.inf, 0
    for i, value in enumerate(logits.tolist()):
        if value > best:
            best, best_i = value, i
    return best_i


def uniform_from_counter(seed: int, request: int, step: int) -> float:
    """The draw in [0, 1) that the package's temperature sampler documents for
    (seed, request index, decode step): a 64-bit mix of the three, top 24 bits."""
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + request * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB
         + 0x2545F4914F6CDD1D) & mask
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & mask
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & mask
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


def temperature_probabilities(logits: torch.Tensor, temperature: float,
                              top_k: Optional[int] = None) -> torch.Tensor:
    """softmax(logits / T) after an optional top-k cut that keeps every logit not below
    the k-th largest (tools/model.py:331-338), in float64."""
    z = logits.double() / temperature
    if top_k is not None:
        kth = torch.topk(z, min(top_k, z.numel())).values[-1]
        z = torch.where(z < kth, torch.full_like(z, -math.inf), z)
    e = torch.exp(z - z.max())
    return e / e.sum()


def inverse_cdf_pick(probs: torch.Tensor, u: float) -> int:
    """First index whose cumulative probability exceeds u."""
    c = torch.cumsum(probs, dim=0)
    idx = int(torch.searchsorted(c, torch.tensor([u * float(c[-1])], dtype=c.dtype), right=True))
    return min(idx, probs.numel() - 1)


def greedy_generate(w: Dict[str, torch.Tensor], c: dict, prompt: Sequence[int], max_new_tokens: int,
                    stop_ids: Sequence[int] = ()) -> List[int]:
    """Feed the whole sequence again for every new token; the stop token ends the
    sequence and is not emitted (demo/main.cpp:30-32 tests it before it is appended)."""
    tokens = list(prompt)
    new: List[int] = []
    for _ in range(max_new_tokens):
        nxt = argmax_token(forward_logits(w, c, tokens)[-1])
        if nxt in stop_ids:
            break
        tokens.append(nxt)
        new.append(nxt)
    return new
