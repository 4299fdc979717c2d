"""Each part of a layer alone against the plain implementation's function for it, and the
proof that parts are pluggable: a toy mixer with state of its own, a layer scheduled twice,
and an execution that reads another one's cache, all without a change to the package."""
from __future__ import annotations

import dataclasses
import math

import pytest
import torch

import plain_llama
from helpers import assert_close, config_dict, random_tokens, tolerance

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _runtime(dtype):
    from kuiperllama_b200.parts import Runtime
    return Runtime(device=DEV, dtype=DT[dtype])


def _dense(t):
    """A part may return float32 partial sums [S, n, hidden]; their sum is the result."""
    return t.sum(dim=0) if t.dim() == 3 else t


def _step_for(engine, slots_tokens):
    """A StepContext through the engine's own packing (slots_tokens: [(slot, n_tokens)])."""
    from kuiperllama_b200.engine import SequenceInput
    ctx, _, _ = engine._pack([SequenceInput(s, [0] * n, []) for s, n in slots_tokens], 0)
    return ctx


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    from kuiperllama_b200.config import PartSpec
    from kuiperllama_b200.parts import RMSNorm
    torch.manual_seed(0)
    w = (1 + 0.1 * torch.randn(200)).bfloat16()
    part = RMSNorm(PartSpec("rmsnorm", {"size": 200, "eps": 1e-4, "name": "n.weight"}), "L.", {"L.n.weight": w}, _runtime(dtype))
    assert list(RMSNorm.manifest(part.spec, "L.")) == ["L.n.weight"]
    x = torch.randn(9, 200, device=DEV)
    d = torch.randn(9, 200, device=DEV).to(DT[dtype])
    ref = plain_llama.rmsnorm((x + d.float()).cpu(), w.float(), 1e-4)
    out = part.forward(x, d, 9)
    assert_close(out, ref, dtype, "RMSNorm part")
    assert out.dtype == DT[dtype] and part.weight.dtype == torch.float32


def test_position_part_llama3_scaling():
    from kuiperllama_b200.config import PartSpec
    from kuiperllama_b200.parts import RotaryPosition
    for name in ("tiny1", "tiny2", "tiny3"):
        d = config_dict(name)
        hd = d.get("head_dim", d["hidden_size"] // d["num_attention_heads"])
        part = RotaryPosition(PartSpec("rope", {"head_dim": hd, "theta": d["rope_theta"], "scaling": d["rope_scaling"]}),
                              "", {}, _runtime("float32"))
        inv, rot = part.rotary()
        ref = plain_llama.rope_inverse_frequencies(hd, d["rope_theta"], d["rope_scaling"])
        assert rot == hd and inv.dtype == torch.float32 and torch.equal(inv.cpu(), ref)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_part(dtype):
    from kuiperllama_b200.config import PartSpec
    from kuiperllama_b200.parts import SwiGLUFeedForward
    torch.manual_seed(1)
    hid, inter = 96, 172
    names = {"gate": "g.weight", "up": "u.weight", "down": "d.weight"}
    w = {"P.g.weight": torch.randn(inter, hid) * 0.1, "P.u.weight": torch.randn(inter, hid) * 0.1,
         "P.d.weight": torch.randn(hid, inter) * 0.1}
    w = {k: v.bfloat16() for k, v in w.items()}
    part = SwiGLUFeedForward(PartSpec("swiglu", {"hidden_size": hid, "intermediate_size": inter, "names": names}), "P.", w,
                             _runtime(dtype))
    x = torch.randn(13, hid, device=DEV).to(DT[dtype])
    pw = {"P.mlp.gate_proj.weight": w["P.g.weight"].float(), "P.mlp.up_proj.weight": w["P.u.weight"].float(),
          "P.mlp.down_proj.weight": w["P.d.weight"].float()}
    ref = plain_llama.swiglu_feed_forward(x.float().cpu(), pw, "P.")
    assert_close(_dense(part.forward(x, None)), ref, dtype, "SwiGLU part")


def _attention_weights(hid, H, KV, hd, seed):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: (torch.randn(*s, generator=g) * 0.08).bfloat16()
    return {"A.q.weight": mk(H * hd, hid), "A.k.weight": mk(KV * hd, hid), "A.v.weight": mk(KV * hd, hid),
            "A.o.weight": mk(hid, H * hd)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,KV,hd", [(4, 4, 16), (6, 2, 48), (8, 1, 64)])
def test_attention_part_whole_and_token_by_token(dtype, H, KV, hd):
    from kuiperllama_b200.cache import SequenceCache
    from kuiperllama_b200.config import PartSpec
    from kuiperllama_b200.engine import Engine
    from kuiperllama_b200.parts import AttentionMixer, RotaryPosition
    hid, T = 80, 75
    w = _attention_weights(hid, H, KV, hd, seed=2)
    rt = _runtime(dtype)
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 32}
    pos = RotaryPosition(PartSpec("rope", {"head_dim": hd, "theta": 1e5, "scaling": scaling}), "", {}, rt)
    spec = PartSpec("attention", {"hidden_size": hid, "num_heads": H, "num_kv_heads": KV, "head_dim": hd, "window": None,
                                  "names": {"q": "q.weight", "k": "k.weight", "v": "v.weight", "o": "o.weight"}})
    mixer = AttentionMixer(spec, "A.", w, rt, pos)
    cache = SequenceCache([mixer.kv_request()], [None], [None], max_tokens=64 * 4, max_seq_len=128, dtype=DT[dtype], device=DEV)

    class _M:                                                      # the engine needs only these of a model here
        runtime = rt
        class spec:
            vocab_size = 10
    engine = Engine(_M, cache)
    x = torch.randn(T, hid, device=DEV).to(DT[dtype])
    c = {"num_attention_heads": H, "num_key_value_heads": KV, "head_dim": hd}
    pw = {"A.self_attn.q_proj.weight": w["A.q.weight"].float(), "A.self_attn.k_proj.weight": w["A.k.weight"].float(),
          "A.self_attn.v_proj.weight": w["A.v.weight"].float(), "A.self_attn.o_proj.weight": w["A.o.weight"].float()}
    ref = plain_llama.attention_mixer(x.float().cpu(), pw, "A.", c, plain_llama.rope_inverse_frequencies(hd, 1e5, scaling))
    with torch.inference_mode():
        slot = cache.alloc_slot()
        step = _step_for(engine, [(slot, T)])
        whole = _dense(mixer.forward(x, step, cache.view(0)))
        cache.free_slot(slot)
        slot = cache.alloc_slot()
        parts = []
        step = _step_for(engine, [(slot, T - 10)])
        parts.append(_dense(mixer.forward(x[:T - 10].contiguous(), step, cache.view(0))).float())
        cache.lengths[slot] = T - 10
        for t in range(T - 10, T):
            step = _step_for(engine, [(slot, 1)])
            parts.append(_dense(mixer.forward(x[t:t + 1].contiguous(), step, cache.view(0))).float())
            cache.lengths[slot] = t + 1
        cache.free_slot(slot)
    assert_close(whole, ref, dtype, "attention part, whole")
    assert_close(torch.cat(parts), ref, dtype, "attention part, last 10 one by one")


# ----------------------------------------------------------------------------- pluggable parts

def _register_toy_parts():
    """A mixer that keeps a running mean of its sequence's inputs as per-slot state (no keys
    or values), defined here, outside the package."""
    from kuiperllama_b200.cache import StateRequest
    from kuiperllama_b200.parts import Mixer, register_mixer
    from kuiperllama_b200.weights import TensorDecl

    @register_mixer("toy_running_mean")
    class RunningMeanMixer(Mixer):
        @classmethod
        def manifest(cls, spec, prefix):
            return {prefix + "toy.gain": TensorDecl((spec["hidden_size"],), role="vector", init="one_plus_normal")}

        def __init__(self, spec, prefix, tensors, runtime, position=None):
            super().__init__(spec, prefix, tensors, runtime, position)
            self.hidden = spec["hidden_size"]
            self.gain = tensors[prefix + "toy.gain"].to(device=runtime.device, dtype=torch.float32)

        def state_request(self):
            return StateRequest((self.hidden + 1,), torch.float32)   # running sum and count

        def forward(self, x, step, cache):
            # A test part may use torch operations; the package's own parts call its kernels.
            out = torch.empty_like(x)
            for i in range(step.n_seqs):
                slot, n = step.host_slots[i], step.host_new[i]
                r0 = sum(step.host_new[:i])
                rows = x[r0:r0 + n].float()
                st = cache.state[slot]
                sums = st[:self.hidden] + torch.cumsum(rows, dim=0)
                counts = st[self.hidden] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                out[r0:r0 + n] = (self.gain * sums / counts[:, None]).to(x.dtype)
                st[:self.hidden] = sums[-1]
                st[self.hidden] = counts[-1]
            return out
    return RunningMeanMixer


def _toy_reference(w, c, spec, tokens, toy_layers, schedule):
    """The plain implementation with the toy mixer in some layers and a schedule."""
    inv = plain_llama.rope_inverse_frequencies(c["head_dim"], c["rope_theta"], c["rope_scaling"])
    x = plain_llama.embedding(w["model.embed_tokens.weight"], tokens)
    eps = c["rms_norm_eps"]
    for layer in schedule:
        p = f"model.layers.{layer}."
        n = plain_llama.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        if layer in toy_layers:
            counts = torch.arange(1, len(tokens) + 1, dtype=torch.float32)[:, None]
            x = x + w[p + "toy.gain"] * torch.cumsum(n, dim=0) / counts
        else:
            x = x + plain_llama.attention_mixer(n, w, p, c, inv)
        x = x + plain_llama.swiglu_feed_forward(plain_llama.rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps), w, p)
    return plain_llama.output_logits(x, w, c)


def test_a_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    """Layer 1 of a three-layer model gets the toy mixer; layer 0 is scheduled twice (each
    execution has a cache of its own).  Built and stepped through the unchanged engine."""
    from kuiperllama_b200.config import PartSpec, ScheduleEntry, config_from_dict
    from kuiperllama_b200.engine import DecoderModel, Engine, SequenceInput, model_manifest
    from kuiperllama_b200.parts import Runtime
    from kuiperllama_b200.weights.random_init import random_tensor
    _register_toy_parts()
    cfg = config_from_dict(config_dict("tiny2"))
    spec = cfg.to_model_spec()
    layers = list(spec.layers)
    layers[1] = dataclasses.replace(layers[1], mixer=PartSpec("toy_running_mean", {"hidden_size": cfg.hidden_size}), position=None)
    order = [0, 1, 0, 2]
    spec = dataclasses.replace(spec, layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in order))
    manifest = model_manifest(spec)
    assert "model.layers.1.toy.gain" in manifest and "model.layers.1.self_attn.q_proj.weight" not in manifest
    tensors = {n: random_tensor(n, d, seed=5, std=0.02) for n, d in manifest.items()}
    model = DecoderModel(spec, tensors, Runtime(DEV, torch.float32))
    kv, st, _ = model.cache_requests()
    assert [r is not None for r in kv] == [True, False, True, True] and [s is not None for s in st] == [False, True, False, False]
    cache = model.new_cache(max_tokens=64 * 6)
    assert tuple(cache.groups[0].k.shape)[0] == 3 and cache.states[1].shape == (6, cfg.hidden_size + 1)
    engine = Engine(model, cache)
    w = {k: v.float() for k, v in tensors.items()}
    c = dict(config_dict("tiny2"), head_dim=cfg.head_dim)
    reqs = [random_tokens(n, cfg.vocab_size, seed=40 + n) for n in (30, 9)]
    with torch.inference_mode():
        for round_ in range(2):                                    # twice: the second time on reused slots and state
            slots = [engine.alloc_slot() for _ in reqs]
            first = engine.step([SequenceInput(s, r[:5], [0, 1, 2, 3, 4]) for s, r in zip(slots, reqs)])
            rest = {0: [], 1: []}
            for t in range(5, 30):
                live = [i for i in (0, 1) if t < len(reqs[i])]
                lg = engine.step([SequenceInput(slots[i], [reqs[i][t]], [0]) for i in live])
                for j, i in enumerate(live):
                    rest[i].append(lg[j:j + 1])
            for s in slots:
                engine.free_slot(s)
            for i in (0, 1):
                got = torch.cat([first[5 * i:5 * i + 5]] + rest[i])
                ref = _toy_reference(w, c, spec, reqs[i], {1}, order)
                assert_close(got, ref, "float32", f"toy model, request {i}, round {round_}")


def test_an_execution_can_read_another_executions_cache():
    """Schedule [0, 1, 1 reading entry 1's cache]: the third execution appends nothing and
    attends over what the second wrote."""
    from kuiperllama_b200.config import ScheduleEntry, config_from_dict
    from kuiperllama_b200.engine import DecoderModel, Engine, SequenceInput, model_manifest
    from kuiperllama_b200.parts import Runtime
    from kuiperllama_b200.weights.random_init import random_tensor
    cfg = config_from_dict(config_dict("tiny1"))
    spec = dataclasses.replace(cfg.to_model_spec(), schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1, cache_from=1)))
    tensors = {n: random_tensor(n, d, seed=6, std=0.05) for n, d in model_manifest(spec).items()}
    model = DecoderModel(spec, tensors, Runtime(DEV, torch.float32))
    cache = model.new_cache(max_tokens=64 * 4)
    assert tuple(cache.groups[0].k.shape)[0] == 2
    engine = Engine(model, cache)
    w = {k: v.float() for k, v in tensors.items()}
    c = dict(config_dict("tiny1"), head_dim=cfg.head_dim)
    tokens = random_tokens(70, cfg.vocab_size, seed=50)
    # reference: the third execution uses keys and values of the SECOND execution's input
    inv = plain_llama.rope_inverse_frequencies(c["head_dim"], c["rope_theta"], c["rope_scaling"])
    x = plain_llama.embedding(w["model.embed_tokens.weight"], tokens)
    x = plain_llama.decoder_block(x, w, 0, c, inv)
    p = "model.layers.1."
    n2 = plain_llama.rmsnorm(x, w[p + "input_layernorm.weight"], c["rms_norm_eps"])
    x = plain_llama.decoder_block(x, w, 1, c, inv)
    n3 = plain_llama.rmsnorm(x, w[p + "input_layernorm.weight"], c["rms_norm_eps"])
    T, H, KV, hd = len(tokens), c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    pos = torch.arange(T)
    q = plain_llama.rope_rotate((n3 @ w[p + "self_attn.q_proj.weight"].T).view(T, H, hd), pos, inv)
    k = plain_llama.rope_rotate((n2 @ w[p + "self_attn.k_proj.weight"].T).view(T, KV, hd), pos, inv)
    v = (n2 @ w[p + "self_attn.v_proj.weight"].T).view(T, KV, hd)
    x = x + plain_llama.attention_scores_softmax_values(q, k, v).reshape(T, H * hd) @ w[p + "self_attn.o_proj.weight"].T
    x = x + plain_llama.swiglu_feed_forward(plain_llama.rmsnorm(x, w[p + "post_attention_layernorm.weight"], c["rms_norm_eps"]), w, p)
    ref = plain_llama.output_logits(x, w, c)
    with torch.inference_mode():
        slot = engine.alloc_slot()
        got = [engine.step([SequenceInput(slot, tokens[:66], list(range(66)))])]
        got += [engine.step([SequenceInput(slot, [t], [0])]) for t in tokens[66:]]
        engine.free_slot(slot)
    assert_close(torch.cat(got), ref, "float32", "cache read from another execution")


def test_toy_feed_forward_with_routing_and_toy_position_encoding():
    """Two more kinds of parts defined outside the package: a feed-forward that routes every token
    to one of three small experts (router logits in float32), and a learned absolute position
    encoding that is added to the embeddings.  Registered, built from a ModelSpec and stepped
    whole and token by token through the unchanged engine."""
    from kuiperllama_b200.config import PartSpec, config_from_dict
    from kuiperllama_b200.engine import DecoderModel, Engine, SequenceInput, model_manifest
    from kuiperllama_b200.parts import FeedForward, PositionEncoding, Runtime, register_feed_forward, register_position
    from kuiperllama_b200.weights import TensorDecl
    from kuiperllama_b200.weights.random_init import random_tensor

    @register_feed_forward("toy_top1_experts")
    class Top1Experts(FeedForward):
        @classmethod
        def manifest(cls, spec, prefix):
            h, e, i = spec["hidden_size"], spec["experts"], spec["inner"]
            m = {prefix + "moe.router": TensorDecl((e, h), role="vector")}
            for k in range(e):
                m[prefix + f"moe.{k}.up"] = TensorDecl((i, h))
                m[prefix + f"moe.{k}.down"] = TensorDecl((h, i))
            return m

        def __init__(self, spec, prefix, tensors, runtime):
            super().__init__(spec, prefix, tensors, runtime)
            e = spec["experts"]
            self.router = tensors[prefix + "moe.router"].to(runtime.device, torch.float32)
            self.up = [tensors[prefix + f"moe.{k}.up"].to(runtime.device, torch.float32) for k in range(e)]
            self.down = [tensors[prefix + f"moe.{k}.down"].to(runtime.device, torch.float32) for k in range(e)]

        def forward(self, x, step):
            xf = x.float()
            choice = (xf @ self.router.T).argmax(dim=-1)                 # float32 router logits
            out = torch.zeros_like(xf)
            for k in range(len(self.up)):
                rows = (choice == k).nonzero().flatten()
                if rows.numel():
                    out[rows] = torch.relu(xf[rows] @ self.up[k].T) @ self.down[k].T
            return out.to(x.dtype)

    @register_position("toy_learned_absolute")
    class LearnedAbsolute(PositionEncoding):
        @classmethod
        def manifest(cls, spec, prefix):
            return {prefix + "pos.table": TensorDecl((spec["positions"], spec["hidden_size"]), role="vector")}

        def __init__(self, spec, prefix, tensors, runtime):
            super().__init__(spec, prefix, tensors, runtime)
            self.table = tensors[prefix + "pos.table"].to(runtime.device, torch.float32)

        def add_to_embeddings(self, residual, step):
            residual[:step.n_tokens] += self.table[step.positions[:step.n_tokens].long()]

    cfg = config_from_dict(config_dict("tiny1"))
    spec = cfg.to_model_spec()
    layers = list(spec.layers)
    pos = PartSpec("toy_learned_absolute", {"positions": 128, "hidden_size": cfg.hidden_size})
    ffn = PartSpec("toy_top1_experts", {"hidden_size": cfg.hidden_size, "experts": 3, "inner": 40})
    layers[0] = dataclasses.replace(layers[0], position=pos)               # no rotation in layer 0: absolute table instead
    layers[1] = dataclasses.replace(layers[1], feed_forward=ffn)
    spec = dataclasses.replace(spec, layers=tuple(layers))
    manifest = model_manifest(spec)
    assert "model.layers.0.pos.table" in manifest and "model.layers.1.moe.2.down" in manifest
    assert "model.layers.1.mlp.gate_proj.weight" not in manifest
    tensors = {n: random_tensor(n, d, seed=8, std=0.05) for n, d in manifest.items()}
    model = DecoderModel(spec, tensors, Runtime(DEV, torch.float32))
    engine = Engine(model, model.new_cache(max_tokens=64 * 4))
    w = {k: v.float() for k, v in tensors.items()}
    c = dict(config_dict("tiny1"), head_dim=cfg.head_dim)
    tokens = random_tokens(40, cfg.vocab_size, seed=60)
    # the same model with the plain implementation's functions
    inv = plain_llama.rope_inverse_frequencies(c["head_dim"], c["rope_theta"], None)
    x = plain_llama.embedding(w["model.embed_tokens.weight"], tokens) + w["model.layers.0.pos.table"][:40]
    for layer in (0, 1):
        p = f"model.layers.{layer}."
        n = plain_llama.rmsnorm(x, w[p + "input_layernorm.weight"], c["rms_norm_eps"])
        no_rotation = torch.zeros_like(inv)                                 # angle 0: layer 0 has no rotary part
        x = x + plain_llama.attention_mixer(n, w, p, c, no_rotation if layer == 0 else inv)
        n = plain_llama.rmsnorm(x, w[p + "post_attention_layernorm.weight"], c["rms_norm_eps"])
        if layer == 1:
            choice = (n @ w[p + "moe.router"].T).argmax(-1)
            f = torch.stack([torch.relu(n[t] @ w[p + f"moe.{int(choice[t])}.up"].T) @ w[p + f"moe.{int(choice[t])}.down"].T
                             for t in range(40)])
        else:
            f = plain_llama.swiglu_feed_forward(n, w, p)
        x = x + f
    ref = plain_llama.output_logits(x, w, c)
    with torch.inference_mode():
        slot = engine.alloc_slot()
        got = [engine.step([SequenceInput(slot, tokens[:33], list(range(33)))])]
        got += [engine.step([SequenceInput(slot, [t], [0])]) for t in tokens[33:]]
        engine.free_slot(slot)
    assert_close(torch.cat(got), ref, "float32", "toy routed feed-forward and absolute positions")


def _windowed_reference(w, c, tokens, windows):
    """The plain implementation with a window in some layers: a query at position p reads the
    keys max(0, p - window + 1) .. p (``windows[layer]`` None: all keys)."""
    inv = plain_llama.rope_inverse_frequencies(c["head_dim"], c["rope_theta"], c["rope_scaling"])
    x = plain_llama.embedding(w["model.embed_tokens.weight"], tokens)
    eps, T = c["rms_norm_eps"], len(tokens)
    H, KV, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    for layer, window in enumerate(windows):
        p = f"model.layers.{layer}."
        n = plain_llama.rmsnorm(x, w[p + "input_layernorm.weight"], eps)
        if window is None:
            x = x + plain_llama.attention_mixer(n, w, p, c, inv)
        else:
            pos = torch.arange(T)
            q = plain_llama.rope_rotate((n @ w[p + "self_attn.q_proj.weight"].T).view(T, H, hd), pos, inv)
            k = plain_llama.rope_rotate((n @ w[p + "self_attn.k_proj.weight"].T).view(T, KV, hd), pos, inv)
            v = (n @ w[p + "self_attn.v_proj.weight"].T).view(T, KV, hd)
            o = torch.empty(T, H, hd)
            for t in range(T):
                lo = max(0, t - window + 1)
                o[t] = plain_llama.attention_scores_softmax_values(q[lo:t + 1], k[lo:t + 1], v[lo:t + 1])[-1]
            x = x + o.reshape(T, H * hd) @ w[p + "self_attn.o_proj.weight"].T
        x = x + plain_llama.swiglu_feed_forward(plain_llama.rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps), w, p)
    return plain_llama.output_logits(x, w, c)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_with_a_window_beside_layers_without(dtype):
    """Layer 1 of two reads all keys, layer 0 a window of 70: two cache groups, and the windowed
    one gives pages back while the sequences grow (its pool is too small to hold them whole).
    Pages given back by one sequence are taken by the other at once, so a kernel that read
    below the window would read the other sequence's keys.  Two rounds: slots and pages reused."""
    from kuiperllama_b200.config import PartSpec, config_from_dict
    from kuiperllama_b200.engine import DecoderModel, Engine, SequenceInput, model_manifest
    from kuiperllama_b200.parts import Runtime
    from kuiperllama_b200.weights.random_init import random_tensor
    W = 70
    cfg = config_from_dict(config_dict("tiny3"))
    spec = cfg.to_model_spec()
    layers = list(spec.layers)
    layers[0] = dataclasses.replace(layers[0], mixer=PartSpec("attention", dict(layers[0].mixer.params, window=W)))
    spec = dataclasses.replace(spec, layers=tuple(layers))
    manifest = model_manifest(spec)
    tensors = {n: random_tensor(n, d, seed=9, std=0.05) for n, d in manifest.items()}
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    model = DecoderModel(spec, tensors, Runtime(DEV, dt))
    cache = model.new_cache(max_tokens=64 * 12, max_seq_len=64 * 6, max_slots=2, window_step_tokens=130)
    by_window = {g.request.window: g for g in cache.groups}
    assert set(by_window) == {None, W} and by_window[W].pages.n == 2 * 5 < by_window[None].pages.n
    engine = Engine(model, cache)
    w = {k: v.to(dt).float() for k, v in tensors.items()}
    c = dict(config_dict("tiny3"))
    reqs = [random_tokens(n, cfg.vocab_size, seed=60 + n) for n in (330, 170)]
    prompt = (130, 100)
    with torch.inference_mode():
        for round_ in range(2):
            slots = [engine.alloc_slot() for _ in reqs]
            first = engine.step([SequenceInput(s, r[:n], list(range(n))) for s, r, n in zip(slots, reqs, prompt)])
            got = {0: [first[:prompt[0]]], 1: [first[prompt[0]:]]}
            done = list(prompt)
            while any(done[i] < len(reqs[i]) for i in (0, 1)):
                live = [i for i in (0, 1) if done[i] < len(reqs[i])]
                lg = engine.step([SequenceInput(slots[i], [reqs[i][done[i]]], [0]) for i in live])
                for j, i in enumerate(live):
                    got[i].append(lg[j:j + 1].clone())
                    done[i] += 1
            assert by_window[W].first_block[slots[0]] == (330 - 1 - W + 1) // 64 > 0
            assert len(by_window[W].pages_of(slots[0])) <= 3 and len(by_window[None].pages_of(slots[0])) == 6
            for s in slots:
                engine.free_slot(s)
            assert cache.pages_held() == [0, 0]
            for i in (0, 1):
                ref = _windowed_reference(w, c, reqs[i], [W, None])
                assert_close(torch.cat(got[i]), ref, dtype, f"window in layer 0, request {i}, round {round_}", layers=2, stream="wide")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_options_around_the_layers_embedding_multiplier_and_logit_scale_and_soft_cap(dtype):
    """A ``ModelSpec`` may ask for x = m * E[token] and for logits = c * tanh(s * logits / c): steps
    some decoders have around the layers and the Llama decoder has not.  They are fields of the
    spec (None for Llama), not code of an architecture."""
    from kuiperllama_b200.config import config_from_dict
    from kuiperllama_b200.engine import DecoderModel, Engine, SequenceInput, model_manifest
    from kuiperllama_b200.parts import Runtime
    from kuiperllama_b200.weights.random_init import random_tensor
    cfg = config_from_dict(config_dict("tiny3"))                    # untied: the classifier is not the embedding table
    mult, scale, cap = math.sqrt(cfg.hidden_size), 4.0, 1.5
    spec = dataclasses.replace(cfg.to_model_spec(), embedding_multiplier=mult, logit_scale=scale, logit_softcap=cap)
    tensors = {n: random_tensor(n, d, seed=21, std=0.05) for n, d in model_manifest(spec).items()}
    dt = DT[dtype]
    model = DecoderModel(spec, tensors, Runtime(DEV, dt))
    engine = Engine(model, model.new_cache(max_tokens=64 * 4))
    w = {k: v.to(dt).float() for k, v in tensors.items()}
    w["model.embed_tokens.weight"] = w["model.embed_tokens.weight"] * mult
    tokens = random_tokens(90, cfg.vocab_size, seed=77)
    raw = plain_llama.forward_logits(w, dict(config_dict("tiny3")), tokens)
    ref = cap * torch.tanh(scale * raw / cap)
    assert float(ref.abs().max()) > 0.5 * cap                       # the cap bites
    with torch.inference_mode():
        slot = engine.alloc_slot()
        got = [engine.step([SequenceInput(slot, tokens[:60], list(range(60)))])]
        got += [engine.step([SequenceInput(slot, [t], [0])]) for t in tokens[60:]]
        engine.free_slot(slot)
    got = torch.cat(got).float().cpu()
    # tanh only shrinks differences, so the error after the cap is bounded by the error before it
    assert float((got - ref).abs().max()) <= tolerance(dtype, scale * raw, layers=2, stream="wide")
    assert float((got - ref).abs().max()) < 0.05 * float((got - scale * raw).abs().max())      # and the cap was applied
    with pytest.raises(ValueError, match="logit_softcap"):
        dataclasses.replace(spec, logit_softcap=0.0).validate()
