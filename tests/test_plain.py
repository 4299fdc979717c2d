"""The plain implementation itself (no GPU): against the logits that ExiledOfCode/KuiperLLama's
own tools/model.py gave for the same weights (tests/golden/make_golden.py), and its parts
against independent formulas."""
import math
import os

import pytest
import torch

import plain_llama
from helpers import config_dict, plain_logits

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["tiny1", "tiny2"])
def test_against_the_reference_models_logits(name):
    """The golden file carries the weights that KuiperLLama's tools/model.py ran on, so this anchor
    holds whatever random numbers the torch build at hand would draw."""
    gold = torch.load(os.path.join(GOLDEN, f"{name}.pt"))
    c = config_dict(name)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    c.setdefault("head_dim", c["hidden_size"] // c["num_attention_heads"])
    w = {k: v.float() for k, v in gold["weights"].items()}
    got = plain_llama.forward_logits(w, c, gold["tokens"])
    assert got.shape == gold["logits"].shape
    assert float((got - gold["logits"]).abs().max()) < 2e-5 * float(gold["logits"].abs().max())


def test_random_weights_mode_is_stable(model_folders):
    """The random-weights mode writes the tensors the golden files were made from; if a torch build
    draws other numbers this fails and says how to make the files anew (nothing is skipped)."""
    for name, seed in (("tiny1", 0), ("tiny2", 1)):
        gold = torch.load(os.path.join(GOLDEN, f"{name}.pt"))
        w = plain_llama.read_weights(model_folders(name, seed=seed))
        same = set(w) == set(gold["weights"]) and all(torch.equal(w[k], gold["weights"][k].float()) for k in w)
        assert same, (f"{name}: this torch build draws other random weights than the one that made tests/golden/{name}.pt; "
                      "the anchor above still holds (it uses the stored weights); to refresh: "
                      "python tests/golden/make_golden.py <checkout of ExiledOfCode/KuiperLLama>")


# Worked by hand from the published meaning of rope_type "llama3" (wavelength = 2 pi / freq; below
# original / high_freq_factor: unchanged; above original / low_freq_factor: divided by factor; between:
# smooth = (original / wavelength - low) / (high - low), freq * ((1 - smooth) / factor + smooth)).
# (name, head_dim, theta, scaling, last unchanged j, first fully divided j, (j, smooth, new freq) of one pair between)
LLAMA3_ROPE_PINS = [
    ("Llama-3.1-8B", 128, 500000.0, dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                         original_max_position_embeddings=8192), 28, 35, (32, 0.2812826, 5.248462e-4)),
    ("Llama-3.2-1B", 64, 500000.0, dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                        original_max_position_embeddings=8192), 14, 18, (16, 0.2812826, 4.295568e-4)),
    ("tiny2", 32, 500000.0, dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                 original_max_position_embeddings=64), 1, 3, (2, 0.3250936, 7.940301e-2)),
]


@pytest.mark.parametrize("pin", LLAMA3_ROPE_PINS, ids=[p[0] for p in LLAMA3_ROPE_PINS])
def test_llama3_rope_scaling_against_worked_values(pin):
    """Both statements of the rule (the oracle's and the package's) against numbers worked out by
    hand for the parameter sets of Llama-3.1-8B, Llama-3.2-1B and tiny2: where the unchanged band
    ends, where the divided band starts, and one interpolated frequency."""
    from kuiperllama_b200.parts.position import rotary_inverse_frequencies
    _, hd, theta, scaling, last_same, first_divided, (j, smooth, value) = pin
    plain = plain_llama.rope_inverse_frequencies(hd, theta, scaling).double().tolist()
    ours = rotary_inverse_frequencies(hd, theta, scaling)
    base = [theta ** (-2.0 * i / hd) for i in range(hd // 2)]
    for got in (plain, ours):
        assert len(got) == hd // 2
        for i in range(hd // 2):
            if i <= last_same:
                assert got[i] == pytest.approx(base[i], rel=1e-6), i
            elif i >= first_divided:
                assert got[i] == pytest.approx(base[i] / scaling["factor"], rel=1e-6), i
            else:
                assert base[i] / scaling["factor"] < got[i] < base[i], i
        assert got[j] == pytest.approx(value, rel=2e-6)
        assert got[j] == pytest.approx(base[j] * ((1 - smooth) / scaling["factor"] + smooth), rel=2e-6)
    assert ours == pytest.approx(plain, rel=1e-6)


def test_rope_frequencies_against_float64_numpy():
    import numpy as np
    for name in ("tiny1", "tiny2", "tiny3"):
        c = config_dict(name)
        hd = c.get("head_dim", c["hidden_size"] // c["num_attention_heads"])
        got = plain_llama.rope_inverse_frequencies(hd, c["rope_theta"], c["rope_scaling"]).double().numpy()
        f = c["rope_theta"] ** (-np.arange(0, hd, 2, dtype=np.float64) / hd)
        if c["rope_scaling"]:
            s = c["rope_scaling"]
            lam = 2 * np.pi / f
            o = s["original_max_position_embeddings"]
            smooth = np.clip((o / lam - s["low_freq_factor"]) / (s["high_freq_factor"] - s["low_freq_factor"]), 0, 1)
            f = (1 - smooth) * f / s["factor"] + smooth * f
        assert np.allclose(got, f, rtol=1e-6)
        if c["rope_scaling"]:
            assert got[0] == pytest.approx(1.0) and got[-1] < (c["rope_theta"] ** (-(hd - 2) / hd)) * 0.9


def test_rotation_keeps_norms_and_relative_angles():
    inv = plain_llama.rope_inverse_frequencies(32, 10000.0, None)
    q, k = torch.randn(1, 1, 32), torch.randn(1, 1, 32)
    d = []
    for p in (0, 5, 40):
        rq = plain_llama.rope_rotate(q, torch.tensor([p + 3]), inv)
        rk = plain_llama.rope_rotate(k, torch.tensor([p]), inv)
        assert torch.allclose(rq.norm(), q.norm(), rtol=1e-5)
        d.append(float((rq * rk).sum()))
    assert abs(d[0] - d[1]) < 1e-4 and abs(d[0] - d[2]) < 1e-4        # the score depends on the distance only


def test_attention_is_causal_and_groups_heads():
    T, H, KV, hd = 6, 4, 2, 8
    q, k, v = torch.randn(T, H, hd), torch.randn(T, KV, hd), torch.randn(T, KV, hd)
    o = plain_llama.attention_scores_softmax_values(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -9.0                                     # the future does not reach positions 0..3
    assert torch.equal(plain_llama.attention_scores_softmax_values(q, k2, v2)[:4], o[:4])
    assert torch.allclose(o[0], v[0].repeat_interleave(2, dim=0))  # one key: the value itself, heads 0,1 -> kv head 0
    kk, vv = k.repeat_interleave(2, dim=1), v.repeat_interleave(2, dim=1)
    s = torch.einsum("thd,shd->hts", q, kk) / math.sqrt(hd)
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), -math.inf)
    assert torch.allclose(o, torch.einsum("hts,shd->thd", torch.softmax(s, -1), vv), atol=1e-6)


def test_rmsnorm_swiglu_argmax_and_sampling_helpers():
    x, w = torch.randn(3, 10), torch.randn(10)
    assert torch.allclose(plain_llama.rmsnorm(x, w, 1e-5), w * x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5), atol=1e-6)
    assert plain_llama.argmax_token(torch.tensor([1.0, 3.0, 3.0, 2.0])) == 1   # the lowest index among equals
    p = plain_llama.temperature_probabilities(torch.tensor([0.0, 1.0, 2.0, 3.0]), 0.5, top_k=2)
    assert p[0] == 0 and p[1] == 0 and abs(float(p.sum()) - 1) < 1e-12 and float(p[3] / p[2]) == pytest.approx(math.exp(2.0))
    assert plain_llama.inverse_cdf_pick(torch.tensor([0.25, 0.25, 0.5]), 0.49) == 1
    assert plain_llama.inverse_cdf_pick(torch.tensor([0.25, 0.25, 0.5]), 0.5) == 2
    from kuiperllama_b200.sampling import uniform_from_counter
    us = [plain_llama.uniform_from_counter(7, r, s) for r in range(20) for s in range(20)]
    assert us == [uniform_from_counter(7, r, s) for r in range(20) for s in range(20)]
    assert 0.4 < sum(us) / len(us) < 0.6 and min(us) >= 0 and max(us) < 1 and len(set(us)) > 390
