"""Generation through the Python entry point and the command line against the plain
implementation: greedy tokens, temperature and top-k draws, stop tokens, more requests than
fit in one batch."""
from __future__ import annotations

import os
import subprocess
import sys

import pytest
import torch

import plain_llama
from helpers import config_dict, random_tokens, tolerance

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _check_greedy(folder, dtype, prompt, got, stop=()):
    """Every generated token is the plain implementation's greedy token, unless the plain
    logits' two best are closer than the dtype's tolerance (then either may win)."""
    c, w = plain_llama.read_config(folder), plain_llama.read_weights(folder)
    seq = list(prompt)
    for tok in got:
        logits = plain_llama.forward_logits(w, c, seq)[-1]
        best = plain_llama.argmax_token(logits)
        if tok != best:
            assert float(logits[best] - logits[tok]) <= 2 * tolerance(dtype, logits), (dtype, len(seq), tok, best)
        assert tok not in stop
        seq.append(tok)
    return seq


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,seed", [("tiny1", 0), ("tiny2", 1)])
def test_greedy_generation_through_the_entry_point(model_folders, name, seed, dtype):
    import kuiperllama_b200 as kl
    folder = model_folders(name, seed=seed)
    vocab = config_dict(name)["vocab_size"]
    lens = [5, 9, 13] if name == "tiny1" else [1, 7, 20, 33]          # the workloads of the two tiny configurations
    prompts = [random_tokens(n, vocab, seed=10 * n) for n in lens]
    m = kl.load(folder, dtype=dtype, max_tokens=64 * 8, max_batch=8)
    out = m.generate(prompts, max_new_tokens=12, stop_ids=[])
    assert [len(o) for o in out] == [12] * len(prompts)
    for p, o in zip(prompts, out):
        _check_greedy(folder, dtype, p, o)
    if dtype == "float32":
        c, w = plain_llama.read_config(folder), plain_llama.read_weights(folder)
        assert out[1] == plain_llama.greedy_generate(w, c, prompts[1], 12)
    assert m.cache.slots.held() == 0 and m.cache.pages_held() == [0]
    assert m.generate(prompts[0], max_new_tokens=3, stop_ids=[]) == out[0][:3]     # a single prompt, not nested


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_log_probabilities_and_logits_of_the_generated_tokens(model_folders, dtype):
    """``return_logprobs`` / ``return_logits``: every new token comes with log softmax(logits)[token]
    and with the logits row it was chosen from, also when batches shrink and graphs replay."""
    import kuiperllama_b200 as kl
    folder = model_folders("tiny2", seed=1)
    vocab = config_dict("tiny2")["vocab_size"]
    prompts = [random_tokens(n, vocab, seed=40 + n) for n in (6, 30, 2)]
    m = kl.load(folder, dtype=dtype, max_tokens=64 * 6, max_batch=4)
    out = m.generate(prompts, max_new_tokens=9, temperature=0.9, seed=3, stop_ids=[7], return_logprobs=True, return_logits=True)
    results = m.last_results
    assert out == m.generate(prompts, max_new_tokens=9, temperature=0.9, seed=3, stop_ids=[7])       # asking changes no token
    c, w = plain_llama.read_config(folder), plain_llama.read_weights(folder)
    assert len({len(o) for o in out}) > 1 or all(len(o) == 9 for o in out)
    assert all(r.logprobs is None and r.logits is None for r in m.last_results)
    for p, o, res in zip(prompts, out, results):
        assert res.tokens == o and len(res.logprobs) == len(o) == len(res.logits)
        ref = plain_llama.forward_logits(w, c, list(p) + o)[len(p) - 1:-1] if o else None
        for i, tok in enumerate(o):
            row = res.logits[i]
            assert row.shape == (vocab,) and row.dtype == torch.float32
            assert float((row - ref[i]).abs().max()) <= tolerance(dtype, ref[i])
            want = float(torch.log_softmax(row.double(), dim=0)[tok])
            assert abs(res.logprobs[i] - want) < 1e-4, (i, tok, res.logprobs[i], want)
    assert m.cache.slots.held() == 0


def test_stop_tokens_and_more_requests_than_the_cache_holds(model_folders):
    import kuiperllama_b200 as kl
    folder = model_folders("tiny2", seed=1)
    vocab = config_dict("tiny2")["vocab_size"]
    prompts = [random_tokens(3 + (7 * i) % 40, vocab, seed=900 + i) for i in range(10)]
    m = kl.load(folder, dtype="float32", max_tokens=64 * 3, max_batch=4)          # three pages: three requests at a time
    free = m.generate(prompts, max_new_tokens=10, stop_ids=[])
    assert m.last_stats.batches == 4
    # make the 4th token of request 2 and the 1st of request 5 stop tokens
    stop = [free[2][3], free[5][0]]
    got = m.generate(prompts, max_new_tokens=10, stop_ids=stop)
    for i, (f, g) in enumerate(zip(free, got)):
        cut = next((j for j, t in enumerate(f) if t in stop), len(f))
        assert g == f[:cut], f"request {i}"
        assert m.last_results[i].finish_reason == ("stop" if cut < len(f) else "length")
    assert got[5] == [] and len(got[2]) <= 3
    assert m.cache.slots.held() == 0 and m.cache.pages_held() == [0]
    # the configuration's own eos ids (7 and 9) are the default stop set
    assert m.stop_token_ids == (7, 9)
    assert m.generate(prompts, max_new_tokens=10, stop_ids=stop, include_stop=True)[5] == [free[5][0]]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_sampling_follows_the_counter_draw(model_folders, dtype):
    """12 steps at temperature 0.8 with a seeded sampler (the workload of the second tiny
    configuration): every drawn token's interval of the plain cumulative distribution holds
    the draw of (seed, request, step); batch of four and one by one give the same tokens."""
    import kuiperllama_b200 as kl
    folder = model_folders("tiny2", seed=1)
    c, w = plain_llama.read_config(folder), plain_llama.read_weights(folder)
    prompts = [random_tokens(n, c["vocab_size"], seed=20 * n) for n in (1, 7, 20, 33)]
    m = kl.load(folder, dtype=dtype, max_tokens=64 * 8)
    out = m.generate(prompts, max_new_tokens=12, temperature=0.8, seed=77, stop_ids=[])
    slack = {"float32": 1e-4, "bfloat16": 3e-2}[dtype]
    for r, (p, o) in enumerate(zip(prompts, out)):
        seq = list(p)
        for step, tok in enumerate(o):
            probs = plain_llama.temperature_probabilities(plain_llama.forward_logits(w, c, seq)[-1], 0.8)
            u = plain_llama.uniform_from_counter(77, r, step)
            cdf = torch.cumsum(probs, 0)
            lo = float(cdf[tok - 1]) if tok else 0.0
            assert lo - slack <= u <= float(cdf[tok]) + slack, (dtype, r, step, tok, u, lo, float(cdf[tok]))
            seq.append(tok)
    assert out != m.generate(prompts, max_new_tokens=12, temperature=0.8, seed=78, stop_ids=[])
    if dtype == "float32":
        assert m.generate(prompts, max_new_tokens=12, temperature=0.8, seed=77, stop_ids=[]) == out
        # request 2 alone, told that it is request 2: the same tokens as inside the batch
        from kuiperllama_b200.engine import EngineBackend, run_requests
        from kuiperllama_b200.sampling import Sampler, SamplingParams
        be = EngineBackend(m.engine, Sampler(SamplingParams(temperature=0.8, seed=77)))

        class Shift:
            def __getattr__(self, k): return getattr(be, k)
            def prefill(self, s, p, ids): return be.prefill(s, p, [2])
            def decode(self, s, prev, take, ids, st): return be.decode(s, prev, take, [2], st)
        with torch.inference_mode():
            alone = run_requests(Shift(), [prompts[2]], 12)
        assert alone[0].tokens == out[2]
    topk = m.generate(prompts, max_new_tokens=6, temperature=1.5, top_k=3, seed=5, stop_ids=[])
    for p, o in zip(prompts, topk):
        seq = list(p)
        for tok in o:
            logits = plain_llama.forward_logits(w, c, seq)[-1]
            third = float(torch.topk(logits, 3).values[-1])
            assert float(logits[tok]) >= third - 2 * tolerance(dtype, logits)
            seq.append(tok)


def test_command_line(model_folders):
    folder = model_folders("tiny1", seed=0)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "llama_infer"), folder, "--prompt-ids", "1,5,9,200", "--prompt-ids",
           "7 8", "--steps", "12", "--dtype", "float32"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = r.stdout.strip().splitlines()
    assert lines[0] == "Generating..." and any(l.startswith("steps/s:") for l in lines)
    first = [int(t) for t in lines[1].split()]
    c, w = plain_llama.read_config(folder), plain_llama.read_weights(folder)
    # --steps counts positions, prompt included, as the demo does: 12 - 2 + 1 new tokens for the shorter prompt
    assert len(first) <= 11 and first == plain_llama.greedy_generate(w, c, [1, 5, 9, 200], 11, stop_ids=[2])[:len(first)]
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llama_infer"), folder], capture_output=True, text=True, timeout=600)
    assert bad.returncode != 0 and "tokenizer" in bad.stderr


def test_command_line_without_a_folder_with_a_prompt_file_logits_and_rates(tmp_path):
    """``--config FILE --random-weights`` builds the model from a config.json alone; ``--prompt-file`` brings
    one prompt a line; ``--print-logits`` shows every new token's logit, log-probability and the top five;
    ``--bench`` runs twice and prints the second run's rates as one JSON line."""
    import json
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(config_dict("tiny2")))
    prompts = tmp_path / "prompts.txt"
    prompts.write_text("1, 5, 9\n\n44 45 46 47 48\n")
    cmd = [sys.executable, os.path.join(ROOT, "bin", "llama_infer"), "--config", str(cfg), "--random-weights", "--seed", "3",
           "--prompt-file", str(prompts), "--max-new-tokens", "4", "--stop-ids", "", "--print-logits", "--bench", "--max-ctx", "128",
           "--max-batch", "2"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = r.stdout.strip().splitlines()
    tokens = [[int(t) for t in l.split()] for l in lines if l and all(c.isdigit() or c == " " for c in l)]
    assert [len(t) for t in tokens] == [4, 4]
    shown = [l for l in lines if l.startswith("  token ")]
    assert len(shown) == 8
    first = shown[0].split()                                      # "token T logit X logprob Y | top: i:v ..."
    assert int(first[1]) == tokens[0][0] and float(first[5]) <= 0.0
    top = first[first.index("top:") + 1]
    assert int(top.split(":")[0]) == tokens[0][0] and abs(float(top.split(":")[1]) - float(first[3])) < 1e-3    # greedy: the top one
    rates = [json.loads(l) for l in lines if l.startswith("{")]
    assert len(rates) == 1 and rates[0]["prompts"] == 2 and rates[0]["prefill_tokens"] == 8 and rates[0]["decode_steps"] == 3
    assert rates[0]["decode_tokens_per_s"] > 0
    # neither a folder nor a configuration: refused with the way out
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llama_infer"), "--random-weights"], capture_output=True, text=True, timeout=600)
    assert bad.returncode != 0 and "--config" in bad.stderr


def test_per_kernel_timing_of_a_generation(model_folders):
    """``profiling.kernel_timing``: every kernel entry point between two CUDA events, summed by name."""
    import kuiperllama_b200 as kl
    from kuiperllama_b200 import profiling
    from kuiperllama_b200.csrc import ops
    folder = model_folders("tiny3", seed=2)
    m = kl.load(folder, dtype="bfloat16", max_tokens=64 * 4, max_batch=2, use_graphs=False)
    prompts = [random_tokens(n, config_dict("tiny3")["vocab_size"], seed=n) for n in (40, 9)]
    plain = m.generate(prompts, max_new_tokens=5, stop_ids=[])
    before = ops.gemm_skinny
    with profiling.kernel_timing() as times:
        assert m.generate(prompts, max_new_tokens=5, stop_ids=[]) == plain           # timing changes no token
    assert ops.gemm_skinny is before                                                 # the entry points are back
    totals = times.totals()
    assert totals["embedding"][0] == 5 and totals["argmax_rows"][0] == 5             # one prefill and four decode steps
    assert totals["attention_tcgen05"][0] == 2 and totals["attention_decode_fused"][0] == 2 * 4
    assert all(ms > 0 for _, ms in totals.values())
    assert "total over" in times.report()
