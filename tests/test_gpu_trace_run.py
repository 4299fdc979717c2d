"""bin/trace_run as a user runs it: the same requests whole, with the last 32 tokens one by
one, and in batches of unequal lengths, in float32 and bfloat16, against the plain
implementation."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import assert_close, config_dict, plain_logits, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _replay(folder, dtype, steps, out_dir, max_tokens):
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens)]
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        for s in steps:
            p.stdin.write(json.dumps(s) + "\n")
            p.stdin.flush()
            line = p.stdout.readline().strip()                     # the next step only after "done <step>"
            assert line == f"done {s['step']}", (line, p.stderr.read()[-3000:] if p.poll() is not None else "")
        p.stdin.close()
        assert p.wait(timeout=120) == 0, p.stderr.read()[-3000:]
    finally:
        if p.poll() is None:
            p.kill()


def _read(out_dir, step, vocab):
    return torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(-1, vocab).copy())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,seed", [("tiny1", 0), ("tiny2", 1)])
def test_trace_replay(model_folders, tmp_path, name, seed, dtype):
    folder = model_folders(name, seed=seed)
    vocab = config_dict(name)["vocab_size"]
    reqs = {rid: random_tokens(n, vocab, seed=3000 + n) for rid, n in (("a", 100), ("b", 40), ("c", 77), ("d", 33))}
    ref = {rid: plain_logits(folder, t) for rid, t in reqs.items()}
    steps, expect = [], {}
    no = 0

    def add(entries, end=()):
        nonlocal no
        steps.append({"step": no, "entries": entries, "end": list(end)})
        rows = [ref[e["id"][0]][e["_at"] + w] for e in entries for w in e["want"]]
        for e in entries:
            del e["_at"]
        if rows:
            expect[no] = torch.stack(rows)
        no += 1

    # 1. each request alone and whole, every position wanted
    for rid, t in reqs.items():
        add([{"id": rid + "-whole", "tokens": t, "want": list(range(len(t))), "_at": 0}], end=[rid + "-whole"])
    # 2. the last 32 tokens one by one (nothing wanted from the first part of "c")
    for rid in ("a", "c"):
        t = reqs[rid]
        head = len(t) - 32
        add([{"id": rid + "-split", "tokens": t[:head], "want": [head - 1] if rid == "a" else [], "_at": 0}])
        for i in range(head, len(t)):
            add([{"id": rid + "-split", "tokens": [t[i]], "want": [0], "_at": i}], end=[rid + "-split"] if i == len(t) - 1 else [])
    # 3. a batch of unequal lengths whose shorter requests end earlier; then a second batch on the freed slots
    for batch, given in ((("a", "b", "d"), {"a": 60, "b": 39, "d": 1}), (("c", "b"), {"c": 70, "b": 10})):
        ids = {r: f"{r}-batch{batch[0]}" for r in batch}
        add([{"id": ids[r], "tokens": reqs[r][:given[r]], "want": [0, given[r] - 1], "_at": 0} for r in batch])
        done = dict(given)
        while any(done[r] < len(reqs[r]) for r in batch):
            live = [r for r in batch if done[r] < len(reqs[r])]
            entries = [{"id": ids[r], "tokens": [reqs[r][done[r]]], "want": [0], "_at": done[r]} for r in live]
            for r in live:
                done[r] += 1
            add(entries, end=[ids[r] for r in live if done[r] == len(reqs[r])])
    out_dir = str(tmp_path / "out")
    # live at once at most: 100 + 40 + 33 tokens -> 128 + 64 + 64
    _replay(folder, dtype, steps, out_dir, max_tokens=256)
    assert sorted(int(f[:-4]) for f in os.listdir(out_dir)) == sorted(expect)
    for no_, want in expect.items():
        assert_close(_read(out_dir, no_, vocab), want, dtype, f"{name} step {no_}")
