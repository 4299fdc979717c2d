"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the same
``load_model``, ``Engine.step`` and ``SequenceCache`` that generation uses.  ExiledOfCode/
KuiperLLama has nothing like it (its only model-level check, test/test_model/
test_llama_cpu.cpp:14-30, is disabled).

Steps arrive on standard input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` brings each request's next tokens and the places among them whose logits are
wanted; ``end`` names requests that are finished after the step, whose slots and pages are
handed back.  For a step that wants something, ``<out>/<step>.f32`` receives the logits as
little-endian float32 [wanted, vocab] in the order of the entries and of ``want``.  After every
step the line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, List

import torch


def main(argv: List[str] = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    from .cache import PAGE
    from .engine import Engine, SequenceInput, load_model

    os.makedirs(args.out, exist_ok=True)
    with torch.inference_mode():
        model = load_model(args.model, dtype=args.dtype, device=args.device)
        max_tokens = max(PAGE, (args.max_tokens + PAGE - 1) // PAGE * PAGE)
        cache = model.new_cache(max_tokens=max_tokens)
        engine = Engine(model, cache)
        slots: Dict[str, int] = {}
        for line in sys.stdin:
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            step_no = rec["step"]
            inputs = []
            for e in rec.get("entries", []):
                rid = str(e["id"])
                if rid not in slots:
                    slots[rid] = engine.alloc_slot()
                inputs.append(SequenceInput(slots[rid], e["tokens"], e.get("want", [])))
            if inputs:
                logits = engine.step(inputs)
                if logits is not None:
                    data = logits.to("cpu", torch.float32).contiguous().numpy()
                    tmp = os.path.join(args.out, f".{step_no}.f32.tmp")
                    data.astype("<f4").tofile(tmp)
                    os.replace(tmp, os.path.join(args.out, f"{step_no}.f32"))
                else:
                    torch.cuda.synchronize()
            for rid in rec.get("end", []):
                rid = str(rid)
                if rid in slots:
                    engine.free_slot(slots.pop(rid))
            engine.check_device_errors()
            print(f"done {step_no}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
