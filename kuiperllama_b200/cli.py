"""The command line, in the manner of ExiledOfCode/KuiperLLama's demo:

    llama_infer <checkpoint> [<tokenizer>] [options]

There the two positional arguments are the exported checkpoint and the tokenizer model, the
prompt "hello" and 128 steps are fixed in the source, a step is one position (prompt
positions included), the text is printed and then ``steps/s`` (demo/main.cpp:50-75).  Here
``<checkpoint>`` is a model folder (config.json + model.safetensors).  ``<tokenizer>`` is
optional: with a sentencepiece model the prompt may be text and the output is decoded
(BOS in front, as kuiper/source/op/encode.cpp:40-42); without it prompts are token ids.
``--steps`` keeps the demo's meaning (positions, prompt included); ``--max-new-tokens``
counts new tokens only.  Without a folder, ``--config FILE --random-weights`` builds a model of
that configuration with random weights.  ``--prompt-file`` brings one prompt a line (token ids,
or text with a tokenizer); ``--print-logits`` prints, for every new token, its logit, its
log-probability and the five largest logits; ``--bench`` runs the generation twice and prints
the second run's prefill and decode rates as one JSON line.
"""
from __future__ import annotations

import argparse
import sys
import time
from typing import List, Optional


def _ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="llama_infer", description="Generate with a Llama 2/3 model folder on a B200.")
    ap.add_argument("checkpoint", nargs="?", default=None, help="model folder with config.json and model.safetensors")
    ap.add_argument("tokenizer", nargs="?", default=None, help="sentencepiece tokenizer.model (optional)")
    ap.add_argument("--prompt", default=None, help='prompt text (needs a tokenizer; the demo\'s default is "hello")')
    ap.add_argument("--prompt-ids", action="append", default=[], help="a prompt as token ids, e.g. 1,15043 (repeatable)")
    ap.add_argument("--prompt-file", default=None, help="a file with one prompt a line: token ids, or text with a tokenizer")
    ap.add_argument("--random-prompts", default=None, metavar="B:LEN", help="B random prompts of LEN tokens")
    ap.add_argument("--steps", type=int, default=128, help="positions to run, prompt included (the demo's total_steps)")
    ap.add_argument("--max-new-tokens", type=int, default=None, help="new tokens per prompt (overrides --steps)")
    ap.add_argument("--temperature", type=float, default=0.0, help="0: argmax, as the demo's sampler")
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--seed", type=int, default=0, help="seed of the sampler and of random prompts and weights")
    ap.add_argument("--stop-ids", default=None, help="stop token ids (default: eos_token_id of config.json)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--random-weights", action="store_true", help="ignore model.safetensors; random weights from --seed")
    ap.add_argument("--config", default=None, metavar="FILE", help="a config.json for --random-weights without a model folder")
    ap.add_argument("--print-logits", action="store_true", help="print each new token's logit, log-probability and the top five")
    ap.add_argument("--bench", action="store_true", help="run twice; print the second run's rates as one JSON line")
    ap.add_argument("--max-batch", type=int, default=64)
    ap.add_argument("--max-ctx", type=int, default=None, help="longest sequence the cache holds")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--stream-fusion", action="store_true",
                    help="decode steps of up to 4 sequences fold the residual add and the norms into the products")
    args = ap.parse_args(argv)
    if args.checkpoint is None and not (args.config and args.random_weights):
        ap.error("give a model folder, or --config FILE --random-weights")
    if args.config and not args.random_weights:
        ap.error("--config is for --random-weights; a model folder brings its own config.json")

    import json
    import torch
    from . import load

    tok = None
    if args.tokenizer:
        import sentencepiece
        tok = sentencepiece.SentencePieceProcessor(model_file=args.tokenizer)
    m = load(args.checkpoint, dtype=args.dtype, device=args.device, random_weights=args.random_weights, seed=args.seed,
             config=args.config, max_batch=args.max_batch, max_seq_len=args.max_ctx, stream_fusion=args.stream_fusion)
    prompts: List[List[int]] = [_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            for line in f:
                line = line.strip()
                if not line:
                    continue
                if all(c.isdigit() or c in ", \t" for c in line):
                    prompts.append(_ids(line))
                elif tok is not None:
                    prompts.append([tok.bos_id()] + tok.encode(line))
                else:
                    ap.error(f"--prompt-file: a line of text needs a tokenizer: {line[:40]!r}")
    if args.random_prompts:
        b, n = (int(x) for x in args.random_prompts.split(":"))
        g = torch.Generator().manual_seed(args.seed)
        prompts += torch.randint(0, m.model.spec.vocab_size, (b, n), generator=g).tolist()
    if args.prompt is not None or not prompts:
        if tok is None:
            ap.error("a text prompt needs a tokenizer; give --prompt-ids or --random-prompts instead")
        prompts.append([tok.bos_id()] + tok.encode(args.prompt if args.prompt is not None else "hello"))
    stop = _ids(args.stop_ids) if args.stop_ids is not None else None
    if tok is not None and stop is None:
        stop = list(m.stop_token_ids) or [tok.eos_id()]
    max_new = args.max_new_tokens
    if max_new is None:
        max_new = max(0, args.steps - min(len(p) for p in prompts) + 1)
    print("Generating...", flush=True)
    for _ in range(2 if args.bench else 1):                      # --bench: the first run warms up and captures the graphs
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = m.generate(prompts, max_new_tokens=max_new, temperature=args.temperature, top_k=args.top_k, seed=args.seed,
                         stop_ids=stop, return_logprobs=args.print_logits, return_logits=args.print_logits)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    for i, (p, o) in enumerate(zip(prompts, out)):
        print(tok.decode(o) if tok is not None else " ".join(str(t) for t in o), flush=True)
        if args.print_logits:
            res = m.last_results[i]
            for t, lp, row in zip(res.tokens, res.logprobs, res.logits):
                top = torch.topk(row, min(5, row.numel()))
                best = " ".join(f"{int(j)}:{float(v):.4f}" for v, j in zip(top.values, top.indices))
                print(f"  token {t} logit {float(row[t]):.4f} logprob {lp:.4f} | top: {best}")
    st = m.last_stats
    positions = sum(len(p) - 1 for p in prompts) + sum(len(o) for o in out)
    if args.bench:
        print(json.dumps({"prompts": len(prompts), "prefill_tokens": st.prefill_tokens,
                          "prefill_tokens_per_s": round(st.prefill_tokens / max(st.prefill_seconds, 1e-9), 1),
                          "decode_tokens": st.decode_tokens, "decode_steps": st.decode_steps,
                          "decode_tokens_per_s": round(st.decode_tokens / max(st.decode_seconds, 1e-9), 1),
                          "seconds": round(dt, 4), "dtype": args.dtype}))
    print(f"\nsteps/s:{positions / dt:f}")
    print(f"prefill: {st.prefill_tokens} tokens in {st.prefill_seconds:.4f} s; decode: {st.decode_tokens} tokens in "
          f"{st.decode_seconds:.4f} s ({st.decode_tokens / max(st.decode_seconds, 1e-9):.1f} tok/s)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
