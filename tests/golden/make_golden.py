"""Compare the plain implementation (tests/plain_llama.py) once with ExiledOfCode/KuiperLLama's
own PyTorch model code (its tools/model.py, imported from a checkout given on the command
line; nothing of it is copied here) on tiny random models, and store that model's logits.

    python tests/golden/make_golden.py /path/to/KuiperLLama

tiny1 runs through tools/model.py as it is.  Its rotary pairing is interleaved
(tools/model.py:64-65), so the q and k rows of our HF-layout weights go through the
project's own ``permute_reverse`` rule (tools/export_llama.py:572-573) first.
tiny2 (grouped heads, tied embeddings) also runs through it, but tools/model.py builds its
rotary table with theta 10000 and has no frequency scaling (tools/model.py:41,227); its
``freqs_cos`` / ``freqs_sin`` buffers are overwritten with our table, so for tiny2 theta and
the llama3 scaling rule rest on the formulas alone, everything else on KuiperLLama's code.

Writes tests/golden/<name>.pt: {"tokens", "logits" (float32 [T, vocab]), "weights" (the model's
tensors as stored, bfloat16, so that the comparison does not depend on which random numbers a
torch build draws), "weights_sha256"}.
"""
import hashlib
import importlib.util
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import helpers          # noqa: E402
import plain_llama      # noqa: E402

SEEDS = {"tiny1": 0, "tiny2": 1}
LENGTHS = {"tiny1": 13, "tiny2": 33}


def weights_digest(w):
    h = hashlib.sha256()
    for name in sorted(w):
        h.update(name.encode())
        h.update(w[name].contiguous().numpy().tobytes())
    return h.hexdigest()


def permute_reverse(w, n_heads, dim1, dim2):
    # HF half-split rows -> interleaved rows, the rule of tools/export_llama.py:572-573
    return w.view(n_heads, 2, dim1 // n_heads // 2, dim2).transpose(1, 2).reshape(dim1, dim2)


def reference_logits(ref, c, w, tokens):
    args = ref.ModelArgs(dim=c["hidden_size"], n_layers=c["num_hidden_layers"], n_heads=c["num_attention_heads"],
                         n_kv_heads=c["num_key_value_heads"], vocab_size=c["vocab_size"],
                         hidden_dim=c["intermediate_size"], norm_eps=c["rms_norm_eps"],
                         max_seq_len=c["max_position_embeddings"])
    m = ref.Transformer(args)
    P = torch.nn.Parameter
    hd = c["head_dim"]
    m.tok_embeddings.weight = P(w["model.embed_tokens.weight"].clone())
    m.output.weight = P((w["model.embed_tokens.weight"] if c["tie_word_embeddings"] else w["lm_head.weight"]).clone())
    m.norm.weight = P(w["model.norm.weight"].clone())
    for i, layer in enumerate(m.layers):
        p = f"model.layers.{i}."
        layer.attention_norm.weight = P(w[p + "input_layernorm.weight"].clone())
        layer.ffn_norm.weight = P(w[p + "post_attention_layernorm.weight"].clone())
        layer.attention.wq.weight = P(permute_reverse(w[p + "self_attn.q_proj.weight"], c["num_attention_heads"],
                                                      c["num_attention_heads"] * hd, c["hidden_size"]).clone())
        layer.attention.wk.weight = P(permute_reverse(w[p + "self_attn.k_proj.weight"], c["num_key_value_heads"],
                                                      c["num_key_value_heads"] * hd, c["hidden_size"]).clone())
        layer.attention.wv.weight = P(w[p + "self_attn.v_proj.weight"].clone())
        layer.attention.wo.weight = P(w[p + "self_attn.o_proj.weight"].clone())
        layer.feed_forward.w1.weight = P(w[p + "mlp.gate_proj.weight"].clone())
        layer.feed_forward.w2.weight = P(w[p + "mlp.down_proj.weight"].clone())
        layer.feed_forward.w3.weight = P(w[p + "mlp.up_proj.weight"].clone())
    if c["rope_theta"] != 10000.0 or c["rope_scaling"] is not None:
        inv = plain_llama.rope_inverse_frequencies(hd, c["rope_theta"], c["rope_scaling"])
        ang = torch.outer(torch.arange(c["max_position_embeddings"]).float(), inv)
        m.freqs_cos = torch.cos(ang)
        m.freqs_sin = torch.sin(ang)
    m.eval()
    t = torch.tensor([tokens], dtype=torch.long)
    with torch.no_grad():
        return m(t, targets=torch.zeros_like(t))[0].float()


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/KuiperLLama")
    ref_root = sys.argv[1]
    spec = importlib.util.spec_from_file_location("kuiper_tools_model", os.path.join(ref_root, "tools", "model.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    for name, seed in SEEDS.items():
        folder = tempfile.mkdtemp()
        helpers.write_folder(folder, name, seed)
        c = plain_llama.read_config(folder)
        w = plain_llama.read_weights(folder)
        tokens = helpers.random_tokens(LENGTHS[name], c["vocab_size"], seed=1000 + seed)
        mine = plain_llama.forward_logits(w, c, tokens)
        theirs = reference_logits(ref, c, w, tokens)
        err = float((mine - theirs).abs().max())
        print(f"{name}: max |plain - KuiperLLama tools/model.py| = {err:.3e} (scale {float(theirs.abs().max()):.3e})")
        assert err < 2e-5 * float(theirs.abs().max()) + 1e-6
        stored = {k: v.to(torch.bfloat16) for k, v in w.items()}
        assert all(torch.equal(stored[k].float(), w[k]) for k in w)        # the folder holds bfloat16: nothing is lost
        torch.save({"tokens": tokens, "logits": theirs, "weights": stored, "weights_sha256": weights_digest(w)},
                   os.path.join(HERE, f"{name}.pt"))


if __name__ == "__main__":
    main()
