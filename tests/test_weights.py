"""Safetensors reading and writing, the loader's one error, random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

from helpers import config_dict
from kuiperllama_b200.config import config_from_dict
from kuiperllama_b200.engine import model_manifest, ignorable_tensor_suffixes, write_random_model_folder
from kuiperllama_b200.weights import (SafetensorsFile, SafetensorsFormatError, TensorDecl, WeightsError, load_tensors,
                                      write_safetensors)


def _manifest(name):
    return model_manifest(config_from_dict(config_dict(name)).to_model_spec())


def test_manifest_names_and_shapes():
    m = _manifest("tiny2")
    assert m["model.embed_tokens.weight"].shape == (384, 192)
    assert "lm_head.weight" not in m                               # tied
    assert m["model.layers.2.self_attn.k_proj.weight"].shape == (2 * 32, 192)
    assert m["model.layers.0.mlp.down_proj.weight"].shape == (192, 512)
    assert m["model.norm.weight"].role == "vector" and m["model.norm.weight"].init == "one_plus_normal"
    assert len(m) == 1 + 3 * 9 + 1
    assert _manifest("tiny1")["lm_head.weight"].shape == (256, 64)


def test_writer_agrees_with_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file
    tensors = {"a": torch.randn(3, 5).bfloat16(), "b.c": torch.arange(7, dtype=torch.int32), "d": torch.randn(2, 2, 2)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, tensors.items(), metadata={"k": "v"})
    theirs = load_file(p)
    for k, v in tensors.items():
        assert torch.equal(theirs[k], v)
    q = str(tmp_path / "y.safetensors")
    save_file(tensors, q)
    mine = SafetensorsFile(q)
    assert set(mine.names()) == set(tensors)
    for k, v in tensors.items():
        assert torch.equal(mine.tensor(k), v) and mine.entries[k].shape == tuple(v.shape)


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    cfg = config_from_dict(config_dict("tiny1"))
    write_random_model_folder(str(tmp_path), cfg, seed=3)
    assert json.load(open(tmp_path / "config.json"))["architectures"] == ["LlamaForCausalLM"]
    t = load_tensors(str(tmp_path), _manifest("tiny1"))
    w = t["model.layers.1.mlp.gate_proj.weight"]
    assert w.dtype == torch.bfloat16 and w.shape == (172, 64)
    assert abs(float(w.float().std()) - 0.02) < 0.002 and abs(float(w.float().mean())) < 0.002
    n = t["model.layers.0.input_layernorm.weight"].float()
    assert abs(float(n.mean()) - 1.0) < 0.02
    other = tmp_path / "again"
    write_random_model_folder(str(other), cfg, seed=3)
    assert torch.equal(load_tensors(str(other), _manifest("tiny1"))["lm_head.weight"], t["lm_head.weight"])
    third = tmp_path / "third"
    write_random_model_folder(str(third), cfg, seed=4)
    assert not torch.equal(load_tensors(str(third), _manifest("tiny1"))["lm_head.weight"], t["lm_head.weight"])


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    cfg = config_from_dict(config_dict("tiny1"))
    write_random_model_folder(str(tmp_path), cfg, seed=0)
    sf = SafetensorsFile(str(tmp_path / "model.safetensors"))
    tensors = {n: sf.tensor(n).clone() for n in sf.names()}
    del tensors["model.layers.1.self_attn.v_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary.extra"] = torch.zeros(4)
    tensors["model.layers.0.mlp.up_proj.weight"] = torch.zeros(171, 64, dtype=torch.bfloat16)
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors.items())
    with pytest.raises(WeightsError) as e:
        load_tensors(str(tmp_path), _manifest("tiny1"))
    err = e.value
    assert err.missing == ["model.layers.1.self_attn.v_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary.extra"]
    assert len(err.wrong) == 2 and "[171, 64], expected [172, 64]" in str(err) and "int32" in str(err)
    for name in err.missing + err.unexpected:
        assert name in str(err)


def test_storage_rule_and_ignorable_names(tmp_path):
    spec = config_from_dict(config_dict("tiny2")).to_model_spec()
    m = model_manifest(spec)
    gen = torch.Generator().manual_seed(0)
    tensors = {}
    for i, (n, d) in enumerate(m.items()):
        t = torch.randn(d.shape, generator=gen) * 0.02
        tensors[n] = t if i % 3 == 0 else (t.half() if i % 3 == 1 else t.bfloat16())
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()          # stored beside a tied table
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors.items())
    with pytest.raises(WeightsError):
        load_tensors(str(tmp_path), m)
    got = load_tensors(str(tmp_path), m, ignorable=ignorable_tensor_suffixes(spec))
    for i, n in enumerate(m):
        # 32-bit stays 32-bit; 16-bit floats stay what they are (a float32 run then sees a float16
        # checkpoint's exact values instead of values rounded to bfloat16 first)
        assert got[n].dtype == (torch.float32, torch.float16, torch.bfloat16)[i % 3], n
        assert torch.equal(got[n].float(), tensors[n].float()), n
    ints = {"t": torch.arange(6, dtype=torch.int64).view(2, 3)}
    write_safetensors(str(tmp_path / "model.safetensors"), ints.items())
    assert load_tensors(str(tmp_path), {"t": TensorDecl((2, 3), role="int_table")})["t"].dtype == torch.int32


def test_broken_files(tmp_path):
    with pytest.raises(WeightsError, match="neither model.safetensors"):
        load_tensors(str(tmp_path), {})
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(WeightsError, match="shorter than"):
        load_tensors(str(tmp_path), {})
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsFormatError, match="exceeds the file size"):
        SafetensorsFile(str(p))
    write_safetensors(str(p), [("a", torch.zeros(100))])
    data = p.read_bytes()
    p.write_bytes(data[:-50])                                       # truncated
    with pytest.raises(SafetensorsFormatError, match="truncated"):
        SafetensorsFile(str(p))


def test_sharded_checkpoint_with_index(tmp_path):
    cfg = config_from_dict(config_dict("tiny1"))
    src = tmp_path / "src"
    write_random_model_folder(str(src), cfg, seed=0)
    sf = SafetensorsFile(str(src / "model.safetensors"))
    names = sf.names()
    half = len(names) // 2
    dst = tmp_path / "dst"
    dst.mkdir()
    write_safetensors(str(dst / "model-00001-of-00002.safetensors"), [(n, sf.tensor(n)) for n in names[:half]])
    write_safetensors(str(dst / "model-00002-of-00002.safetensors"), [(n, sf.tensor(n)) for n in names[half:]])
    index = {"weight_map": {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                            for i, n in enumerate(names)}}
    (dst / "model.safetensors.index.json").write_text(json.dumps(index))
    got = load_tensors(str(dst), _manifest("tiny1"))
    assert torch.equal(got[names[-1]], sf.tensor(names[-1]))
