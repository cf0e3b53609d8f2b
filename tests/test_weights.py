"""Weights by tensor name: storage dtypes, the one error that lists everything wrong with a
folder, sharded folders, and the random-weights mode."""
import json
import os

import pytest
import torch

import tiny
from rllm_b200.config import config_from_dict
from rllm_b200.weights import (TensorStore, WeightError, WeightFileError, load_weights,
                               random_tensors, write_random_model, write_safetensors)


def build(cfg):
    arch, c = config_from_dict(cfg)
    return arch.build(c)


def test_random_mode_writes_a_folder_the_loader_reads(tmp_path):
    d = write_random_model(tiny.TINY_B, 1, str(tmp_path / "m"), std=0.05, norm_std=0.1)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    model = build(json.load(open(os.path.join(d, "config.json"))))
    load_weights(model, d, torch.bfloat16, "cpu")
    blk = model.blocks[2]
    assert blk.mixer.w_qkv.shape == (96 + 2 * 32, 96) and blk.mixer.w_qkv.dtype == torch.bfloat16
    assert blk.ffn.w_gate_up.shape == (448, 96) and blk.ffn.w_down.shape == (96, 224)
    assert model.head.weight.shape == (384, 96) and model.embedding.table.shape == (384, 96)
    store = TensorStore(d)
    q = store.read("model.layers.2.self_attn.q_proj.weight")
    v = store.read("model.layers.2.self_attn.v_proj.weight")
    assert torch.equal(blk.mixer.w_qkv[:96], q) and torch.equal(blk.mixer.w_qkv[128:], v)
    assert torch.equal(blk.ffn.w_gate_up[224:], store.read("model.layers.2.mlp.up_proj.weight"))
    assert blk.mixer.position.inv_freq.dtype == torch.float32 and blk.mixer.position.inv_freq.numel() == 16


def test_same_seed_same_weights_other_seed_other_weights():
    a, b, c = (random_tensors(build(tiny.TINY_A), s) for s in (0, 0, 1))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert any(not torch.equal(a[k], c[k]) for k in a)
    assert float(a["model.norm.weight"].float().min()) == 1.0


def test_storage_rule(tmp_path):
    """Matrices take the run dtype; a vector stored in 32-bit stays 32-bit in the bfloat16
    run; everything is float32 in the 32-bit run."""
    model = build(tiny.TINY_A)
    t = random_tensors(model, 0, dtype=torch.bfloat16)
    t["model.norm.weight"] = t["model.norm.weight"].float() * 1.00001      # stored as F32
    d = tmp_path / "m"; d.mkdir()
    (d / "config.json").write_text(json.dumps(tiny.TINY_A))
    write_safetensors(str(d / "model.safetensors"), t)
    load_weights(model, str(d), torch.bfloat16, "cpu")
    assert model.head.norm.weight.dtype == torch.float32
    assert model.blocks[0].mixer_norm.weight.dtype == torch.bfloat16
    assert model.embedding.table.dtype == torch.bfloat16
    load_weights(model, str(d), torch.float32, "cpu")
    assert {p.dtype for part in model.parts() for p in
            [getattr(part, q.attr) for q in part.params()]} == {torch.float32}
    assert torch.equal(model.embedding.table, t["model.embed_tokens.weight"].float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    model = build(tiny.TINY_A)
    t = random_tensors(model, 0)
    del t["model.layers.1.mlp.up_proj.weight"], t["model.norm.weight"]
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    t["model.layers.0.self_attn.qkv_proj.weight"] = torch.zeros(4, 4, dtype=torch.bfloat16)
    t["model.layers.1.mlp.gate_up_proj.weight"] = torch.zeros(4, 4, dtype=torch.bfloat16)
    t["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)       # tied model: a redundant copy, passed over
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)     # harmless leftover
    t["model.layers.0.input_layernorm.weight"] = torch.ones(64, dtype=torch.int32)
    d = tmp_path / "m"; d.mkdir()
    write_safetensors(str(d / "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        load_weights(model, str(d), torch.bfloat16, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.qkv_proj.weight", "model.layers.1.mlp.gate_up_proj.weight"]
    assert [(n, tuple(exp), tuple(got)) for n, exp, got in err.wrong_shape] == \
        [("model.layers.0.self_attn.k_proj.weight", (32, 64), (16, 64))]
    assert err.wrong_dtype == [("model.layers.0.input_layernorm.weight", "I32")]
    for word in ("missing", "unexpected", "wrong shape", "expected [32, 64] got [16, 64]"):
        assert word in str(err)


def test_sharded_folder_and_absent_shard(tmp_path):
    model = build(tiny.TINY_A)
    t = random_tensors(model, 0)
    names = sorted(t)
    halves = {"a.safetensors": names[: len(names) // 2], "b.safetensors": names[len(names) // 2:]}
    d = tmp_path / "m"; d.mkdir()
    for f, ns in halves.items():
        write_safetensors(str(d / f), {n: t[n] for n in ns})
    (d / "model.safetensors.index.json").write_text(
        json.dumps({"weight_map": {n: f for f, ns in halves.items() for n in ns}}))
    load_weights(model, str(d), torch.bfloat16, "cpu")
    assert torch.equal(model.embedding.table, t["model.embed_tokens.weight"])
    os.remove(d / "b.safetensors")
    with pytest.raises(WeightFileError) as e:
        load_weights(model, str(d), torch.bfloat16, "cpu")
    assert "b.safetensors" in str(e.value)
    with pytest.raises(WeightFileError):
        TensorStore(str(tmp_path))


def test_truncated_file_is_refused(tmp_path):
    d = write_random_model(tiny.TINY_A, 0, str(tmp_path / "m"))
    p = os.path.join(d, "model.safetensors")
    blob = open(p, "rb").read()
    open(p, "wb").write(blob[: len(blob) // 2])
    with pytest.raises(WeightFileError):
        TensorStore(d)
