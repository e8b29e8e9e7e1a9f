"""Weights: safetensors by name, fusing, dtype policy, one clear error, random mode."""

import json
import os

import pytest
import torch

import tiny
from freetoken_b200.models import Model
from freetoken_b200.registry import architecture_of
from freetoken_b200.weights import (Checkpoint, Name, TensorSpec, WeightError, device_dtype,
                                    load_tensors, plan_loading, write_model_folder, write_safetensors)
from plain_model import read_safetensors


def specs_of(config):
    arch = architecture_of(config)
    return arch, Model(arch.build_plan(arch.read_config(config))).tensor_specs()


def test_safetensors_round_trip_agrees_with_an_independent_reader(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b.c": torch.randn(7).to(torch.bfloat16),
               "ids": torch.arange(6, dtype=torch.int32).view(2, 3), "scalar": torch.tensor(2.5)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors)
    back = read_safetensors(path)                        # the plain implementation's reader
    with Checkpoint(str(tmp_path)) as ck:
        for name, t in tensors.items():
            assert torch.equal(back[name], t) and torch.equal(ck.read(name), t)
            assert ck.entries[name].shape == tuple(t.shape)
    try:
        from safetensors.torch import load_file
    except ImportError:
        return
    lib = load_file(path)
    for name, t in tensors.items():
        assert torch.equal(lib[name], t)


def test_random_folder_loads_fused_and_keeps_dtypes(tmp_path):
    folder = tiny.write_tiny(str(tmp_path), "A")
    arch, specs = specs_of(tiny.TINY_A)
    raw = read_safetensors(os.path.join(folder, "model.safetensors"))
    assert "model.layers.0.self_attn.q_proj.weight" in raw and "model.layers.1.block_sparse_moe.experts.3.w2.weight" in raw
    assert raw["model.layers.0.block_sparse_moe.gate.weight"].dtype == torch.float32   # stored in 32 bits
    for compute in (torch.float32, torch.bfloat16):
        t = load_tensors(specs, folder, compute, "cpu", arch.rename_tensor)
        qkv = t["model.layers.0.self_attn.qkv_proj.weight"]
        assert qkv.dtype == torch.bfloat16 and qkv.shape == (64 + 32 + 32, 64)     # bf16 stays bf16 in both modes
        assert torch.equal(qkv[:64], raw["model.layers.0.self_attn.q_proj.weight"])
        assert torch.equal(qkv[96:], raw["model.layers.0.self_attn.v_proj.weight"])
        gu = t["model.layers.1.block_sparse_moe.experts.gate_up_proj"]
        assert gu.shape == (4, 64, 64)
        assert torch.equal(gu[2, :32], raw["model.layers.1.block_sparse_moe.experts.2.w1.weight"])
        assert torch.equal(gu[2, 32:], raw["model.layers.1.block_sparse_moe.experts.2.w3.weight"])
        assert t["model.layers.0.block_sparse_moe.gate.weight"].dtype == torch.float32
        assert t["model.layers.0.input_layernorm.weight"].dtype == torch.float32     # small tensors: float32


def test_float32_files_stay_float32_only_in_float32_mode(tmp_path):
    folder = tiny.write_tiny(str(tmp_path), "B", file_dtype=torch.float32)
    arch, specs = specs_of(tiny.TINY_B)
    f32 = load_tensors(specs, folder, torch.float32, "cpu", arch.rename_tensor)
    b16 = load_tensors(specs, folder, torch.bfloat16, "cpu", arch.rename_tensor)
    name = "model.layers.2.self_attn.o_proj.weight"
    assert f32[name].dtype == torch.float32 and b16[name].dtype == torch.bfloat16
    assert torch.equal(b16[name], f32[name].to(torch.bfloat16))
    assert "lm_head.weight" not in f32                                   # tied head has no tensor
    # a tied checkpoint that still carries lm_head.weight is accepted, the tensor dropped
    raw = read_safetensors(os.path.join(folder, "model.safetensors"))
    raw["lm_head.weight"] = raw["model.embed_tokens.weight"].clone()
    os.makedirs(tmp_path / "with_head")
    write_safetensors(str(tmp_path / "with_head" / "model.safetensors"), raw)
    again = load_tensors(specs, str(tmp_path / "with_head"), torch.float32, "cpu", arch.rename_tensor)
    assert torch.equal(again["model.embed_tokens.weight"], f32["model.embed_tokens.weight"])
    assert device_dtype("int32", torch.int64, torch.bfloat16) == torch.int32


def test_fused_names_and_language_model_prefix_are_accepted(tmp_path):
    arch, specs = specs_of(tiny.TINY_A)
    fused = str(tmp_path / "fused")
    write_model_folder(fused, tiny.TINY_A, specs, 0, torch.bfloat16, tiny.random_options("A"), fused_names=True)
    split = tiny.write_tiny(str(tmp_path / "split"), "A")
    a = load_tensors(specs, fused, torch.float32, "cpu", arch.rename_tensor)
    b = load_tensors(specs, split, torch.float32, "cpu", arch.rename_tensor)
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    prefixed = {f"language_model.{k}": v for k, v in read_safetensors(os.path.join(split, "model.safetensors")).items()}
    prefixed["vision_tower.patch_embed.weight"] = torch.zeros(2, 2)
    os.makedirs(tmp_path / "vl")
    write_safetensors(str(tmp_path / "vl" / "model.safetensors"), prefixed)
    c = load_tensors(specs, str(tmp_path / "vl"), torch.float32, "cpu", arch.rename_tensor)
    assert all(torch.equal(c[k], b[k]) for k in b)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = tiny.write_tiny(str(tmp_path / "ok"), "A")
    arch, specs = specs_of(tiny.TINY_A)
    raw = read_safetensors(os.path.join(folder, "model.safetensors"))
    del raw["model.layers.0.self_attn.k_proj.weight"]                        # incomplete q/k/v group
    del raw["model.norm.weight"]
    raw["model.layers.0.mlp.gate_proj.weight"] = torch.zeros(2, 2)           # nobody asked for it
    raw["model.layers.1.self_attn.o_proj.weight"] = torch.zeros(64, 60).to(torch.bfloat16)
    raw["lm_head.weight"] = torch.zeros(250, 64).to(torch.bfloat16)
    bad = tmp_path / "bad"
    os.makedirs(bad)
    write_safetensors(str(bad / "model.safetensors"), raw)
    with pytest.raises(WeightError) as err:
        load_tensors(specs, str(bad), torch.float32, "cpu", arch.rename_tensor)
    e = err.value
    assert e.missing == ["model.layers.0.self_attn.k_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.mlp.gate_proj.weight"]
    assert sorted(n for n, _, _ in e.wrong_shape) == ["lm_head.weight", "model.layers.1.self_attn.o_proj.weight"]
    text = str(e)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (2)",
                   "expected [64, 64], found [64, 60]"):
        assert needle in text


def test_plan_loading_prefers_complete_sources():
    spec = TensorSpec("w", (4, 2), sources=(Name("alt", (4, 2)),))
    assert plan_loading([spec], {"w": (4, 2)})["w"].name == "w"
    assert plan_loading([spec], {"alt": (4, 2)})["w"].name == "alt"
    with pytest.raises(WeightError):
        plan_loading([spec], {})
    optional = TensorSpec("o", (1,), optional=True)
    assert plan_loading([optional], {}) == {}


def test_random_mode_is_seeded_per_tensor(tmp_path):
    arch, specs = specs_of(tiny.TINY_B)
    one = str(tmp_path / "one")
    two = str(tmp_path / "two")
    write_model_folder(one, tiny.TINY_B, specs, 7, torch.bfloat16)
    write_model_folder(two, tiny.TINY_B, list(reversed(specs)), 7, torch.bfloat16)   # other creation order
    a = read_safetensors(os.path.join(one, "model.safetensors"))
    b = read_safetensors(os.path.join(two, "model.safetensors"))
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    other = str(tmp_path / "other")
    write_model_folder(other, tiny.TINY_B, specs, 8, torch.bfloat16)
    c = read_safetensors(os.path.join(other, "model.safetensors"))
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    w = a["model.layers.0.self_attn.q_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.003                                 # matrices ~N(0, 0.02^2)
    assert json.load(open(os.path.join(one, "config.json")))["hidden_size"] == 96
    # gemma-form norm weights are stored as (scale - 1): mean 0; plain form: mean 1
    assert float(a["model.norm.weight"].float().abs().max()) == 0.0
    _, specs_a = specs_of(tiny.TINY_A)
    write_model_folder(str(tmp_path / "A"), tiny.TINY_A, specs_a, 0, torch.bfloat16, tiny.random_options("A"))
    na = read_safetensors(str(tmp_path / "A" / "model.safetensors"))
    assert torch.all(na["model.norm.weight"].float() == 1.0)
    assert float(na["model.layers.0.block_sparse_moe.e_score_correction_bias"].std()) > 0


def test_a_score_correction_bias_in_the_checkpoint_is_used_even_if_the_config_is_silent(tmp_path):
    """The reference's block always adds ``e_score_correction_bias`` when it chooses
    experts (python/freetoken/models/minimax_m3/moe.py:75) and its loader always
    reads it (weight.py:220): a config.json without ``use_routing_bias`` must not
    make routing ignore a bias the checkpoint carries."""
    with_bias = dict(tiny.TINY_B, use_routing_bias=True)
    folder = tiny.write_tiny(str(tmp_path), "B", config=with_bias)
    silent = {k: v for k, v in tiny.TINY_B.items() if k != "use_routing_bias"}
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(silent, f)
    arch = architecture_of(silent)
    model = Model(arch.build_plan(arch.read_config(silent)))
    tensors = load_tensors(model.tensor_specs(), folder, torch.float32, "cpu", arch.rename_tensor)
    name = "model.layers.1.block_sparse_moe.e_score_correction_bias"
    assert name in tensors and tensors[name].dtype == torch.float32
    model.bind(tensors, torch.float32)
    for block in model.blocks:
        assert block.feed_forward.w_bias is not None
    # absent and not asked for: fine, and no bias is used
    folder2 = tiny.write_tiny(str(tmp_path / "plain"), "B")
    tensors = load_tensors(model.tensor_specs(), folder2, torch.float32, "cpu", arch.rename_tensor)
    model.bind(tensors, torch.float32)
    assert all(block.feed_forward.w_bias is None for block in model.blocks)
    # asked for and absent: one error that names it
    model = Model(arch.build_plan(arch.read_config(with_bias)))
    with pytest.raises(WeightError) as err:
        load_tensors(model.tensor_specs(), folder2, torch.float32, "cpu", arch.rename_tensor)
    assert name in err.value.missing
