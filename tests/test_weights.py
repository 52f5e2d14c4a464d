"""Weights by name, their errors, and the random-weights mode (no GPU)."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from simple_inference_b200.models.load import runtime_for
from simple_inference_b200.weights import (WeightError, load_tensors, model_for_config,
                                           write_random_model)
from tests.conftest import TINY_A, TINY_B


def _specs(cfg):
    _, model = model_for_config(cfg)
    return model, model.tensor_specs(), model.optional_tensor_names()


def test_random_folder_has_config_and_every_tensor(tmp_path):
    write_random_model(tmp_path, TINY_B, seed=5)
    assert json.loads((tmp_path / "config.json").read_text())["num_hidden_layers"] == 3
    stored = load_file(str(tmp_path / "model.safetensors"))
    model, specs, _ = _specs(TINY_B)
    assert set(stored) == set(specs)
    assert "lm_head.weight" in stored               # Tiny B is untied
    assert all(t.dtype == torch.bfloat16 for t in stored.values())
    g = stored["model.layers.0.input_layernorm.weight"].float()
    assert 0.6 < g.mean() < 1.4                     # gains are 1 + N(0, 0.1)
    w = stored["model.layers.1.mlp.down_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.004


def test_same_seed_same_tensors_other_seed_other_tensors(tmp_path):
    a = load_file(str(write_random_model(tmp_path / "a", TINY_A, 1) / "model.safetensors"))
    b = load_file(str(write_random_model(tmp_path / "b", TINY_A, 1) / "model.safetensors"))
    c = load_file(str(write_random_model(tmp_path / "c", TINY_A, 2) / "model.safetensors"))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    assert "lm_head.weight" not in a                # Tiny A is tied


def test_dtypes_kept(tmp_path):
    write_random_model(tmp_path, TINY_A, 1)
    stored = load_file(str(tmp_path / "model.safetensors"))
    stored["model.norm.weight"] = stored["model.norm.weight"].float()   # one gain stored in 32-bit
    save_file(stored, str(tmp_path / "model.safetensors"))
    _, specs, opt = _specs(TINY_A)
    bf = load_tensors(tmp_path, specs, opt, runtime_for("bfloat16", "cpu"))
    assert bf["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert bf["model.layers.0.input_layernorm.weight"].dtype == torch.bfloat16
    assert bf["model.norm.weight"].dtype == torch.float32           # stored 32-bit stays 32-bit
    fp = load_tensors(tmp_path, specs, opt, runtime_for("float32", "cpu"))
    assert all(t.dtype == torch.float32 for t in fp.values())
    assert torch.equal(fp["model.embed_tokens.weight"], bf["model.embed_tokens.weight"].float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    write_random_model(tmp_path, TINY_B, 1)
    stored = load_file(str(tmp_path / "model.safetensors"))
    del stored["model.layers.2.mlp.up_proj.weight"]
    del stored["lm_head.weight"]
    stored["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    stored["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(32, 95, dtype=torch.bfloat16)
    stored["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)
    save_file(stored, str(tmp_path / "model.safetensors"))
    _, specs, opt = _specs(TINY_B)
    with pytest.raises(WeightError) as e:
        load_tensors(tmp_path, specs, opt, runtime_for("bfloat16", "cpu"))
    err = e.value
    assert err.missing == ["lm_head.weight", "model.layers.2.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert len(err.wrong) == 2
    msg = str(err)
    for needle in ("lm_head.weight", "rotary_emb.inv_freq", "(32, 95)", "(32, 96)", "I32"):
        assert needle in msg


def test_tied_checkpoint_may_carry_a_head_but_untied_must(tmp_path):
    write_random_model(tmp_path, TINY_A, 1)
    stored = load_file(str(tmp_path / "model.safetensors"))
    stored["lm_head.weight"] = stored["model.embed_tokens.weight"].clone()
    save_file(stored, str(tmp_path / "model.safetensors"))
    _, specs, opt = _specs(TINY_A)
    load_tensors(tmp_path, specs, opt, runtime_for("bfloat16", "cpu"))  # accepted, ignored


def test_sharded_folder(tmp_path):
    write_random_model(tmp_path, TINY_A, 1)
    stored = load_file(str(tmp_path / "model.safetensors"))
    names = sorted(stored)
    half = len(names) // 2
    save_file({n: stored[n] for n in names[:half]}, str(tmp_path / "s1.safetensors"))
    save_file({n: stored[n] for n in names[half:]}, str(tmp_path / "s2.safetensors"))
    (tmp_path / "model.safetensors").unlink()
    index = {"weight_map": {n: ("s1.safetensors" if i < half else "s2.safetensors")
                            for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    _, specs, opt = _specs(TINY_A)
    got = load_tensors(tmp_path, specs, opt, runtime_for("bfloat16", "cpu"))
    assert all(torch.equal(got[n], stored[n]) for n in names)


def test_missing_files(tmp_path):
    _, specs, opt = _specs(TINY_A)
    with pytest.raises(FileNotFoundError):
        load_tensors(tmp_path, specs, opt, runtime_for("bfloat16", "cpu"))


def test_a_float16_checkpoint_loads_and_is_served_in_bfloat16(tmp_path):
    """torch_dtype "float16" (reference config.py:137-142): tensors are converted as they load."""
    write_random_model(tmp_path, {**TINY_A, "torch_dtype": "float16"}, 1)
    stored = load_file(str(tmp_path / "model.safetensors"))
    assert all(t.dtype == torch.float16 for t in stored.values())
    _, specs, opt = _specs(TINY_A)
    bf = load_tensors(tmp_path, specs, opt, runtime_for("bfloat16", "cpu"))
    assert all(t.dtype == torch.bfloat16 for t in bf.values())
    name = "model.layers.0.mlp.up_proj.weight"
    assert torch.equal(bf[name], stored[name].to(torch.bfloat16))
