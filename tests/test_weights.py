"""Weights: the random-weights folder, reading by name, the one error that lists every
fault, and the storage rule."""

from __future__ import annotations

import pytest
import torch
from safetensors.torch import load_file, save_file

from mercury_b200.config import config_from_dict
from mercury_b200.models import Model
from mercury_b200.parts import PartSetup
from mercury_b200.weights import WeightError, read_checkpoint, write_random_model
from tiny import TINY_A, TINY_B


def specs_of(raw):
    entry, cfg = config_from_dict(raw)
    model = Model(entry.describe(cfg))
    return cfg, model


def test_random_folder_round_trip(tmp_path):
    cfg, model = specs_of(TINY_B)
    folder = write_random_model(tmp_path / "m", cfg, seed=1)
    assert (folder / "config.json").exists() and (folder / "model.safetensors").exists()
    tensors = read_checkpoint(folder, model.tensor_specs(), model.optional_tensors())
    names = {s.name for s in model.tensor_specs()}
    assert set(tensors) == names
    assert "lm_head.weight" in names                      # B is untied
    assert tensors["model.layers.2.self_attn.k_proj.bias"].shape == (32,)
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    norm = tensors["model.layers.0.input_layernorm.weight"].float()
    assert abs(float(norm.mean()) - 1.0) < 0.05            # 1 + N(0, 0.05)
    assert abs(float(tensors["model.embed_tokens.weight"].float().std()) - 0.02) < 0.002


def test_same_seed_same_values_other_seed_other_values(tmp_path):
    cfg, _model = specs_of(TINY_A)
    a = load_file(str(write_random_model(tmp_path / "a", cfg, 0) / "model.safetensors"))
    b = load_file(str(write_random_model(tmp_path / "b", cfg, 0) / "model.safetensors"))
    c = load_file(str(write_random_model(tmp_path / "c", cfg, 1) / "model.safetensors"))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    assert "lm_head.weight" not in a                       # A is tied


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg, model = specs_of(TINY_A)
    folder = write_random_model(tmp_path / "m", cfg, 0)
    tensors = load_file(str(folder / "model.safetensors"))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.extra.weight"] = torch.zeros(3)
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(65, dtype=torch.bfloat16)
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError) as info:
        read_checkpoint(folder, model.tensor_specs(), model.optional_tensors())
    err = info.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.bias", (65,), (64,))]
    text = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape", "(65,)", "(64,)"):
        assert word in text


def test_a_tied_model_tolerates_a_copy_of_the_head(tmp_path):
    cfg, model = specs_of(TINY_A)
    folder = write_random_model(tmp_path / "m", cfg, 0)
    tensors = load_file(str(folder / "model.safetensors"))
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, str(folder / "model.safetensors"))
    read_checkpoint(folder, model.tensor_specs(), model.optional_tensors())


def test_no_weights_at_all(tmp_path):
    _cfg, model = specs_of(TINY_A)
    with pytest.raises(FileNotFoundError):
        read_checkpoint(tmp_path, model.tensor_specs())


def test_storage_rule():
    bf = PartSetup(torch.device("cpu"), torch.bfloat16, None, 16)
    fp = PartSetup(torch.device("cpu"), torch.float32, None, 16)
    assert bf.place(torch.zeros(2, dtype=torch.bfloat16)).dtype == torch.bfloat16
    assert bf.place(torch.zeros(2, dtype=torch.float16)).dtype == torch.bfloat16
    assert bf.place(torch.zeros(2, dtype=torch.float32)).dtype == torch.float32   # stays 32-bit
    assert bf.place(torch.zeros(2, dtype=torch.int64)).dtype == torch.int32
    assert fp.place(torch.zeros(2, dtype=torch.bfloat16)).dtype == torch.float32
    assert fp.place(torch.zeros(2, dtype=torch.int16)).dtype == torch.int32
