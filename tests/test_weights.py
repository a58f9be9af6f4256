"""Weights by tensor name: round trip through a written model folder, and one clear error."""

from __future__ import annotations

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

import tiny_configs
from llmserve_triton_kernels_b200 import models  # noqa: F401
from llmserve_triton_kernels_b200.config import LlamaConfig
from llmserve_triton_kernels_b200.models.load import load_model, random_model
from llmserve_triton_kernels_b200.models.model import Model
from llmserve_triton_kernels_b200.models.llama import llama_plan
from llmserve_triton_kernels_b200.weights import WeightError, check_tensors, read_safetensors, write_random_model


def test_written_folder_has_the_checkpoint_names_and_shapes(model_folder):
    cfg = tiny_configs.TINY_A
    folder = model_folder(cfg, 0, torch.bfloat16)
    assert json.loads((folder / "config.json").read_text())["num_hidden_layers"] == 2
    tensors = load_file(str(folder / "model.safetensors"))
    assert len(tensors) == 2 * 9 + 3  # 9 per layer, token table, final norm, output matrix
    assert tensors["model.layers.1.self_attn.k_proj.weight"].shape == (2 * 16, 64)
    assert tensors["model.layers.0.mlp.down_proj.weight"].shape == (64, 172)
    assert tensors["lm_head.weight"].dtype == torch.bfloat16
    norm = tensors["model.norm.weight"].float()
    assert 0.9 < norm.mean() < 1.1 and norm.std() > 0.005  # 1 + N(0, 0.02): a forgotten norm weight shows
    assert abs(tensors["model.embed_tokens.weight"].float().std() - 0.02) < 0.004


def test_same_seed_same_weights_other_seed_other_weights(tmp_path):
    cfg = LlamaConfig.from_dict(tiny_configs.TINY_B)
    a = load_file(str(write_random_model(tmp_path / "a", cfg, seed=5) / "model.safetensors"))
    b = load_file(str(write_random_model(tmp_path / "b", cfg, seed=5) / "model.safetensors"))
    c = load_file(str(write_random_model(tmp_path / "c", cfg, seed=6) / "model.safetensors"))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert "lm_head.weight" not in a  # tied


def test_stored_precision_is_kept(tmp_path):
    cfg = LlamaConfig.from_dict(tiny_configs.TINY_A)
    folder = write_random_model(tmp_path, cfg, seed=1, dtype=torch.float32)
    tensors = load_file(str(folder / "model.safetensors"))
    tensors["model.norm.weight"] = tensors["model.norm.weight"].to(torch.bfloat16)
    tensors["model.layers.0.mlp.up_proj.weight"] = tensors["model.layers.0.mlp.up_proj.weight"].to(torch.float16)
    save_file(tensors, str(folder / "model.safetensors"))
    read = read_safetensors(folder)
    assert read["model.embed_tokens.weight"].dtype == torch.float32  # stored in 32-bit: stays so
    assert read["model.norm.weight"].dtype == torch.bfloat16
    assert read["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16  # half precision becomes bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = LlamaConfig.from_dict(tiny_configs.TINY_A)
    folder = write_random_model(tmp_path, cfg, seed=1, dtype=torch.float32)
    tensors = load_file(str(folder / "model.safetensors"))
    del tensors["model.layers.1.mlp.gate_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    tensors["model.layers.0.self_attn.v_proj.weight"] = torch.zeros(16, 64)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)  # legacy buffer: skipped silently
    save_file(tensors, str(folder / "model.safetensors"))
    with pytest.raises(WeightError) as err:
        load_model(folder, "float32", "cpu")
    e = err.value
    assert e.missing == ["model.layers.1.mlp.gate_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert e.wrong_shape == [("model.layers.0.self_attn.v_proj.weight", (32, 64), (16, 64))]
    text = str(e)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (1)", "expected [32, 64] got [16, 64]"):
        assert word in text


def test_tied_head_is_one_tensor_and_a_stored_copy_is_ignored(tmp_path):
    cfg = LlamaConfig.from_dict(tiny_configs.TINY_B)
    folder = write_random_model(tmp_path, cfg, seed=2, dtype=torch.float32)
    tensors = load_file(str(folder / "model.safetensors"))
    tensors["lm_head.weight"] = torch.zeros(384, 96)  # the reference overrides such a copy too (weights.py:49-52)
    save_file(tensors, str(folder / "model.safetensors"))
    model, _ = load_model(folder, "float32", "cpu")
    assert model.head.data_ptr() == model.embedding.data_ptr()


def test_no_safetensors_is_an_error(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(tiny_configs.TINY_A))
    with pytest.raises(FileNotFoundError, match="safetensors"):
        load_model(tmp_path, "float32", "cpu")


def test_model_declares_every_tensor_once_and_random_model_matches_the_folder(tmp_path):
    cfg = LlamaConfig.from_dict(tiny_configs.TINY_A)
    specs = Model(llama_plan(cfg), torch.float32, "cpu").tensor_specs()
    folder = write_random_model(tmp_path, cfg, seed=9, dtype=torch.bfloat16)
    stored = load_file(str(folder / "model.safetensors"))
    assert set(specs) == set(stored)
    check_tensors(stored, specs)
    direct = random_model(cfg, 9, "float32", "cpu", storage=torch.bfloat16)
    loaded, _ = load_model(folder, "float32", "cpu")
    assert torch.equal(direct.embedding, loaded.embedding)
    assert torch.equal(direct.blocks[1].mixer.w_in, loaded.blocks[1].mixer.w_in)
    # the stacked projection is [q | k | v] rows
    q = stored["model.layers.1.self_attn.q_proj.weight"].float()
    assert torch.equal(loaded.blocks[1].mixer.w_in[: q.shape[0]], q)
