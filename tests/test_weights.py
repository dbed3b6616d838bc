"""Weight loading errors and the random-weights mode (no GPU: tensors stay on the CPU)."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from helpers import make_model_dir, tiny_config
from tinyserve_b200.parts import build_model
from tinyserve_b200.weights import WeightError, expected_tensors, load_weights, write_random_model


def test_random_folder_is_complete_and_deterministic(tmp_path):
    a = make_model_dir(tmp_path / "a", "B", seed=5)
    b = make_model_dir(tmp_path / "b", "B", seed=5)
    c = make_model_dir(tmp_path / "c", "B", seed=6)
    ta, tb, tc = (load_file(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    assert set(ta) == {e.name for e in expected_tensors(build_model(tiny_config("B")))}
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert any(not torch.equal(ta[k], tc[k]) for k in ta)
    assert ta["model.layers.0.self_attn.q_proj.weight"].shape == (8 * 32, 96)
    assert ta["model.layers.0.self_attn.k_proj.weight"].shape == (2 * 32, 96)
    assert "lm_head.weight" in ta and ta["model.norm.weight"].dtype == torch.bfloat16
    w = ta["model.layers.1.mlp.down_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    n = ta["model.layers.1.input_layernorm.weight"].float()
    # 1 + U(-0.1, 0.1), then rounded to bfloat16 (8 bits of mantissa)
    assert 0.9 - 2 ** -8 <= n.min().item() and n.max().item() <= 1.1 + 2 ** -8
    assert json.load(open(os.path.join(a, "config.json")))["architectures"] == ["Qwen3ForCausalLM"]
    tied = load_file(os.path.join(make_model_dir(tmp_path / "t", "A"), "model.safetensors"))
    assert "lm_head.weight" not in tied


def test_loading_fuses_by_name_and_keeps_dtypes(tmp_path):
    folder = make_model_dir(tmp_path, "B", seed=1, store_dtype="bfloat16", vector_dtype="float32")
    stored = load_file(os.path.join(folder, "model.safetensors"))
    model = build_model(tiny_config("B"))
    load_weights(model, folder, torch.bfloat16, "cpu")
    attn = model.blocks[2].mixer
    p = "model.layers.2.self_attn."
    fused = torch.cat([stored[p + "q_proj.weight"], stored[p + "k_proj.weight"], stored[p + "v_proj.weight"]])
    assert torch.equal(attn.w["qkv_proj.weight"], fused) and fused.dtype == torch.bfloat16
    mlp = model.blocks[0].ffn
    assert torch.equal(mlp.w["gate_up_proj.weight"][160:], stored["model.layers.0.mlp.up_proj.weight"])
    # a width that is a multiple of 64 (configuration A): gate and up rows alternate in blocks of 64
    folder_a = make_model_dir(tmp_path / "a", "A", seed=1)
    stored_a = load_file(os.path.join(folder_a, "model.safetensors"))
    model_a = build_model(tiny_config("A"))
    load_weights(model_a, folder_a, torch.float32, "cpu")
    w = model_a.blocks[1].ffn.w["gate_up_proj.weight"]
    gate, up = stored_a["model.layers.1.mlp.gate_proj.weight"].float(), stored_a["model.layers.1.mlp.up_proj.weight"].float()
    assert gate.shape[0] == 128 and model_a.blocks[1].ffn.block == 64
    assert torch.equal(w, torch.cat([gate[:64], up[:64], gate[64:], up[64:]]))
    # a vector stored in 32-bit stays 32-bit; a matrix takes the engine's dtype
    assert model.norm.w["weight"].dtype == torch.float32
    assert attn.q_norm.w["weight"].dtype == torch.float32
    assert model.embed_tokens.w["weight"].dtype == torch.bfloat16
    model32 = build_model(tiny_config("B"))
    load_weights(model32, folder, torch.float32, "cpu")
    assert model32.lm_head.w["weight"].dtype == torch.float32
    assert torch.equal(model32.lm_head.w["weight"], stored["lm_head.weight"].float())


def test_one_error_lists_everything(tmp_path):
    folder = make_model_dir(tmp_path, "B", seed=1)
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.7.extra.weight"] = torch.zeros(3)
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(32, 96, dtype=torch.bfloat16)
    save_file(t, path)
    with pytest.raises(WeightError) as err:
        load_weights(build_model(tiny_config("B")), folder, torch.bfloat16, "cpu")
    e = err.value
    assert set(e.missing) == {"model.layers.1.mlp.up_proj.weight", "model.norm.weight"}
    assert e.unexpected == ["model.layers.7.extra.weight"]
    assert e.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 96), (64, 96))]
    msg = str(e)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "is [32, 96], expected [64, 96]"):
        assert piece in msg


def test_tied_model_ignores_a_stored_head_and_shards_are_read(tmp_path):
    folder = make_model_dir(tmp_path, "A", seed=2)
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    names = sorted(t)
    os.remove(path)
    save_file({k: t[k] for k in names[::2]}, os.path.join(folder, "model-00001-of-00002.safetensors"))
    rest = {k: t[k] for k in names[1::2]}
    rest["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    save_file(rest, os.path.join(folder, "model-00002-of-00002.safetensors"))
    model = build_model(tiny_config("A"))
    load_weights(model, folder, torch.float32, "cpu")
    assert torch.equal(model.embed_tokens.w["weight"], t["model.embed_tokens.weight"].float())
    with pytest.raises(FileNotFoundError):
        load_weights(model, str(tmp_path / "nowhere_else"), torch.float32, "cpu")
