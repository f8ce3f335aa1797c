"""Weights: the random writer, the loader's dtype rules and its one error for everything wrong."""

import os
import struct

import pytest
import torch
from safetensors import safe_open
from safetensors.torch import load_file, save_file

from conftest import TINY_A, TINY_B
from qwen3_from_scratch_b200.registry import build_model_spec, config_from_dict
from qwen3_from_scratch_b200.weights import WeightsError, load_weights, model_weight_specs, write_random_model
from qwen3_from_scratch_b200.weights.safetensors_io import SafetensorsFile


def _folder(tmp_path, data=TINY_A, seed=0, **kw):
    folder = str(tmp_path / "m")
    cfg = config_from_dict(data)
    write_random_model(folder, cfg, seed, **kw)
    return folder, model_weight_specs(build_model_spec(cfg))


def test_writer_is_read_by_the_safetensors_package_and_is_seeded(tmp_path):
    folder, specs = _folder(tmp_path)
    other = str(tmp_path / "again")
    write_random_model(other, config_from_dict(TINY_A), 0)
    a, b = load_file(os.path.join(folder, "model.safetensors")), load_file(os.path.join(other, "model.safetensors"))
    assert set(a) == {s.name for s in specs}
    assert all(torch.equal(a[k], b[k]) for k in a)
    third = str(tmp_path / "seed1")
    write_random_model(third, config_from_dict(TINY_A), 1)
    c = load_file(os.path.join(third, "model.safetensors"))
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    emb = a["model.embed_tokens.weight"].float()
    norm = a["model.norm.weight"].float()
    assert a["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert abs(float(emb.std()) - 0.02) < 0.002 and abs(float(emb.mean())) < 0.002
    assert abs(float(norm.mean()) - 1.0) < 0.1
    assert "lm_head.weight" not in a  # tied


def test_a_tensor_does_not_depend_on_the_rest_of_the_model(tmp_path):
    small = dict(TINY_A)
    deeper = dict(TINY_A, num_hidden_layers=3)
    f1, f2 = str(tmp_path / "s"), str(tmp_path / "d")
    write_random_model(f1, config_from_dict(small), 4)
    write_random_model(f2, config_from_dict(deeper), 4)
    a, b = load_file(f1 + "/model.safetensors"), load_file(f2 + "/model.safetensors")
    assert all(torch.equal(a[k], b[k]) for k in a)


def test_dtype_rules(tmp_path):
    folder, specs = _folder(tmp_path, float32_tensors={"model.layers.0.mlp.down_proj.weight": True})
    bf = load_weights(folder, specs, device="cpu", compute_dtype=torch.bfloat16)
    assert bf["model.embed_tokens.weight"].dtype == torch.bfloat16          # bfloat16 stays bfloat16
    assert bf["model.layers.0.mlp.down_proj.weight"].dtype == torch.float32  # stored in 32-bit stays so
    assert bf["model.norm.weight"].dtype == torch.float32                    # norm weights: float32 arithmetic
    f32 = load_weights(folder, specs, device="cpu", compute_dtype=torch.float32)
    assert all(t.dtype == torch.float32 for t in f32.values())
    assert torch.equal(f32["model.embed_tokens.weight"], bf["model.embed_tokens.weight"].float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder, specs = _folder(tmp_path)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32, dtype=torch.bfloat16)
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int64)
    save_file(tensors, path)
    with pytest.raises(WeightsError) as info:
        load_weights(folder, specs, device="cpu", compute_dtype=torch.bfloat16)
    e = info.value
    assert set(e.missing) == {"model.layers.1.mlp.up_proj.weight", "model.norm.weight"}
    assert e.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert e.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (64, 32), (64, 64))]
    assert e.wrong_dtype[0][0] == "model.layers.0.input_layernorm.weight"
    text = str(e)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (1)", "wrong dtype (1)", "[64, 32]", "[64, 64]"):
        assert word in text


def test_tied_checkpoint_may_carry_a_head_copy(tmp_path):
    folder, specs = _folder(tmp_path)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, path)
    with pytest.raises(WeightsError, match="unexpected"):
        load_weights(folder, specs, device="cpu", compute_dtype=torch.bfloat16)
    spec = build_model_spec(config_from_dict(TINY_A))
    out = load_weights(folder, specs, device="cpu", compute_dtype=torch.bfloat16, ignorable=spec.ignorable_weights)
    assert "lm_head.weight" not in out


def test_untied_model_needs_its_head(tmp_path):
    folder, specs = _folder(tmp_path, data=TINY_B, seed=2)
    assert "lm_head.weight" in {s.name for s in specs}
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    del tensors["lm_head.weight"]
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    with pytest.raises(WeightsError, match="lm_head.weight"):
        load_weights(folder, specs, device="cpu", compute_dtype=torch.bfloat16)


def test_truncated_and_absent_files(tmp_path):
    folder, specs = _folder(tmp_path)
    path = os.path.join(folder, "model.safetensors")
    data = open(path, "rb").read()
    open(path, "wb").write(data[: len(data) - 100])
    with pytest.raises(WeightsError, match="truncated"):
        load_weights(folder, specs, device="cpu", compute_dtype=torch.bfloat16)
    os.remove(path)
    with pytest.raises(WeightsError, match="no model.safetensors"):
        load_weights(folder, specs, device="cpu", compute_dtype=torch.bfloat16)


def test_sharded_folder_with_index(tmp_path):
    folder, specs = _folder(tmp_path)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    names = sorted(tensors)
    half = len(names) // 2
    save_file({k: tensors[k] for k in names[:half]}, os.path.join(folder, "model-00001-of-00002.safetensors"))
    save_file({k: tensors[k] for k in names[half:]}, os.path.join(folder, "model-00002-of-00002.safetensors"))
    os.remove(path)
    out = load_weights(folder, specs, device="cpu", compute_dtype=torch.float32)
    assert set(out) == set(names)
    assert torch.equal(out[names[0]], tensors[names[0]].float())


def test_own_reader_agrees_with_the_package(tmp_path):
    folder, _ = _folder(tmp_path, data=TINY_B, seed=2)
    path = os.path.join(folder, "model.safetensors")
    mine = SafetensorsFile(path)
    with safe_open(path, framework="pt") as f:
        for name in f.keys():
            assert torch.equal(mine.get(name), f.get_tensor(name))
    mine.close()
