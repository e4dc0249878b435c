"""Safetensors reading/writing and the one error that lists what does not fit (no GPU)."""
import json
import os

import pytest
import torch

import replay_util as ru
from dispec_b200.config import load_model_config
from dispec_b200.weights import (CheckpointFolder, SafetensorsError, WeightError, build_model,
                                 random_tensors, write_random_model, write_safetensors)
from dispec_b200.weights.loader import check_source


def test_written_folder_is_read_by_the_safetensors_library_and_back(tmp_path):
    from safetensors.torch import load_file, save_file
    cfg = load_model_config(ru.CONFIG_B)
    write_random_model(cfg, str(tmp_path), seed=1, std=0.05, dtype="bfloat16")
    theirs = load_file(str(tmp_path / "model.safetensors"))
    mine = CheckpointFolder(str(tmp_path))
    assert set(theirs) == set(mine.names())
    for name, t in theirs.items():
        assert t.dtype == torch.bfloat16 and torch.equal(t, mine.get(name))
    # a file written by the library is read by this package
    save_file({"x": torch.arange(6, dtype=torch.int32).reshape(2, 3), "y": torch.ones(3)},
              str(tmp_path / "other.safetensors"))
    from dispec_b200.weights import SafetensorsFile
    f = SafetensorsFile(str(tmp_path / "other.safetensors"))
    assert f.get("x").tolist() == [[0, 1, 2], [3, 4, 5]] and f.dtype("y") == torch.float32
    assert json.load(open(tmp_path / "config.json"))["architectures"] == ["Qwen2ForCausalLM"]


def test_random_weights_follow_the_rule_and_the_seed():
    cfg = load_model_config(ru.CONFIG_A)
    a = random_tensors(cfg, 0, 0.02, "float32")
    b = random_tensors(cfg, 0, 0.02, "float32")
    c = random_tensors(cfg, 1, 0.02, "float32")
    assert all(torch.equal(a[k], b[k]) for k in a) and not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    assert abs(a["model.norm.weight"].mean().item() - 1.0) < 0.02
    assert abs(a["model.embed_tokens.weight"].std().item() - 0.02) < 0.002
    assert abs(a["model.layers.0.self_attn.q_proj.bias"].mean().item()) < 0.02


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = load_model_config(ru.CONFIG_B)
    tensors = random_tensors(cfg, 1, 0.05, "bfloat16")
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(32, 95, dtype=torch.bfloat16)
    tensors["model.layers.7.extra.weight"] = torch.zeros(3)
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(96, dtype=torch.int32)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    model = build_model(cfg)
    with pytest.raises(WeightError) as e:
        check_source(model, CheckpointFolder(str(tmp_path)), "folder")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 95), (32, 96))]
    assert err.wrong_type[0][0] == "model.layers.0.self_attn.q_proj.bias"
    text = str(err)
    for piece in ("missing (2)", "unexpected (1)", "model.layers.7.extra.weight", "(32, 95)", "(32, 96)"):
        assert piece in text


def test_tied_model_tolerates_a_stored_head_and_untied_needs_it(tmp_path):
    cfg = load_model_config(ru.CONFIG_A)
    tensors = random_tensors(cfg, 0, 0.02, "bfloat16")
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    check_source(build_model(cfg), CheckpointFolder(str(tmp_path)), "folder")
    cfg_b = load_model_config(ru.CONFIG_B)
    tb = random_tensors(cfg_b, 1, 0.05, "bfloat16")
    del tb["lm_head.weight"]
    os.makedirs(tmp_path / "b")
    write_safetensors(str(tmp_path / "b" / "model.safetensors"), tb)
    with pytest.raises(WeightError, match="lm_head.weight"):
        check_source(build_model(cfg_b), CheckpointFolder(str(tmp_path / "b")), "folder")


def test_truncated_and_sharded_files(tmp_path):
    cfg = load_model_config(ru.CONFIG_A)
    tensors = random_tensors(cfg, 0, 0.02, "bfloat16")
    path = tmp_path / "model.safetensors"
    write_safetensors(str(path), tensors)
    data = path.read_bytes()
    (tmp_path / "cut").mkdir()
    (tmp_path / "cut" / "model.safetensors").write_bytes(data[:len(data) // 2])
    with pytest.raises(SafetensorsError, match="truncated"):
        CheckpointFolder(str(tmp_path / "cut"))
    with pytest.raises(SafetensorsError, match="neither"):
        CheckpointFolder(str(tmp_path / "nothing_here"))
    # two shards with an index
    names = list(tensors)
    (tmp_path / "sh").mkdir()
    half = len(names) // 2
    write_safetensors(str(tmp_path / "sh" / "model-00001-of-00002.safetensors"), {n: tensors[n] for n in names[:half]})
    write_safetensors(str(tmp_path / "sh" / "model-00002-of-00002.safetensors"), {n: tensors[n] for n in names[half:]})
    index = {"weight_map": {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                            for i, n in enumerate(names)}}
    (tmp_path / "sh" / "model.safetensors.index.json").write_text(json.dumps(index))
    folder = CheckpointFolder(str(tmp_path / "sh"))
    check_source(build_model(cfg), folder, "shards")
    assert torch.equal(folder.get(names[-1]), tensors[names[-1]])
