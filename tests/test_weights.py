import json

import pytest
import torch
from safetensors import safe_open
from safetensors.torch import save_file

from conftest import tiny_configs
from slipstream_b200.parts.base import Runtime
from slipstream_b200.registry import load_config
from slipstream_b200.weights.loader import WeightError, load_weights, safetensor_files
from slipstream_b200.weights.random_init import write_random_model

CPU = Runtime(torch.device("cpu"), torch.bfloat16)


def _folder(tmp_path, name="A", **kw):
    config, _ = tiny_configs()[name]
    write_random_model(config, tmp_path, seed=3, **kw)
    return config


def _specs(folder):
    arch, cfg = load_config(folder)
    return arch.build(cfg).weight_specs()


def _rewrite(tmp_path, edit):
    path = tmp_path / "model.safetensors"
    with safe_open(str(path), framework="pt") as h:
        tensors = {k: h.get_tensor(k) for k in h.keys()}
    edit(tensors)
    save_file(tensors, str(path))


def test_random_folder_is_seeded_and_complete(tmp_path):
    config = _folder(tmp_path / "a")
    _folder(tmp_path / "b")
    wa = load_weights(tmp_path / "a", _specs(tmp_path / "a"), CPU)
    wb = load_weights(tmp_path / "b", _specs(tmp_path / "b"), CPU)
    assert set(wa) == set(wb) and all(torch.equal(wa[k], wb[k]) for k in wa)
    assert json.loads((tmp_path / "a" / "config.json").read_text())["architectures"] == ["Qwen2ForCausalLM"]
    # tied: the head is the embedding matrix itself, and is not stored
    assert wa["lm_head.weight"] is wa["model.embed_tokens.weight"]
    with safe_open(str(tmp_path / "a" / "model.safetensors"), framework="pt") as h:
        assert "lm_head.weight" not in h.keys()
    # statistics of the draw
    assert abs(wa["model.layers.0.mlp.up_proj.weight"].float().std().item() - 0.02) < 2e-3
    assert abs(wa["model.layers.0.input_layernorm.weight"].float().mean().item() - 1.0) < 0.05
    assert config.tie_word_embeddings


def test_kept_dtypes(tmp_path):
    _folder(tmp_path, dtype="float32")
    specs = _specs(tmp_path)
    bf = load_weights(tmp_path, specs, Runtime(torch.device("cpu"), torch.bfloat16))
    assert bf["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16  # matrices: compute dtype
    assert bf["model.norm.weight"].dtype == torch.float32  # a vector stored in 32-bit stays so
    assert bf["model.layers.0.self_attn.q_proj.bias"].dtype == torch.float32
    f32 = load_weights(tmp_path, specs, Runtime(torch.device("cpu"), torch.float32))
    assert all(t.dtype == torch.float32 for t in f32.values())
    _folder(tmp_path / "bf", dtype="bfloat16")
    up = load_weights(tmp_path / "bf", _specs(tmp_path / "bf"), Runtime(torch.device("cpu"), torch.float32))
    assert all(t.dtype == torch.float32 for t in up.values())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    _folder(tmp_path, "B")

    def edit(t):
        del t["model.layers.1.mlp.down_proj.weight"]
        del t["lm_head.weight"]  # untied: must be there
        t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(4)  # skipped silently
        t["model.layers.7.extra.weight"] = torch.zeros(2)
        t["model.norm.weight"] = torch.zeros(5)
    _rewrite(tmp_path, edit)
    with pytest.raises(WeightError) as err:
        load_weights(tmp_path, _specs(tmp_path), CPU)
    text = str(err.value)
    assert "missing tensors (2)" in text and "model.layers.1.mlp.down_proj.weight" in text and "lm_head.weight" in text
    assert "unexpected tensors (1)" in text and "model.layers.7.extra.weight" in text and "inv_freq" not in text
    assert "wrong shapes (1)" in text and "model.norm.weight: file (5,) vs model (96,)" in text


def test_non_finite_and_tied_mismatch(tmp_path):
    _folder(tmp_path, "A")

    def edit(t):
        t["model.norm.weight"][3] = float("nan")
        t["lm_head.weight"] = t["model.embed_tokens.weight"] + 1
    _rewrite(tmp_path, edit)
    with pytest.raises(WeightError) as err:
        load_weights(tmp_path, _specs(tmp_path), CPU)
    assert "non-finite values in: model.norm.weight" in str(err.value)
    assert "tied tensors that differ" in str(err.value)


def test_file_discovery(tmp_path):
    with pytest.raises(FileNotFoundError):
        safetensor_files(tmp_path)
    save_file({"a": torch.zeros(1)}, str(tmp_path / "x-00001.safetensors"))
    assert [p.name for p in safetensor_files(tmp_path)] == ["x-00001.safetensors"]
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "gone.safetensors"}}))
    with pytest.raises(FileNotFoundError, match="missing shard"):
        safetensor_files(tmp_path)
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {}}))
    with pytest.raises(FileNotFoundError, match="empty weight_map"):
        safetensor_files(tmp_path)


def test_sharded_checkpoint_loads(tmp_path):
    _folder(tmp_path, "B")
    with safe_open(str(tmp_path / "model.safetensors"), framework="pt") as h:
        tensors = {k: h.get_tensor(k) for k in h.keys()}
    (tmp_path / "model.safetensors").unlink()
    names = sorted(tensors)
    half = len(names) // 2
    save_file({k: tensors[k] for k in names[:half]}, str(tmp_path / "m-1.safetensors"))
    save_file({k: tensors[k] for k in names[half:]}, str(tmp_path / "m-2.safetensors"))
    weight_map = {k: ("m-1.safetensors" if i < half else "m-2.safetensors") for i, k in enumerate(names)}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    got = load_weights(tmp_path, _specs(tmp_path), Runtime(torch.device("cpu"), torch.float32))
    assert all(torch.equal(got[k], tensors[k].float()) for k in names)
