"""Shared fixtures: tiny Qwen2.5 configurations that differ in every size and option,
model folders with random weights made in a temporary folder, and the ``gpu`` marker."""
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def tiny_configs():
    from slipstream_b200.config.model_config import Qwen2Config

    return {
        # 2 layers, 4 heads in 2 groups, head 16, tied, theta 1e4, eps 1e-6, page 4
        "A": (Qwen2Config(vocab_size=256, hidden_size=64, num_hidden_layers=2, max_position_embeddings=128,
                          torch_dtype="float32", intermediate_size=176, num_attention_heads=4,
                          num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, rope_theta=10000.0,
                          tie_word_embeddings=True), 4),
        # 3 layers, 3 heads on 1 kv head, head 32, untied, theta 1e6, eps 1e-5, page 8
        "B": (Qwen2Config(vocab_size=320, hidden_size=96, num_hidden_layers=3, max_position_embeddings=256,
                          torch_dtype="float32", intermediate_size=224, num_attention_heads=3,
                          num_key_value_heads=1, head_dim=32, rms_norm_eps=1e-5, rope_theta=1000000.0,
                          tie_word_embeddings=False), 8),
        # 1 layer, 5 heads each with its own kv head, head 48 (not hidden / heads), odd vocabulary,
        # no q/k/v bias, biased feed-forward, page 16, bfloat16 on disk
        "C": (Qwen2Config(vocab_size=263, hidden_size=80, num_hidden_layers=1, max_position_embeddings=512,
                          torch_dtype="bfloat16", intermediate_size=120, num_attention_heads=5,
                          num_key_value_heads=5, head_dim=48, rms_norm_eps=1e-6, rope_theta=50000.0,
                          tie_word_embeddings=False, attention_bias=False, mlp_bias=True), 16),
    }


def sharpen(folder, factor=8.0):
    """Scale the query and key projections so that attention is far from uniform: a wrong or
    missing key then changes the logits visibly."""
    from safetensors import safe_open
    from safetensors.torch import save_file

    path = Path(folder) / "model.safetensors"
    tensors = {}
    with safe_open(str(path), framework="pt") as handle:
        for key in handle.keys():
            t = handle.get_tensor(key).clone()
            if ".q_proj." in key or ".k_proj." in key:
                t = (t.float() * factor).to(t.dtype)
            if "mlp." in key or "embed_tokens" in key or "lm_head" in key:
                t = (t.float() * 3.0).to(t.dtype)
            tensors[key] = t.contiguous()
    save_file(tensors, str(path), metadata={"format": "pt"})


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """{name: (folder, config, page_size)} for the tiny configurations, weights sharpened."""
    from slipstream_b200.weights.random_init import write_random_model

    out = {}
    for name, (config, page) in tiny_configs().items():
        folder = tmp_path_factory.mktemp(f"tiny{name}")
        write_random_model(config, folder, seed=11 + ord(name))
        sharpen(folder)
        out[name] = (str(folder), config, page)
    return out


def random_tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return [int(t) for t in torch.randint(0, vocab, (n,), generator=g)]
