"""The kernels at the layer sizes of Qwen2.5-7B (hidden 3584, 28 heads on 4 kv heads of 128, feed-forward
18944, vocabulary 152064), two layers deep so that the plain implementation on the CPU stays quick: a prompt
in portions, then decode steps (which take the CUDA-graph, split-KV and tcgen05 paths), in float32 and bfloat16."""
import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from conftest import random_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def big_folder(tmp_path_factory):
    from slipstream_b200.config.model_config import Qwen2Config
    from slipstream_b200.weights.random_init import write_random_model
    config = Qwen2Config(vocab_size=152064, hidden_size=3584, num_hidden_layers=2, max_position_embeddings=8192,
                         torch_dtype="bfloat16", intermediate_size=18944, num_attention_heads=28,
                         num_key_value_heads=4, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
                         tie_word_embeddings=False)
    folder = tmp_path_factory.mktemp("qwen7b_2layers")
    # at this width N(0, 0.02) weights already give attention scores of order ten: no sharpening needed
    write_random_model(config, folder, seed=3)
    return str(folder), config


@pytest.mark.parametrize("dtype, tol", [("float32", 5e-5), ("bfloat16", 3e-2)])
def test_two_layers_of_the_7b_shape(big_folder, dtype, tol):
    from slipstream_b200.engine.runner import ModelRunner, StepEntry
    folder, config = big_folder
    tokens = random_tokens(config.vocab_size, 150, 9)
    cfg, weights = plain.read_model_folder(folder, torch.float32)
    want = plain.forward_logits(cfg, weights, tokens)
    del weights
    runner = ModelRunner(folder, dtype=dtype, page_size=16, num_pages=64, max_num_seqs=4)
    rows, i = [], 0
    for take in (100, 37, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1):
        rows.append(runner.step([StepEntry("r", tokens[i:i + take], list(range(take)))]).cpu())
        i += take
    got = torch.cat(rows)
    assert i == 150 and got.shape == want.shape
    err = (got - want).abs().max(dim=1).values
    assert err.max() <= tol * want.abs().max(), (dtype, int(err.argmax()), err.max().item(), want.abs().max().item())
    runner.check()
