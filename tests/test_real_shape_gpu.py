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


def test_a_portion_of_2048_tokens_runs_every_projection_on_the_two_sm_kernel(big_folder, monkeypatch):
    """From 2,048 tokens the q/k/v, o and down projections of a prompt portion leave the library for the
    persistent two-SM tcgen05 kernel (gate/up with its SwiGLU is there already).  A prompt of 2,100 tokens as
    portions of 2,048 and 52; logits of rows of both portions against the plain implementation."""
    from slipstream_b200 import ops
    from slipstream_b200.engine.runner import ModelRunner, StepEntry
    folder, config = big_folder
    n = 2100
    tokens = random_tokens(config.vocab_size, n, 12)
    assert n - 52 >= ops.functions.MANY_TOKENS and config.hidden_size >= ops.functions.MANY_WIDTH
    cfg, weights = plain.read_model_folder(folder, torch.float32)
    s = plain.sizes(cfg)
    x = weights["model.embed_tokens.weight"][torch.as_tensor(tokens)]
    for index in range(s["layers"]):
        x = plain.decoder_layer(x, torch.arange(n), weights, index, s)
    rows = [0, 1, 63, 64, 1000, 2047, 2048, 2049, 2099]
    want = plain.rms_norm(x[rows], weights["model.norm.weight"], s["eps"]) @ weights["lm_head.weight"].T
    del weights, x
    runner = ModelRunner(folder, dtype="bfloat16", page_size=16, num_pages=160, max_num_seqs=2)
    def library_product(*args, **kwargs):
        raise AssertionError("a library matrix product ran in a 2,048-token portion")

    before = ops.launch_count()
    with monkeypatch.context() as patch:
        patch.setattr(torch, "mm", library_product)
        patch.setattr(torch, "addmm", library_product)
        first = runner.step([StepEntry("r", tokens[:2048], [r for r in rows if r < 2048])]).float().cpu()
    launches = ops.launch_count() - before
    second = runner.step([StepEntry("r", tokens[2048:], [r - 2048 for r in rows if r >= 2048])]).float().cpu()
    got = torch.cat([first, second])
    err = (got - want).abs().max(dim=1).values
    assert err.max() <= 3e-2 * want.abs().max(), (int(err.argmax()), err.max().item(), want.abs().max().item())
    # embedding + per layer (norm, q/k/v, rotary, attention, o, norm, gate/up, down) + final norm + LM head: all ours
    assert launches == 1 + 8 * s["layers"] + 2, launches
    runner.check()
