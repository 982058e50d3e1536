"""The engine at the layer sizes of the Qwen2.5 models (7B: hidden 3584, 28 heads on 4 kv heads of 128,
feed-forward 18944, vocabulary 152064; 0.5B: 896, 14 on 2 of 64, 4864, tied; 14B: 5120, 40 on 8 of 128, 13824),
two layers deep so that the plain implementation on the CPU stays quick.  These are the sizes at which the
tcgen05 attention with groups of 7 heads, the library products between 17 and 2,047 tokens, the two-SM product
from 2,048 tokens, the key-parts clusters and the split decode kernels meet.  Every way of cutting the requests
(whole; the last 32 tokens one by one; portions of changing size; up to four live requests mixed under a pool
so small that pages are used again) in float32 and in bfloat16 against the plain implementation, plus one long
request whose portions of 300 and 2,048 tokens run beside decoded tokens of other requests."""
import numpy as np
import pytest
import torch

import plain_qwen2 as plain
import replay_plans as plans
from conftest import random_tokens
from test_replay_gpu import run_plan

pytestmark = pytest.mark.gpu

TOLERANCE = {"float32": 5e-5, "bfloat16": 3e-2}  # of the largest |logit| of the oracle
SHAPES = {
    "7b": dict(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_attention_heads=28,
               num_key_value_heads=4, head_dim=128, rms_norm_eps=1e-6, tie_word_embeddings=False),
    "0.5b": dict(vocab_size=151936, hidden_size=896, intermediate_size=4864, num_attention_heads=14,
                 num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, tie_word_embeddings=True),
    # the 14B vocabulary is the 7B's; a smaller one (no power of two) keeps the folder and the oracle quick
    "14b": dict(vocab_size=32064, hidden_size=5120, intermediate_size=13824, num_attention_heads=40,
                num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, tie_word_embeddings=False),
}
LENGTHS = {"r0": 150, "r1": 70, "r2": 97, "r3": 33, "r4": 200, "r5": 21}
POOL_TOKENS = 448  # the six requests hold 832 when each is rounded up to 64: pages are used again


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """name -> (folder, config), each written at its first use."""
    from slipstream_b200.config.model_config import Qwen2Config
    from slipstream_b200.weights.random_init import write_random_model

    made = {}

    def get(name):
        if name not in made:
            config = Qwen2Config(num_hidden_layers=2, max_position_embeddings=8192, torch_dtype="bfloat16",
                                 rope_theta=1000000.0, **SHAPES[name])
            folder = tmp_path_factory.mktemp("shape_" + name.replace(".", "_"))
            # at these widths N(0, 0.02) weights already give attention scores of order ten: no sharpening needed
            write_random_model(config, folder, seed=3)
            made[name] = (str(folder), config)
        return made[name]

    return get


def oracle_rows(folder, tokens, rows=None):
    """float32 on the CPU; the folder's matrices are stored in bfloat16, so both precisions of the engine start
    from the same values."""
    cfg, weights = plain.read_model_folder(folder, torch.float32)
    return plain.forward_logits(cfg, weights, tokens, rows=rows).numpy()


def check(rows, want, dtype, what):
    for rid, ref in want.items():
        got = np.stack(rows[rid])
        assert got.shape == ref.shape, (what, rid, got.shape, ref.shape)
        err = np.abs(got - ref).max(axis=1)
        bound = TOLERANCE[dtype] * np.abs(ref).max()
        assert err.max() <= bound, (f"{what}: request {rid}, first wrong row {int(np.argmax(err > bound))}, "
                                    f"worst row {int(err.argmax())}: {err.max():.3e} > {bound:.3e}")


@pytest.fixture(scope="module")
def oracles(folders):
    cache = {}

    def get(name):
        if name not in cache:
            folder, config = folders(name)
            requests = {rid: random_tokens(config.vocab_size, n, 300 + i) for i, (rid, n) in enumerate(LENGTHS.items())}
            cfg, weights = plain.read_model_folder(folder, torch.float32)
            cache[name] = (requests, {rid: plain.forward_logits(cfg, weights, t).numpy() for rid, t in requests.items()})
        return cache[name]

    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_way_of_cutting_at_the_7b_layer_sizes(folders, oracles, dtype):
    from slipstream_b200.engine.runner import ModelRunner

    folder, config = folders("7b")
    requests, want = oracles("7b")
    runner = ModelRunner(folder, dtype=dtype, page_size=16, num_pages=POOL_TOKENS // 16, max_num_seqs=4)
    results = {}
    for what, steps in (("whole", plans.whole(requests)), ("tail one by one", plans.tail_one_by_one(requests)),
                        ("changing portions", plans.changing_portions(requests)),
                        ("mixed", plans.mixed(requests, POOL_TOKENS, 16, seed=5))):
        rows = plans.collect(steps, run_plan(runner, steps))
        check(rows, want, dtype, f"7b {dtype} {what}")
        results[what] = rows
        assert runner.cache.num_free_pages() == POOL_TOKENS // 16
    assert max(len(s["entries"]) for s in plans.mixed(requests, POOL_TOKENS, 16, seed=5)) >= 3
    for what in ("tail one by one", "changing portions", "mixed"):
        for rid in requests:
            a, b = np.stack(results["whole"][rid]), np.stack(results[what][rid])
            assert np.abs(a - b).max() <= 0.5 * TOLERANCE[dtype] * np.abs(a).max(), (what, rid)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["0.5b", "14b"])
def test_mixed_requests_at_the_other_layer_sizes(folders, oracles, name, dtype):
    from slipstream_b200.engine.runner import ModelRunner

    folder, config = folders(name)
    requests, want = oracles(name)
    runner = ModelRunner(folder, dtype=dtype, page_size=16, num_pages=POOL_TOKENS // 16, max_num_seqs=4)
    for seed in (5, 6):
        steps = plans.mixed(requests, POOL_TOKENS, 16, seed=seed)
        rows = plans.collect(steps, run_plan(runner, steps))
        check(rows, want, dtype, f"{name} {dtype} mixed {seed}")
        assert runner.cache.num_free_pages() == POOL_TOKENS // 16


LONG_ROWS = {  # rows of the long request whose logits are compared, per portion (the others are not asked for)
    300: [0, 1, 63, 64, 65, 127, 299], 2048: [0, 1, 17, 18, 1000, 2046, 2047], 52: [0, 1, 51]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_beside_decoded_tokens_of_other_requests(folders, dtype):
    """One request of 2,400 tokens goes in as portions of 300 (between 65 and 2,047 tokens: library products in
    bfloat16), 2,048 (the two-SM tcgen05 product, with rows of other requests making the row count no multiple of
    the tile) and 52, each beside requests that bring one, two or three tokens of their own."""
    from slipstream_b200.engine.runner import ModelRunner

    folder, config = folders("7b")
    requests = {"L": random_tokens(config.vocab_size, 2400, 40), "a": random_tokens(config.vocab_size, 40, 41),
                "b": random_tokens(config.vocab_size, 90, 42), "c": random_tokens(config.vocab_size, 12, 43)}
    cuts, at, long_rows = [], 0, []
    for n in (300, 2048, 52):
        cuts.append((at, n))
        long_rows += [at + r for r in LONG_ROWS[n]]
        at += n
    cfg, weights = plain.read_model_folder(folder, torch.float32)
    want = {rid: plain.forward_logits(cfg, weights, t).numpy() for rid, t in requests.items() if rid != "L"}
    want["L"] = plain.forward_logits(cfg, weights, requests["L"], rows=long_rows).numpy()
    del weights

    def entry(rid, at, n, rows=None):
        return {"id": rid, "tokens": requests[rid][at:at + n], "want": list(range(n)) if rows is None else rows}

    steps = [
        {"entries": [entry("a", 0, 30), entry("b", 0, 80), entry("c", 0, 8)], "end": []},
        {"entries": [entry("L", 0, 300, LONG_ROWS[300]), entry("a", 30, 1)], "end": []},
        {"entries": [entry("a", 31, 1), entry("L", 300, 2048, LONG_ROWS[2048]), entry("b", 80, 1), entry("c", 8, 2)],
         "end": []},
        {"entries": [entry("b", 81, 3), entry("a", 32, 1), entry("c", 10, 1)], "end": []},
        {"entries": [entry("L", 2348, 52, LONG_ROWS[52]), entry("b", 84, 6), entry("a", 33, 7), entry("c", 11, 1)],
         "end": ["L", "a", "b", "c"]},
    ]
    assert sum(len(e["tokens"]) for e in steps[2]["entries"]) == 2052
    runner = ModelRunner(folder, dtype=dtype, page_size=16, num_pages=176, max_num_seqs=4)
    rows = plans.collect(steps, run_plan(runner, steps))
    check(rows, want, dtype, f"7b {dtype} long portions beside decoded tokens")
    assert runner.cache.num_free_pages() == 176


def test_a_portion_of_2048_tokens_runs_every_projection_on_the_two_sm_kernel(folders, monkeypatch):
    """From 2,048 tokens the q/k/v, o and down projections of a prompt portion leave the library for the
    persistent two-SM tcgen05 kernel (gate/up with its SwiGLU is there already): with the library products
    patched to raise, a portion of 2,048 tokens runs, and launches exactly the kernels of this package."""
    from slipstream_b200 import ops
    from slipstream_b200.engine.runner import ModelRunner, StepEntry

    folder, config = folders("7b")
    tokens = random_tokens(config.vocab_size, 2048, 12)
    runner = ModelRunner(folder, dtype="bfloat16", page_size=16, num_pages=160, max_num_seqs=2)

    def library_product(*args, **kwargs):
        raise AssertionError("a library matrix product ran in a 2,048-token portion")

    before = ops.launch_count()
    with monkeypatch.context() as patch:
        patch.setattr(torch, "mm", library_product)
        patch.setattr(torch, "addmm", library_product)
        runner.step([StepEntry("r", tokens, [2047])])
    launches = ops.launch_count() - before
    # embedding + per layer (norm, q/k/v, rotary, attention, o, norm, gate/up, down) + final norm + LM head: all ours
    assert launches == 1 + 8 * config.num_hidden_layers + 2, launches
    runner.check()
