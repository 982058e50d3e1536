"""Replays the same requests whole, with the last 32 tokens one by one, in portions of changing
size, and mixed with other requests under a small pool, in float32 and bfloat16, through the
framework's runner and through bin/trace_run, and compares every logit row with the plain
implementation."""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
import replay_plans as plans
from conftest import ROOT, random_tokens

pytestmark = pytest.mark.gpu

# Largest |difference| allowed, as a fraction of the largest |logit| of the oracle.  float32: sums of
# a few hundred products rounded at 6e-8, through a few layers.  bfloat16: activations are rounded to
# 8 bits of mantissa (4e-3) after every product and norm.
TOLERANCE = {"float32": 2e-5, "bfloat16": 3e-2}
LENGTHS = {"r0": 70, "r1": 45, "r2": 97, "r3": 33, "r4": 64, "r5": 21}


def oracle(folder, requests, dtype):
    config, weights = plain.read_model_folder(folder, torch.float64)
    if dtype == "bfloat16":  # the engine keeps matrices in bfloat16: give the oracle the same values
        weights = {k: v.to(torch.bfloat16).to(torch.float64) if v.dim() == 2 else v for k, v in weights.items()}
    return {rid: plain.forward_logits(config, weights, toks).float().numpy() for rid, toks in requests.items()}


def run_plan(runner, steps):
    from slipstream_b200.engine.runner import StepEntry

    outs = []
    for step in steps:
        logits = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in step["entries"]])
        outs.append(logits.cpu().numpy())
        for rid in step["end"]:
            runner.release(rid)
        runner.cache.check_invariants()
    runner.check()
    return outs


def compare(rows, want, dtype, what):
    for rid, ref in want.items():
        got = np.stack(rows[rid])
        assert got.shape == ref.shape, (what, rid, got.shape, ref.shape)
        err = np.abs(got - ref).max(axis=1)
        bound = TOLERANCE[dtype] * np.abs(ref).max()
        worst = int(err.argmax())
        assert err[worst] <= bound, (f"{what}: request {rid}, first wrong token "
                                     f"{int(np.argmax(err > bound))}, worst token {worst}: {err[worst]:.3e} > {bound:.3e}")


@pytest.fixture(scope="module")
def requests_for():
    def make(config):
        return {rid: random_tokens(config.vocab_size, n, 100 + i) for i, (rid, n) in enumerate(LENGTHS.items())}
    return make


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_every_way_of_cutting_gives_the_plain_logits(model_folders, requests_for, name, dtype):
    from slipstream_b200.engine.runner import ModelRunner

    folder, config, page = model_folders[name]
    requests = requests_for(config)
    want = oracle(folder, requests, dtype)
    max_tokens = 256  # fewer than the 330 tokens of all requests together: pages are used again
    runner = ModelRunner(folder, dtype=dtype, page_size=page, num_pages=max_tokens // page, max_num_seqs=4)
    results = {}
    for what, steps in (("whole", plans.whole(requests)),
                        ("tail one by one", plans.tail_one_by_one(requests)),
                        ("changing portions", plans.changing_portions(requests)),
                        ("mixed", plans.mixed(requests, max_tokens, page, seed=5)),
                        ("mixed again", plans.mixed(requests, max_tokens, page, seed=6))):
        rows = plans.collect(steps, run_plan(runner, steps))
        compare(rows, want, dtype, f"{name} {dtype} {what}")
        results[what] = rows
        assert runner.cache.num_free_pages() == max_tokens // page
    assert max(len(s["entries"]) for s in plans.mixed(requests, max_tokens, page, seed=5)) >= 3
    # the cut changes nothing beyond rounding: compare the ways with one another, tighter than with the oracle
    for what in ("tail one by one", "changing portions", "mixed"):
        for rid in requests:
            a, b = np.stack(results["whole"][rid]), np.stack(results[what][rid])
            assert np.abs(a - b).max() <= 0.5 * TOLERANCE[dtype] * np.abs(a).max(), (what, rid)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_folders, requests_for, tmp_path, dtype):
    folder, config, page = model_folders["B"]
    requests = {k: v for k, v in requests_for(config).items() if k in ("r0", "r1", "r3", "r5")}
    want = oracle(folder, requests, dtype)
    steps = plans.mixed(requests, 192, 16, seed=2) + plans.tail_one_by_one({"r3": requests["r3"]})
    steps.insert(3, {"entries": [], "end": []})  # a step may be empty
    steps[0]["entries"][0]["want"] = steps[0]["entries"][0]["want"]  # keep all
    lines = "".join(json.dumps({"step": i, **s}) + "\n" for i, s in enumerate(steps))
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", str(out), "--max-tokens", "192"], input=lines, capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:-1] == [f"done {i}" for i in range(len(steps))]
    outputs = []
    for i, s in enumerate(steps):
        wanted = sum(len(e["want"]) for e in s["entries"])
        path = out / f"{i}.f32"
        if wanted == 0:
            assert not path.exists()
            outputs.append(None)
            continue
        data = np.fromfile(path, dtype="<f4")
        assert data.size == wanted * config.vocab_size
        outputs.append(data.reshape(wanted, config.vocab_size))
    rows = plans.collect(steps, outputs)
    # r3 was replayed twice: once mixed, once alone
    n3 = len(requests["r3"])
    again = {"r3": rows["r3"][n3:]}
    rows["r3"] = rows["r3"][:n3]
    compare(rows, want, dtype, f"trace_run {dtype} mixed")
    compare(again, {"r3": want["r3"]}, dtype, f"trace_run {dtype} tail")


def test_long_requests_decode_through_a_graph_with_more_slices(tmp_path, monkeypatch):
    """From 8,192 cached tokens a decode step of few requests cuts the keys into more than 8 slices (several
    thread-block clusters whose results meet in scratch memory) and runs a graph captured for that.  The
    logits are those of the same steps with 8 slices, up to the order of the additions."""
    from slipstream_b200 import ops
    from slipstream_b200.config.model_config import Qwen2Config
    from slipstream_b200.engine.runner import ModelRunner, StepEntry
    from slipstream_b200.weights.random_init import write_random_model
    from conftest import sharpen

    config = Qwen2Config(vocab_size=300, hidden_size=128, num_hidden_layers=2, max_position_embeddings=16384,
                         torch_dtype="bfloat16", intermediate_size=256, num_attention_heads=8, num_key_value_heads=2,
                         head_dim=64, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False)
    write_random_model(config, tmp_path, seed=3)
    sharpen(tmp_path, factor=4.0)
    prompts = {"long": random_tokens(300, 8300, 1), "short": random_tokens(300, 40, 2)}
    tails = {rid: random_tokens(300, 6, 10 + i) for i, rid in enumerate(prompts)}

    def run(wide_from):
        monkeypatch.setattr(ops.functions, "WIDE_CONTEXT", wide_from)
        runner = ModelRunner(str(tmp_path), dtype="bfloat16", page_size=16, num_pages=600, max_num_seqs=4)
        for rid, tokens in prompts.items():
            for i in range(0, len(tokens), 2048):
                runner.step([StepEntry(rid, tokens[i:i + 2048], [])])
        rows = []
        for k in range(6):  # the long request alone (bucket 1), then both (bucket 2)
            ids = ["long"] if k < 3 else ["long", "short"]
            rows.append(runner.step([StepEntry(rid, [tails[rid][k]], [0]) for rid in ids]).float().cpu().numpy())
        runner.check()
        return rows, sorted(runner._graphs)

    wide_rows, wide_graphs = run(8192)
    narrow_rows, narrow_graphs = run(10 ** 9)
    assert wide_graphs == [(1, (True,)), (2, (True,))] and narrow_graphs == [(1, (False,)), (2, (False,))]
    assert ops.decode_slices(1, 2, 4, 16384, wide=True) > 8 == ops.decode_slices(1, 2, 4, 16384)
    for a, b in zip(wide_rows, narrow_rows):
        assert np.abs(a - b).max() <= 0.5 * TOLERANCE["bfloat16"] * np.abs(b).max()
        assert not np.array_equal(a, b), "both runs took the same path"


def test_short_portions_behind_a_long_prefix_share_their_keys_among_blocks(tmp_path):
    """A portion of a few dozen tokens behind a thousand cached ones is a handful of query tiles with many key
    tiles each: the tcgen05 prefill kernel then cuts the keys of every query tile into parts that a thread-block
    cluster combines.  Portions of 40 to 636 tokens behind 1,060 to 2,100 cached ones (2 and 4 parts at these
    lengths; the kernel tests cover 8) against the oracle."""
    from slipstream_b200 import ops
    from slipstream_b200.config.model_config import Qwen2Config
    from slipstream_b200.engine.runner import ModelRunner
    from slipstream_b200.weights.random_init import write_random_model
    from conftest import sharpen

    config = Qwen2Config(vocab_size=211, hidden_size=96, num_hidden_layers=2, max_position_embeddings=4096,
                         torch_dtype="bfloat16", intermediate_size=136, num_attention_heads=6, num_key_value_heads=2,
                         head_dim=64, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True)
    write_random_model(config, tmp_path, seed=9)
    sharpen(tmp_path, factor=4.0)
    tokens = random_tokens(211, 2400, 4)
    want = oracle(str(tmp_path), {"r": tokens}, "bfloat16")["r"]
    assert ops.prefill_key_parts([40], [1100], 42, 2) == 2 and ops.prefill_key_parts([300], [2400], 42, 2) == 4
    runner = ModelRunner(str(tmp_path), dtype="bfloat16", page_size=16, num_pages=160, max_num_seqs=2)
    cuts = [1060, 40, 64, 300, 636, 300]
    steps, at = [], 0
    for n in cuts:
        steps.append({"entries": [{"id": "r", "tokens": tokens[at:at + n], "want": list(range(n))}], "end": []})
        at += n
    assert at == len(tokens)
    steps[-1]["end"] = ["r"]
    rows = plans.collect(steps, run_plan(runner, steps))
    compare(rows, {"r": want}, "bfloat16", "portions behind a long prefix")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_tables_of_replayed_decode_steps_follow_their_requests(model_folders, dtype):
    """A replayed decode graph keeps its block tables on the device and receives only what changed.  Three
    requests of about a hundred tokens reach their first common decode step with more changes than the patch
    area holds (the whole mirror is copied), then grow page by page (patches), one ends and its name comes back
    with other tokens in the same row (the row starts over), and the batch shrinks to another bucket and grows
    again.  Every decoded row against the oracle."""
    from slipstream_b200.engine.runner import ModelRunner, StepEntry

    folder, config, page = model_folders["A"]
    vocab = config.vocab_size
    requests = {"x": random_tokens(vocab, 118, 31), "y": random_tokens(vocab, 110, 32), "z": random_tokens(vocab, 125, 33),
                "x2": random_tokens(vocab, 60, 34)}
    want = oracle(folder, requests, dtype)
    runner = ModelRunner(folder, dtype=dtype, page_size=page, num_pages=128, max_num_seqs=4)
    got = {rid: {} for rid in requests}

    def decode(ids, at, names=None):
        """One decode step: request ``ids[k]`` (called ``names[k]`` by the runner) brings its token ``at[ids[k]]``."""
        names = names or ids
        out = runner.step([StepEntry(n, [requests[r][at[r]]], [0]) for r, n in zip(ids, names)]).cpu().numpy()
        for k, r in enumerate(ids):
            got[r][at[r]] = out[k]
            at[r] += 1

    at = {"x": 100, "y": 100, "z": 100, "x2": 40}
    for rid in ("x", "y", "z"):
        runner.step([StepEntry(rid, requests[rid][:100], [])])
    for _ in range(6):
        decode(["x", "y", "z"], at)
    graph = runner._graphs[(4, tuple(False for _ in runner.variant_parts))]
    assert graph.full_copies == 1, "75 new table entries do not fit 64 patches"
    decode(["y", "z"], at)  # bucket 2, its own tables
    decode(["x", "y", "z"], at)  # back: x's row is as it was, y and z grew meanwhile
    while at["y"] < 110:
        decode(["x", "y", "z"], at)
    runner.release("y")
    # another request under the name "x" takes over after x has ended: same name, same row, a table of its own
    while at["x"] < 118:
        decode(["x", "z"], at)
    runner.release("x")
    runner.step([StepEntry("x", requests["x2"][:40], [])])
    while at["x2"] < 60:
        decode(["x2", "z"] if at["z"] < 125 else ["x2"], at, names=["x", "z"] if at["z"] < 125 else ["x"])
    assert graph.full_copies == 1
    runner.check()
    runner.cache.check_invariants()
    for rid, rows in got.items():
        assert rows, rid
        for pos, row in rows.items():
            err = np.abs(row - want[rid][pos]).max()
            assert err <= TOLERANCE[dtype] * np.abs(want[rid]).max(), (rid, pos, err)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_steps_with_prompt_portions_replayed_from_graphs(model_folders, requests_for, name, dtype):
    """Steps with prompt portions are captured per bucket of (tokens, requests) once a bucket has come up a few
    times, and replayed with padding rows, empty requests and empty query tiles.  Here every such step is
    captured at once: the logits must be those of the same steps run kernel by kernel, bit for bit (the padding
    must not reach a live row), and the plain implementation's within the usual bound."""
    from slipstream_b200.engine.graphs import MixedGraph
    from slipstream_b200.engine.runner import ModelRunner

    folder, config, page = model_folders[name]
    requests = requests_for(config)
    want = oracle(folder, requests, dtype)
    max_tokens = 256
    results = {}
    for captured in (False, True):
        runner = ModelRunner(folder, dtype=dtype, page_size=page, num_pages=max_tokens // page, max_num_seqs=4)
        runner.mixed_graph_after = 0 if captured else 10 ** 9
        for what, steps in (("changing portions", plans.changing_portions(requests)),
                            ("mixed", plans.mixed(requests, max_tokens, page, seed=5)),
                            ("serving", [{"entries": [dict(e, want=e["want"][-1:]) for e in s["entries"]], "end": s["end"]}
                                         for s in plans.mixed(requests, max_tokens, page, seed=6)])):
            outs = run_plan(runner, steps)
            rows = plans.collect(steps, outs)
            if what != "serving":
                compare(rows, want, dtype, f"{name} {dtype} {what} captured={captured}")
            results[(what, captured)] = rows
            assert runner.cache.num_free_pages() == max_tokens // page
        graphs = [k for k, g in runner._mixed_graphs.items() if isinstance(g, MixedGraph)]
        assert bool(graphs) == captured
        if captured:  # both kinds were used: logits for every token (a replayed trace) and one per request (serving)
            assert {k[2] for k in graphs} == {True, False}, graphs
    for what in ("changing portions", "mixed", "serving"):
        for rid in results[(what, True)]:
            a, b = np.stack(results[(what, False)][rid]), np.stack(results[(what, True)][rid])
            assert np.array_equal(a, b), (what, rid, np.abs(a - b).max())
