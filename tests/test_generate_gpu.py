"""Generation through the Python entry point and the command line, sampling kernels against their
plain restatement, preemption, long decoding and the first tokens of a sequence."""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from conftest import ROOT, random_tokens

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def make_engine(folder, page, dtype="float32", pages=64, **sched):
    from slipstream_b200 import CacheConfig, EngineConfig, SchedulerConfig
    from slipstream_b200.engine.llm_engine import LLMEngine
    return LLMEngine(EngineConfig.for_model(folder, dtype=dtype, cache=CacheConfig(block_size=page, num_gpu_blocks=pages),
                                            scheduler=SchedulerConfig(**sched)))


def greedy_is_consistent(config, weights, prompt, output, slack):
    """Every generated token is the plain implementation's arg-max, or within ``slack`` of it."""
    tokens = list(prompt)
    for tok in output:
        logits = plain.forward_logits(config, weights, tokens)[-1]
        assert logits[tok] >= logits.max() - slack * logits.abs().max(), (len(tokens), tok, int(logits.argmax()))
        tokens.append(tok)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_the_plain_implementation(model_folders, name):
    """The workloads of the two tiny configurations: several requests at once, whole prompts for A,
    portions of 16 for B."""
    from slipstream_b200 import SamplingParams
    from slipstream_b200.engine.llm_engine import Request
    folder, config, page = model_folders[name]
    lengths, new = ((1, 5, 17, 33), 8) if name == "A" else ((2, 40, 97), 12)
    engine = make_engine(folder, page, prefill_chunk_size=64 if name == "A" else 16)
    prompts = [random_tokens(config.vocab_size, n, 7 + n) for n in lengths]
    params = SamplingParams(max_tokens=new, temperature=0.0, ignore_eos=True)
    outs = engine.generate_batch([Request(f"r{i}", None, p, params, float(i)) for i, p in enumerate(prompts)])
    cfg, weights = plain.read_model_folder(folder, torch.float64)
    for prompt, out in zip(prompts, outs):
        assert len(out) == new
        assert out == plain.generate_greedy(cfg, weights, prompt, new)
    # one at a time and as a stream: the same tokens
    assert engine.generate(Request("x", None, prompts[1], params, 0.0)) == outs[1]
    assert list(engine.stream(Request("y", None, prompts[2], params, 0.0))) == outs[2]
    assert engine.runner.cache.min_free_pages() == 64 and not engine.scheduler.has_work()
    engine.runner.check()


def test_bfloat16_generation_stays_on_the_plain_arg_max(model_folders):
    from slipstream_b200 import SamplingParams
    from slipstream_b200.engine.llm_engine import Request
    folder, config, page = model_folders["B"]
    engine = make_engine(folder, page, dtype="bfloat16")
    prompt = random_tokens(config.vocab_size, 30, 1)
    out = engine.generate(Request("r", None, prompt, SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True), 0.0))
    cfg, weights = plain.read_model_folder(folder, torch.float64)
    greedy_is_consistent(cfg, weights, prompt, out, slack=3e-2)


def test_too_few_pages_preempts_and_still_generates_the_same_tokens(model_folders):
    from slipstream_b200 import SamplingParams
    from slipstream_b200.engine.llm_engine import Request
    folder, config, page = model_folders["A"]
    prompts = [random_tokens(config.vocab_size, n, 50 + n) for n in (14, 9, 11)]
    params = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)
    roomy = make_engine(folder, page, pages=64)
    want = roomy.generate_batch([Request(f"r{i}", None, p, params, float(i)) for i, p in enumerate(prompts)])
    tight = make_engine(folder, page, pages=10, prefill_chunk_size=8)  # 40 token slots for 69 tokens
    got = tight.generate_batch([Request(f"r{i}", None, p, params, float(i)) for i, p in enumerate(prompts)])
    assert got == want and tight.scheduler.preemptions >= 1
    assert tight.runner.cache.min_free_pages() == 10
    tight.runner.cache.check_invariants()
    # a request that can never fit is aborted, the others finish
    outs = tight.generate_batch([Request("big", None, random_tokens(config.vocab_size, 39, 3), params, 0.0),
                                 Request("ok", None, prompts[1], params, 1.0)])
    assert outs[0] == [] and outs[1] == want[1]


def test_requests_released_at_their_arrival_times_and_the_latency_records(model_folders):
    """``generate_batch(..., inject="arrival")`` queues a request when the wall clock reaches its arrival (an offset
    from the call), sleeping while nothing is due: same tokens as the closed burst, later.  Both ways leave the
    time to first token of every request and the gaps between its tokens (slipstream/engine/llm_engine.py:107-119,
    577-598)."""
    import time
    from slipstream_b200 import SamplingParams
    from slipstream_b200.engine.llm_engine import Request, absolute_arrival
    folder, config, page = model_folders["A"]
    engine = make_engine(folder, page)
    prompts = [random_tokens(config.vocab_size, n, 70 + n) for n in (9, 21, 4)]
    params = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    arrivals = (0.0, 0.15, 0.06)
    batch = lambda: [Request(f"r{i}", None, p, params, t) for i, (p, t) in enumerate(zip(prompts, arrivals))]
    burst = engine.generate_batch(batch())
    assert len(engine.last_ttft_s) == 3 and len(engine.last_itl_s) == 3 * 5
    assert all(t >= 0 for t in engine.last_ttft_s + engine.last_itl_s)
    t0 = time.perf_counter()
    timed = engine.generate_batch(batch(), inject="arrival")
    elapsed = time.perf_counter() - t0
    assert timed == burst and elapsed >= 0.15
    assert len(engine.last_ttft_s) == 3 and len(engine.last_itl_s) == 3 * 5
    assert max(engine.last_ttft_s) < 0.15, "the clock of a request starts at its arrival, not at the call"
    assert engine.runner.cache.min_free_pages() == 64 and not engine.scheduler.has_work()
    with pytest.raises(ValueError, match="inject"):
        engine.generate_batch(batch(), inject="sometimes")
    assert absolute_arrival(2.5, 100.0) == 102.5 and absolute_arrival(1.7e9, 100.0) == 1.7e9


def test_stop_rules(model_folders):
    from slipstream_b200 import SamplingParams
    from slipstream_b200.engine.llm_engine import LLM
    folder, config, page = model_folders["A"]
    llm = LLM(folder, dtype="float32", block_size=page, num_gpu_blocks=64)
    prompt = random_tokens(config.vocab_size, 12, 4)
    base = llm.generate(prompt_token_ids=[prompt], sampling_params=SamplingParams(max_tokens=9, temperature=0.0, ignore_eos=True))[0]
    assert base.finish_reason == "length" and len(base.output_token_ids) == 9
    stop_at = base.output_token_ids[3]
    first = base.output_token_ids.index(stop_at)
    out = llm.generate(prompt_token_ids=[prompt], sampling_params=SamplingParams(max_tokens=9, temperature=0.0, stop_token_ids=(stop_at,)))[0]
    assert out.finish_reason == "stop" and out.output_token_ids == base.output_token_ids[:first + 1]  # the stop token stays
    # the context window caps the output
    short = LLM(folder, dtype="float32", block_size=page, num_gpu_blocks=64, max_model_len=16)
    out = short.generate(prompt_token_ids=[prompt], sampling_params=SamplingParams(max_tokens=9, temperature=0.0, ignore_eos=True))[0]
    assert len(out.output_token_ids) == 4 and out.finish_reason == "length"
    with pytest.raises(ValueError, match="exceeds max_model_len"):
        short.generate(prompt_token_ids=[list(range(16))])
    with pytest.raises(ValueError, match="empty prompt"):
        short.generate(prompt_token_ids=[[]])


def test_long_decoding_and_first_tokens(model_folders):
    """200 tokens decoded one by one through CUDA-graph steps, after prompts of one and two tokens,
    against whole-sequence logits."""
    from slipstream_b200.engine.runner import ModelRunner, StepEntry
    folder, config, page = model_folders["B"]
    cfg, weights = plain.read_model_folder(folder, torch.float64)
    for dtype, tol in (("float32", 2e-5), ("bfloat16", 3e-2)):
        runner = ModelRunner(folder, dtype=dtype, page_size=page, num_pages=64, max_num_seqs=4)
        toks = {"a": random_tokens(config.vocab_size, 201, 1), "b": random_tokens(config.vocab_size, 202, 2)}
        w = weights if dtype == "float32" else {k: v.bfloat16().double() if v.dim() == 2 else v for k, v in weights.items()}
        ref = {k: plain.forward_logits(cfg, w, v).float() for k, v in toks.items()}
        got = {"a": [], "b": []}
        got["a"].append(runner.step([StepEntry("a", toks["a"][:1], [0])]).cpu())
        got["b"].append(runner.step([StepEntry("b", toks["b"][:2], [0, 1])]).cpu())
        for i in range(200):
            out = runner.step([StepEntry("a", [toks["a"][1 + i]], [0]), StepEntry("b", [toks["b"][2 + i]], [0])]).cpu()
            got["a"].append(out[0:1]); got["b"].append(out[1:2])
        assert runner._graphs, "decode steps should have gone through a captured graph"
        for k in toks:
            err = (torch.cat(got[k]) - ref[k]).abs().max(dim=1).values
            assert err.max() <= tol * ref[k].abs().max(), (dtype, k, int(err.argmax()), err.max().item())
        runner.check()


# --------------------------------------------------------------------------- sampling

def philox4x32_10(key0, key1, c0, c1, c2, c3):
    """Philox4x32-10 (Salmon et al., 2011) on uint32 numpy arrays."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    c = [np.asarray(x, dtype=np.uint64) for x in (c0, c1, c2, c3)]
    k0, k1 = np.uint64(key0), np.uint64(key1)
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0, p1 = np.uint64(M0) * c[0], np.uint64(M1) * c[2]
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & mask, p1 >> np.uint64(32), p1 & mask
        c = [(hi1 ^ c[1] ^ k0) & mask, lo1, (hi0 ^ c[3] ^ k1) & mask, lo0]
        k0, k1 = (k0 + np.uint64(W0)) & mask, (k1 + np.uint64(W1)) & mask
    return c


def gumbel_noise(seed, draw, vocab):
    i = np.arange(vocab, dtype=np.uint64)
    zeros = np.zeros(vocab, dtype=np.uint64)
    c = philox4x32_10(seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF, i >> np.uint64(2), zeros + np.uint64(draw & 0xFFFFFFFF),
                      zeros + np.uint64(draw >> 32), zeros + np.uint64(0x51195))
    x = np.stack(c, axis=1)[np.arange(vocab), (i & np.uint64(3)).astype(np.int64)]
    u = ((x >> np.uint64(8)).astype(np.float64) + 0.5) / 16777216.0
    return -np.log(-np.log(u))


def run_sample(logits, rows, seen=None, slots=None):
    from slipstream_b200 import ops
    m = logits.shape[0]
    t = lambda vals, dt: torch.tensor(vals, dtype=dt, device=DEV)
    return ops.sample(logits, temperature=t([r["temperature"] for r in rows], torch.float32),
                      top_k=t([r.get("top_k", -1) for r in rows], torch.int32),
                      top_p=t([r.get("top_p", 1.0) for r in rows], torch.float32),
                      min_p=t([r.get("min_p", 0.0) for r in rows], torch.float32),
                      penalty=t([r.get("repetition_penalty", 1.0) for r in rows], torch.float32),
                      seeds=t([r["seed"] for r in rows], torch.int64), draws=t([r["draw"] for r in rows], torch.int64),
                      slots=slots, seen=seen).cpu().tolist()


def test_sampling_kernel_draws_what_the_plain_chain_draws():
    """Per row: filter with the plain chain (float64), add the same Gumbel noise, take the arg-max."""
    torch.manual_seed(0)
    vocab = 5000
    logits = (torch.randn(8, vocab) * 2.5).to(DEV)
    history = [3, 17, 17, 4999, 123]
    rows = [dict(temperature=0.7, seed=11, draw=0), dict(temperature=1.3, seed=11, draw=1, top_k=40),
            dict(temperature=1.0, seed=12, draw=5, top_p=0.8), dict(temperature=0.9, seed=13, draw=2, min_p=0.05),
            dict(temperature=0.8, seed=14, draw=9, top_k=200, top_p=0.9, min_p=0.01),
            dict(temperature=0.0, seed=1, draw=0), dict(temperature=1.0, seed=2 ** 40 + 5, draw=2 ** 33, top_k=1),
            dict(temperature=1.1, seed=15, draw=3, repetition_penalty=1.7, top_k=50)]
    from slipstream_b200 import ops
    seen = torch.zeros(2, (vocab + 31) // 32, dtype=torch.int32, device=DEV)
    ops.mark_seen(seen[1], torch.tensor(history, dtype=torch.int32, device=DEV), vocab)
    slots = torch.tensor([-1] * 7 + [1], dtype=torch.int32, device=DEV)
    got = run_sample(logits, rows, seen=seen, slots=slots)
    for i, r in enumerate(rows):
        row = logits[i].cpu()
        if r["temperature"] == 0.0 or r.get("top_k") == 1:
            assert got[i] == int(row.argmax())
            continue
        kept = plain.filtered_logits(row, temperature=r["temperature"], top_k=r.get("top_k", -1), top_p=r.get("top_p", 1.0),
                                     min_p=r.get("min_p", 0.0), repetition_penalty=r.get("repetition_penalty", 1.0),
                                     history=history if i == 7 else ()).numpy()
        score = kept + gumbel_noise(r["seed"], r["draw"], vocab)
        assert np.isfinite(kept[got[i]]), (i, "the kernel drew a token the plain chain removed")
        assert score[got[i]] >= score.max() - 1e-4, (i, got[i], int(score.argmax()))
    # the sampled token is now marked as seen in the request's slot
    tok = got[7]
    assert (int(seen[1, tok >> 5]) >> (tok & 31)) & 1
    # same seed and draw: same token, whatever else is in the batch
    assert run_sample(logits[2:3].contiguous(), rows[2:3]) == [got[2]]


def test_sampling_follows_the_softmax_distribution():
    vocab, n = 6, 4000
    probs = torch.tensor([0.4, 0.25, 0.15, 0.1, 0.07, 0.03])
    logits = (probs.log() * 0.8).repeat(n, 1).to(DEV).contiguous()  # temperature 0.8 undoes the scaling
    rows = [dict(temperature=0.8, seed=99, draw=d) for d in range(n)]
    counts = np.bincount(run_sample(logits, rows), minlength=vocab)
    expected = probs.numpy() * n
    chi2 = ((counts - expected) ** 2 / expected).sum()
    assert chi2 < 25.0, (counts.tolist(), chi2)  # 5 degrees of freedom: p < 1e-4 beyond 25


def test_seeded_sampling_through_the_engine(model_folders):
    from slipstream_b200 import SamplingParams
    from slipstream_b200.engine.llm_engine import Request
    folder, config, page = model_folders["B"]
    prompts = [random_tokens(config.vocab_size, n, n) for n in (2, 40, 97)]
    params = SamplingParams(max_tokens=12, temperature=0.7, seed=1234, ignore_eos=True)
    eng = make_engine(folder, page, prefill_chunk_size=16)
    a = eng.generate_batch([Request(f"r{i}", None, p, params, float(i)) for i, p in enumerate(prompts)])
    alone = [make_engine(folder, page, prefill_chunk_size=64).generate(Request("s", None, p, params, 0.0)) for p in prompts]
    assert a == alone and all(len(o) == 12 for o in a)
    other = eng.generate(Request("t", None, prompts[1], SamplingParams(max_tokens=12, temperature=0.7, seed=99, ignore_eos=True), 0.0))
    assert other != a[1]
    # every sampled token can be re-derived from the plain logits and the same noise
    cfg, weights = plain.read_model_folder(folder, torch.float64)
    tokens = list(prompts[0])
    for d, tok in enumerate(a[0]):
        logits = plain.forward_logits(cfg, weights, tokens)[-1]
        score = (logits / 0.7).numpy() + gumbel_noise(1234, d, config.vocab_size)
        assert score[tok] >= score.max() - 1e-3
        tokens.append(tok)


def test_command_line(model_folders, tmp_path):
    folder, config, page = model_folders["A"]
    prompt = random_tokens(config.vocab_size, 9, 8)
    cmd = [sys.executable, "-m", "slipstream_b200.entrypoints.cli", "--model", folder, "--dtype", "float32",
           "--block-size", str(page), "--num-gpu-blocks", "32", "--prompt-ids", ",".join(map(str, prompt)),
           "--max-tokens", "6", "--temperature", "0", "--ignore-eos"]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=str(ROOT), timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    record = json.loads(proc.stdout.strip().splitlines()[-1])
    cfg, weights = plain.read_model_folder(folder, torch.float64)
    assert record["output_token_ids"] == plain.generate_greedy(cfg, weights, prompt, 6) and record["finish_reason"] == "length"
    # the random-weights mode of the command line writes a loadable folder
    src = tmp_path / "cfg.json"
    src.write_text(json.dumps(config.to_dict()))
    out = tmp_path / "made"
    proc = subprocess.run([sys.executable, "-m", "slipstream_b200.entrypoints.cli", "--model", str(out),
                           "--write-random-model", str(src), "--seed", "5"], capture_output=True, text=True, cwd=str(ROOT))
    assert proc.returncode == 0 and (out / "model.safetensors").is_file() and (out / "config.json").is_file()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_that_run_ahead_of_the_host_give_the_same_tokens(model_folders, dtype):
    """Decode steps are launched before the tokens of the step before reach the host.  With requests of
    different lengths, a stop token that arrives while the next step already runs, sampling with a penalty
    and a request that joins late, the tokens are those of the engine that waits for every token."""
    from slipstream_b200 import SamplingParams
    from slipstream_b200.engine.llm_engine import Request
    folder, config, page = model_folders["B"]
    prompts = [random_tokens(config.vocab_size, n, 90 + n) for n in (3, 21, 38, 9)]
    probe = make_engine(folder, page, dtype=dtype)
    probe.run_ahead = False
    free = probe.generate(Request("p", None, prompts[1], SamplingParams(max_tokens=20, temperature=0.0, ignore_eos=True), 0.0))
    stop = free[7]  # request 1 stops at the first place where this token appears
    params = [SamplingParams(max_tokens=25, temperature=0.0, ignore_eos=True),
              SamplingParams(max_tokens=20, temperature=0.0, ignore_eos=True, stop_token_ids=[stop]),
              SamplingParams(max_tokens=9, temperature=0.9, top_k=12, top_p=0.9, repetition_penalty=1.3, seed=5, ignore_eos=True),
              SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)]

    def run(ahead):
        engine = make_engine(folder, page, dtype=dtype)
        engine.run_ahead = ahead
        seqs = [engine.add_request(Request(f"r{i}", None, p, s, float(i))) for i, (p, s) in enumerate(zip(prompts[:3], params[:3]))]
        steps = 0
        while engine.scheduler.has_work() and steps < 500:
            if steps == 6:  # joins while the others decode
                seqs.append(engine.add_request(Request("late", None, prompts[3], params[3], 9.0)))
                seqs.append(engine.add_request(Request("late2", None, prompts[0], params[2], 9.5)))
            engine.step()
            steps += 1
        engine.drain()
        assert engine.runner.cache.min_free_pages() == 64 and not engine.scheduler.has_work()
        engine.runner.cache.check_invariants()
        engine.runner.check()
        return [list(s.output_token_ids) for s in seqs], [s.status for s in seqs]

    want, want_status = run(False)
    got, got_status = run(True)
    assert got == want and got_status == want_status
    assert want[1][-1] == stop and len(want[1]) <= 8 and all(t >= 0 for out in got for t in out)
    assert list(map(len, want)) == [25, len(want[1]), 9, 1, 9]


def test_warm_up_captures_every_decode_graph_before_the_first_request(model_folders):
    from slipstream_b200 import SamplingParams
    from slipstream_b200.engine.llm_engine import Request
    folder, config, page = model_folders["A"]
    engine = make_engine(folder, page, dtype="bfloat16", max_num_seqs=6)
    made = engine.warm_up()
    assert made == len(engine.runner._graphs) >= 4  # buckets 1, 2, 4, 8 hold up to 6 requests
    prompts = [random_tokens(config.vocab_size, n, 5 + n) for n in (4, 9, 2, 7, 5)]
    params = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    outs = engine.generate_batch([Request(f"r{i}", None, p, params, float(i)) for i, p in enumerate(prompts)])
    assert len(engine.runner._graphs) == made, "no graph was captured while requests ran"
    cfg, weights = plain.read_model_folder(folder, torch.float64)
    for prompt, out in zip(prompts, outs):
        greedy_is_consistent(cfg, weights, prompt, out, slack=3e-2)
