"""Schedules and failure paths of the engine that the replay tests do not reach: preemption by recompute in
bfloat16 under the TMA-fed decode kernel with a seeded sampling chain; a mixed step whose prefill attention cuts
the keys into parts while other requests bring one to three tokens; a token budget smaller than the number of
decoding requests; the text path (tokenizer.json, stop strings); an error word set on the host; and mutations of
the cache (a block-table entry that names the wrong page, a layer given another layer's pages) that the comparisons must notice."""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
import replay_plans as plans
from conftest import ROOT, random_tokens, sharpen
from test_replay_gpu import TOLERANCE, compare, oracle, run_plan

pytestmark = pytest.mark.gpu


def write_model(folder, seed=5, factor=4.0, **sizes):
    from slipstream_b200.config.model_config import Qwen2Config
    from slipstream_b200.weights.random_init import write_random_model

    base = dict(vocab_size=300, hidden_size=128, num_hidden_layers=2, max_position_embeddings=4096,
                torch_dtype="bfloat16", intermediate_size=208, num_attention_heads=4, num_key_value_heads=2,
                head_dim=64, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=False)
    base.update(sizes)
    config = Qwen2Config(**base)
    write_random_model(config, folder, seed=seed)
    sharpen(folder, factor=factor)
    return config


def make_engine(folder, page, dtype, pages, **sched):
    from slipstream_b200 import CacheConfig, EngineConfig, SchedulerConfig
    from slipstream_b200.engine.llm_engine import LLMEngine

    return LLMEngine(EngineConfig.for_model(str(folder), dtype=dtype,
                                            cache=CacheConfig(block_size=page, num_gpu_blocks=pages),
                                            scheduler=SchedulerConfig(**sched)))


# --------------------------------------------------------------------------- preemption, bfloat16, head size 128
def test_preemption_by_recompute_in_bfloat16_with_a_seeded_sampling_chain(tmp_path):
    """Head size 128 and pages of 16 take the TMA-fed decode kernel, which writes the newest key and value to
    their page itself.  With too few pages the newest request is preempted, loses its pages, and later replays
    prompt and outputs as a prompt portion; its seen-token mask (repetition penalty) restarts from those tokens
    and its draws continue at the same index.  In bfloat16 a replayed key differs from the decoded one by its
    rounding, so the tokens need not equal those of an engine with room for everybody; every token of either
    engine must be the one the plain chain draws from the plain logits with the same noise (penalty over the
    request's own history, temperature, draw number = index of the output token), within the rounding of the
    logits."""
    from slipstream_b200 import SamplingParams, ops
    from slipstream_b200.engine.llm_engine import Request
    from test_generate_gpu import gumbel_noise

    config = write_model(tmp_path, head_dim=128, num_attention_heads=4, num_key_value_heads=2, hidden_size=256)
    assert ops.tcgen05_attention_fits(128, 4, 2, 16, 0)
    prompts = [random_tokens(config.vocab_size, n, 70 + n) for n in (40, 25, 33)]
    temperature, penalty, new = 0.8, 1.3, 24
    params = [SamplingParams(max_tokens=new, temperature=temperature, repetition_penalty=penalty, seed=1000 + i,
                             ignore_eos=True) for i in range(3)]

    def run(pages):
        engine = make_engine(tmp_path, 16, "bfloat16", pages, prefill_chunk_size=32)
        outs = engine.generate_batch([Request(f"r{i}", None, p, params[i], float(i)) for i, p in enumerate(prompts)])
        engine.runner.check()
        engine.runner.cache.check_invariants()
        assert engine.runner.cache.min_free_pages() == pages
        return outs, engine.scheduler.preemptions

    roomy, none = run(64)
    tight, preemptions = run(9)  # 144 token slots for 98 prompt + 72 new tokens
    assert none == 0 and preemptions >= 1
    cfg, weights = plain.read_model_folder(tmp_path, torch.float64)
    weights = {k: v.to(torch.bfloat16).to(torch.float64) if v.dim() == 2 else v for k, v in weights.items()}
    for what, outs in (("roomy", roomy), ("tight", tight)):
        for i, (prompt, out) in enumerate(zip(prompts, outs)):
            assert len(out) == new
            tokens = list(prompt)
            for d, tok in enumerate(out):
                logits = plain.forward_logits(cfg, weights, tokens)[-1]
                kept = plain.filtered_logits(logits, temperature=temperature, repetition_penalty=penalty, history=tokens)
                score = kept.numpy() + gumbel_noise(1000 + i, d, config.vocab_size)
                slack = 2 * 3e-2 * float(logits.abs().max()) / temperature
                assert score[tok] >= score.max() - slack, (what, i, d, tok, int(score.argmax()))
                tokens.append(tok)
    # the requests that were never preempted run the same kernels on the same values in both engines
    assert tight[0] == roomy[0]
    # the chain is not greedy in disguise: another seed gives other tokens
    other = make_engine(tmp_path, 16, "bfloat16", 64)
    again = other.generate(Request("x", None, prompts[0], SamplingParams(
        max_tokens=new, temperature=temperature, repetition_penalty=penalty, seed=77, ignore_eos=True), 0.0))
    assert again != roomy[0]


# --------------------------------------------------------------------------- key parts in a mixed step
def test_a_mixed_step_whose_prefill_attention_cuts_the_keys_into_parts(tmp_path):
    """The number of key parts of the tcgen05 prefill kernel comes from the longest request of the step; short
    requests and single tokens in the same step then get blocks whose part holds no key tile at all.  One
    request with 1,100 and later 2,300 cached tokens brings portions of 40 and 60 tokens beside requests that
    bring 1, 2 and 3 tokens; every row against the oracle."""
    from slipstream_b200 import ops
    from slipstream_b200.engine.runner import ModelRunner

    config = write_model(tmp_path, num_attention_heads=6, num_key_value_heads=2, hidden_size=96, intermediate_size=136,
                         vocab_size=211, tie_word_embeddings=True)
    requests = {"long": random_tokens(211, 2400, 4), "a": random_tokens(211, 30, 5), "b": random_tokens(211, 75, 6),
                "c": random_tokens(211, 9, 7)}
    want = oracle(str(tmp_path), requests, "bfloat16")
    runner = ModelRunner(str(tmp_path), dtype="bfloat16", page_size=16, num_pages=176, max_num_seqs=4)
    tile = 128 // 3
    assert ops.prefill_key_parts([40, 1, 3, 2], [1140, 21, 63, 8], tile, 2) == 2
    assert ops.prefill_key_parts([60, 1, 2], [2360, 24, 70], tile, 2) >= 4

    def entry(rid, at, n):
        return {"id": rid, "tokens": requests[rid][at:at + n], "want": list(range(n))}

    steps = [
        {"entries": [entry("long", 0, 1100)], "end": []},
        {"entries": [entry("a", 0, 20), entry("b", 0, 60), entry("c", 0, 6)], "end": []},
        {"entries": [entry("long", 1100, 40), entry("a", 20, 1), entry("b", 60, 3), entry("c", 6, 2)], "end": []},
        {"entries": [entry("long", 1140, 1160)], "end": []},
        {"entries": [entry("a", 21, 1), entry("long", 2300, 60), entry("b", 63, 2)], "end": []},
        {"entries": [entry("long", 2360, 40), entry("a", 22, 8), entry("b", 65, 10), entry("c", 8, 1)],
         "end": ["long", "a", "b", "c"]},
    ]
    rows = plans.collect(steps, run_plan(runner, steps))
    compare(rows, want, "bfloat16", "key parts beside short requests")


# --------------------------------------------------------------------------- a token budget below the decoders
@pytest.mark.parametrize("run_ahead", [True, False])
def test_fewer_batched_tokens_than_decoding_requests(model_folders, run_ahead):
    """Five requests decode under ``max_num_batched_tokens=3``: every step leaves somebody out, the steps that run
    ahead of the host must not be taken (they would feed all five), and everybody still gets the plain tokens."""
    from slipstream_b200 import SamplingParams
    from slipstream_b200.engine.llm_engine import Request

    folder, config, page = model_folders["A"]
    engine = make_engine(folder, page, "float32", 64, max_num_batched_tokens=3, prefill_chunk_size=3)
    engine.run_ahead = run_ahead
    prompts = [random_tokens(config.vocab_size, n, 30 + n) for n in (4, 7, 2, 9, 5)]
    params = SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True)
    seqs = [engine.add_request(Request(f"r{i}", None, p, params, float(i))) for i, p in enumerate(prompts)]
    most = 0
    while engine.step():
        most = max(most, engine.stats.num_batched_tokens)
        assert engine.stats.num_batched_tokens <= 3
    engine.drain()
    assert most == 3
    cfg, weights = plain.read_model_folder(folder, torch.float64)
    for prompt, seq in zip(prompts, seqs):
        assert seq.output_token_ids == plain.generate_greedy(cfg, weights, prompt, 10)
    assert engine.runner.cache.min_free_pages() == 64
    engine.runner.check()


# --------------------------------------------------------------------------- text in, text out
WORDS = ["<unk>"] + [f"<{i}>" for i in range(1, 256)]  # no word is part of another


def add_tokenizer(folder):
    """A word-level tokenizer over the tiny vocabulary: token i is the word ``<i>``; words are split at spaces and
    joined with spaces again."""
    from tokenizers import Tokenizer, pre_tokenizers
    from tokenizers.models import WordLevel

    tok = Tokenizer(WordLevel({w: i for i, w in enumerate(WORDS)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.save(str(folder) + "/tokenizer.json")


def test_text_prompts_stop_strings_and_output_text(model_folders, tmp_path):
    """slipstream/models/tokenizer.py:11-57 and slipstream/engine/llm_engine.py:223-234: a prompt given as text is
    encoded with the folder's tokenizer.json, the output is decoded into ``RequestOutput.text``, and generation
    stops as soon as the decoded output holds a stop string (the token that completed it stays)."""
    import shutil

    from slipstream_b200 import SamplingParams
    from slipstream_b200.engine.llm_engine import LLM

    folder, config, page = model_folders["A"]
    mine = tmp_path / "with_tokenizer"
    shutil.copytree(folder, mine)
    add_tokenizer(mine)
    llm = LLM(str(mine), dtype="float32", block_size=page, num_gpu_blocks=64)
    ids = random_tokens(config.vocab_size - 1, 11, 3)
    ids = [i + 1 for i in ids]  # no <unk>
    text = " ".join(WORDS[i] for i in ids)
    assert llm.engine.tokenize(type("R", (), {"prompt_token_ids": None, "prompt": text})()) == ids
    greedy = SamplingParams(max_tokens=9, temperature=0.0, ignore_eos=True)
    by_ids = llm.generate(prompt_token_ids=[ids], sampling_params=greedy)[0]
    by_text = llm.generate(prompts=[text], sampling_params=greedy)[0]
    assert by_text.output_token_ids == by_ids.output_token_ids and len(by_ids.output_token_ids) == 9
    assert by_text.text == " ".join(WORDS[t] for t in by_ids.output_token_ids)
    # a stop string that the fifth output token completes
    fifth = by_ids.output_token_ids[4]
    first = by_ids.output_token_ids.index(fifth)
    stopped = llm.generate(prompts=[text], sampling_params=SamplingParams(
        max_tokens=9, temperature=0.0, ignore_eos=True, stop_strings=(WORDS[fifth],)))[0]
    assert stopped.finish_reason == "stop" and stopped.output_token_ids == by_ids.output_token_ids[:first + 1]
    assert stopped.text.endswith(WORDS[fifth])
    # the command line takes the same
    proc = subprocess.run([sys.executable, "-m", "slipstream_b200.entrypoints.cli", "--model", str(mine), "--dtype",
                           "float32", "--block-size", str(page), "--num-gpu-blocks", "64", "--prompt", text,
                           "--max-tokens", "9", "--temperature", "0", "--ignore-eos", "--stop", WORDS[fifth]],
                          capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert proc.returncode == 0, proc.stderr[-2000:]
    record = json.loads(proc.stdout.strip().splitlines()[-1])
    assert record["output_token_ids"] == stopped.output_token_ids and record["text"] == stopped.text
    assert record["finish_reason"] == "stop"
    # without a tokenizer a text prompt and stop strings are refused with a sentence
    bare = LLM(folder, dtype="float32", block_size=page, num_gpu_blocks=64)
    with pytest.raises(ValueError, match="tokenizer.json"):
        bare.generate(prompts=[text], sampling_params=greedy)
    with pytest.raises(ValueError, match="tokenizer.json"):
        bare.generate(prompt_token_ids=[ids], sampling_params=SamplingParams(stop_strings=("<3>",)))


# --------------------------------------------------------------------------- the device error word reaches generate()
@pytest.mark.parametrize("run_ahead", [True, False])
def test_generation_raises_when_a_kernel_has_flagged_an_error(model_folders, run_ahead):
    """Kernels set bits of a device error word instead of trapping (a page or slot out of range, a bounded wait
    that gave up).  The word travels to the host behind the sampled tokens of every step; a non-zero word aborts
    what was running and raises.  The bit is set from the host here: nothing on the device goes wrong."""
    from slipstream_b200 import SamplingParams, ops
    from slipstream_b200.engine.llm_engine import Request

    folder, config, page = model_folders["A"]
    engine = make_engine(folder, page, "float32", 64)
    engine.run_ahead = run_ahead
    prompt = random_tokens(config.vocab_size, 12, 8)
    params = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)
    good = engine.generate(Request("ok", None, prompt, params, 0.0))
    seq = engine.add_request(Request("bad", None, prompt, params, 0.0))
    for _ in range(4):
        assert engine.step()
    ops.error_word(engine.runner.device).fill_(8)
    with pytest.raises(ops.KernelError, match="bounded wait"):
        for _ in range(4):
            engine.step()
        engine.drain()
    assert seq.is_finished and not engine.scheduler.has_work()
    assert engine.runner.cache.min_free_pages() == 64
    engine.runner.cache.check_invariants()
    assert int(ops.error_word(engine.runner.device).item()) == 0
    assert engine.generate(Request("after", None, prompt, params, 0.0)) == good  # the engine is usable again


# --------------------------------------------------------------------------- the comparisons have teeth
def worst_error(rows, ref):
    got = np.stack(rows)
    return float(np.abs(got - ref).max() / np.abs(ref).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_a_wrong_page_or_a_wrong_layers_pages_breaks_the_bound(model_folders, name, dtype):
    """What the replay tests would see if the cache went wrong: (1) an entry of a request's block table pointing at
    another of its pages between the prompt and its decode steps (merely swapping two entries would change
    nothing: keys are stored rotated, and attention does not care in which order it meets the pairs of key and
    value), (2) a layer reading and writing the pages of the layer before it.
    Either must push the error of the decoded rows far beyond the bound the replay tests allow, in float32 and
    in bfloat16; the same steps without the mutation stay within it."""
    from slipstream_b200.engine.runner import ModelRunner, StepEntry

    folder, config, page = model_folders[name]
    tokens = random_tokens(config.vocab_size, 90, 21)
    want = oracle(folder, {"r": tokens}, dtype)["r"]
    head = 70

    def decode_rows(mutate):
        runner = ModelRunner(folder, dtype=dtype, page_size=page, num_pages=64, max_num_seqs=2)
        if mutate == "layer":
            runner.model.bindings[1].kv = runner.model.bindings[0].kv
        runner.step([StepEntry("r", tokens[:head], [])])
        if mutate == "table":
            table = runner.cache.get("r").tables[0]
            table[1] = table[3]  # four (A) or eight (B) keys lost, as many met twice
        rows = [runner.step([StepEntry("r", [t], [0])]).cpu().numpy()[0] for t in tokens[head:]]
        runner.check()
        return rows

    bound = TOLERANCE[dtype]
    assert worst_error(decode_rows(None), want[head:]) <= bound
    for mutate in ("table", "layer"):
        err = worst_error(decode_rows(mutate), want[head:])
        assert err > 4 * bound, (mutate, err, bound)
