"""Decode and prefill throughput of the Qwen2.5-7B shape (random weights, bfloat16) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl reference]

Prints ONE JSON line.  ``value`` is decoded tokens a second at the given batch (a step = one decode
step of the whole batch through the step function, timed on the device with CUDA events); ``e2e`` is
the same through the public engine calls (``add_request`` / ``step``) with host token ids in and
out every step; ``prefill`` is one 2,048-token prompt in one step; ``roofline`` compares the bytes a
decode step must read (every weight once, plus the cache of the live requests) with the measured
copy bandwidth; ``points`` holds decode at batch 1 and 64; ``kernels`` each dominant kernel alone at the
bench shape with its own roofline fraction.  Peaks come from MEASURED_PEAKS.json
beside this file when present.  One GPU only: for --gpus above 1 it says so and exits with 2.

``--only decode|prefill`` runs one part and prints a short line (profiling, and measurements beside the
headline): ``--only decode --batch 1 --prompt-len 32000 --context-len 32768`` is a decode step behind a long
context, ``--only prefill --chunk 512 --prefix 8192 --context-len 32768`` a prompt portion behind cached tokens.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen2.5-7B layer sizes (BASELINE.json configs[2])
SHAPE_7B = dict(vocab_size=152064, hidden_size=3584, num_hidden_layers=28, intermediate_size=18944,
                num_attention_heads=28, num_key_value_heads=4, head_dim=128, rms_norm_eps=1e-6,
                rope_theta=1000000.0, tie_word_embeddings=False, max_position_embeddings=8192,
                torch_dtype="bfloat16")
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

# The other measured workloads of BASELINE.json (configs[3] and configs[4]): end to end through the scheduler.
WORKLOADS = {
    "0.5b-mixed": dict(
        shape=dict(vocab_size=151936, hidden_size=896, num_hidden_layers=24, intermediate_size=4864,
                   num_attention_heads=14, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6,
                   rope_theta=1000000.0, tie_word_embeddings=True, max_position_embeddings=8192, torch_dtype="bfloat16"),
        requests=64, prompt=(16, 2048), new_tokens=128, chunk=512),
    "14b": dict(
        shape=dict(vocab_size=152064, hidden_size=5120, num_hidden_layers=48, intermediate_size=13824,
                   num_attention_heads=40, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5,
                   rope_theta=1000000.0, tie_word_embeddings=False, max_position_embeddings=8192, torch_dtype="bfloat16"),
        requests=32, prompt=(2048, 2048), new_tokens=256, chunk=2048),
}


def run_workload(name: str, args) -> int:
    """Generate through ``LLMEngine.generate_batch`` (scheduler, chunked prefill, continuous batching) and print
    one JSON line with the end-to-end token rates."""
    import numpy as np
    import torch

    from slipstream_b200 import CacheConfig, EngineConfig, SamplingParams, SchedulerConfig
    from slipstream_b200.engine.llm_engine import LLMEngine, Request

    w = WORKLOADS[name]
    folder = tempfile.mkdtemp(prefix=f"bench_{name}_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(w["shape"], architectures=["Qwen2ForCausalLM"], model_type="qwen2"), f)
    rng = np.random.default_rng(0)
    lo, hi = w["prompt"]
    lengths = rng.integers(lo, hi + 1, w["requests"]).tolist()
    pages = sum((n + w["new_tokens"] + 15) // 16 + 1 for n in lengths) + 64
    engine = LLMEngine(EngineConfig.for_model(
        folder, dtype="bfloat16", load_format="random", max_model_len=8192,
        cache=CacheConfig(block_size=16, num_gpu_blocks=pages),
        scheduler=SchedulerConfig(max_num_seqs=w["requests"], max_num_batched_tokens=8192, prefill_chunk_size=w["chunk"])))
    vocab = w["shape"]["vocab_size"]

    def requests(tag: str, new_tokens: int):
        return [Request(f"{tag}{i}", None, rng.integers(0, vocab, n).tolist(),
                        SamplingParams(max_tokens=new_tokens, temperature=0.0, ignore_eos=True), float(i) * 1e-6)
                for i, n in enumerate(lengths)]

    # warm-up: the same workload once, so that kernels are compiled and a graph is captured for every batch
    # bucket the run passes through while its requests finish (a capture inside the timed run costs tens of ms)
    engine.generate_batch(requests("w", w["new_tokens"]))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = engine.generate_batch(requests("r", w["new_tokens"]))
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    assert all(len(o) == w["new_tokens"] for o in outs)
    generated, prompt_tokens = w["requests"] * w["new_tokens"], int(sum(lengths))
    print(json.dumps({"workload": name, "requests": w["requests"], "prompt_tokens": prompt_tokens,
                      "generated_tokens": generated, "seconds": round(seconds, 3),
                      "generated_tokens_per_s": round(generated / seconds, 1),
                      "total_tokens_per_s": round((generated + prompt_tokens) / seconds, 1),
                      "steps": engine.stats.step, "preemptions": engine.scheduler.preemptions,
                      "layers": w["shape"]["num_hidden_layers"], "dtype": "bf16", "data": "synthetic"}))
    return 0


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.samples: list[list[str]] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self) -> None:
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def __exit__(self, *exc) -> None:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = sorted(int(float(s[0])) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(float(self.samples[0][1])), "reasons": reasons,
                "samples": len(mhz)}


def reference_arm(args) -> int:
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "slipstream")):
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is not installed under baseline/_ref (pip install --no-deps --target baseline/_ref <reference>)"}))
        return 0
    from baseline.reference_bench import run_reference  # noqa: E402

    try:
        line = run_reference(args, SHAPE_7B, ref)
    except Exception as exc:  # the reference ran and failed: say so in one line instead of a traceback
        line = {"impl": "reference", "unavailable": f"the reference failed here: {type(exc).__name__}: {exc}"[:240]}
    print(json.dumps(line))
    return 0


def kernel_fractions(engine, batch: int, ctx_tokens: int, prefill_tokens: int, pk: dict) -> dict:
    """Each dominant kernel alone at the bench shape, timed with CUDA events: the decode projections and the
    decode attention against the bytes they must read (measured copy bandwidth), the prefill projections and the
    prefill attention against their flops (measured bf16 peak).  A kernel runs once per layer of the model, on that
    layer's own weights and pages, back to back as inside a step (28 x 33 MB of q/k/v weights and 28 x 17 MB of
    pages are larger than L2, so every launch reads from memory); median of five such sweeps, per launch."""
    import torch

    from slipstream_b200 import ops

    runner = engine.runner
    c = runner.config
    dev = runner.device
    blocks = runner.model.blocks
    gen = torch.Generator(device=dev).manual_seed(1)

    def rand(rows: int, cols: int) -> torch.Tensor:
        return (torch.randn(rows, cols, generator=gen, device=dev) * 0.5).to(torch.bfloat16)

    def sweep(run, layers: int | None = None) -> float:
        """Median microseconds per launch of ``run(layer)`` over ``layers`` layers (default: all).  The tensor-core
        kernels are timed as a burst, like the peak they are compared with: sweeps of a few launches, so that the
        GPU does not reach its power cap (a 2,048-token down projection takes 199 us in a burst and 238 us in
        the middle of thousands of launches)."""
        n = min(layers or len(blocks), len(blocks))
        torch.cuda.synchronize()
        if layers is not None:
            time.sleep(0.2)  # whatever ran before may have left the GPU at its power cap: let the clocks come back
        for layer in range(n):
            run(layer)
        times = []
        for _ in range(5):
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for layer in range(n):
                run(layer)
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) * 1e3 / n)
        return sorted(times)[len(times) // 2]

    h, qkv_w = c.hidden_size, (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim
    o_in, inter = c.num_attention_heads * c.head_dim, c.intermediate_size
    out: dict[str, dict] = {}

    def hbm(name: str, us: float, nbytes: float) -> None:
        gbs = nbytes / (us * 1e-6) / 1e9
        out[name] = {"us": round(us, 2), "gbs": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 3)}

    def tensor(name: str, us: float, flops: float) -> None:
        tf = flops / (us * 1e-6) / 1e12
        out[name] = {"us": round(us, 2), "tflops": round(tf, 1), "frac": round(tf / pk["bf16_tflops"], 3)}

    for tokens, tag in ((batch, "decode"), (prefill_tokens, "prefill")):
        x_h, x_o, x_i = rand(tokens, h), rand(tokens, o_in), rand(tokens, inter)
        shapes = {
            "qkv": (lambda i: ops.linear(x_h, blocks[i].mixer.qkv_weight, blocks[i].mixer.qkv_b), h, qkv_w),
            "o": (lambda i: ops.linear(x_o, blocks[i].mixer.o_weight, None), o_in, h),
            "gate_up": (lambda i: ops.gate_up_swiglu(x_h, blocks[i].feed_forward.gate_up, None,
                                                     blocks[i].feed_forward.block), h, 2 * inter),
            "down": (lambda i: ops.linear(x_i, blocks[i].feed_forward.down, None), inter, h),
        }
        for name, (run, k, n) in shapes.items():
            us = sweep(run, None if tag == "decode" else 8)
            if tag == "decode":
                hbm(f"decode_{name}", us, 2.0 * k * n + 2.0 * tokens * (k + n))
            else:
                tensor(f"prefill_{name}", us, 2.0 * tokens * k * n)
    # LM head: one weight, larger than L2 by itself
    x_rows = rand(batch, h)
    head = runner.model.lm_head
    us = sweep(lambda i: head.forward(x_rows))
    hbm("decode_lm_head", us, 2.0 * c.vocab_size * h + 4.0 * batch * c.vocab_size)

    # attention over the engine's own pages: `batch` requests of `ctx_tokens` cached tokens (what the pages hold
    # does not matter for the time), decode (one token each) and prefill (one request, all tokens new)
    page = runner.cache.page_size
    n_q, n_kv, d = c.num_attention_heads, c.num_key_value_heads, c.head_dim
    kv = runner.store.kv[0]

    def tables(n_req: int, tokens: int) -> torch.Tensor:
        per = (tokens + page - 1) // page
        return torch.arange(n_req * per, dtype=torch.int32, device=dev).view(n_req, per)

    qkv = rand(batch, (n_q + 2 * n_kv) * d)
    att = torch.empty(batch, n_q * d, dtype=torch.bfloat16, device=dev)
    table = tables(batch, ctx_tokens)
    q_start = torch.arange(batch + 1, dtype=torch.int32, device=dev)
    lens = torch.full((batch,), ctx_tokens, dtype=torch.int32, device=dev)
    slices = ops.decode_slices(batch, n_kv, n_q // n_kv, ctx_tokens, False, ops.sm_count(dev))
    us = sweep(lambda i: ops.paged_attention_decode(qkv, qkv.shape[1], att, kv[i], table, q_start, lens, batch, n_q, n_kv,
                                                    d, d ** -0.5, 0, slices))
    hbm("decode_attention", us, batch * ctx_tokens * 2.0 * n_kv * d * 2 + 2.0 * batch * n_q * d * 2)
    if ops.tcgen05_attention_fits(d, n_q, n_kv, page, 0):
        import numpy as np
        from slipstream_b200.engine.context import query_tiles_longest_first_host

        T, tile = prefill_tokens, 128 // (n_q // n_kv)
        qkv_p = rand(T, (n_q + 2 * n_kv) * d)
        att_p = torch.empty(T, n_q * d, dtype=torch.bfloat16, device=dev)
        req, tok0 = (torch.from_numpy(a).to(dev) for a in query_tiles_longest_first_host(
            np.asarray([T], dtype=np.int32), np.asarray([T], dtype=np.int32), tile))
        table_p = tables(1, T)
        q_start_p = torch.tensor([0, T], dtype=torch.int32, device=dev)
        lens_p = torch.tensor([T], dtype=torch.int32, device=dev)
        us = sweep(lambda i: ops.paged_attention_prefill_tcgen05(qkv_p, qkv_p.shape[1], att_p, kv[i], table_p, req, tok0,
                                                                 q_start_p, lens_p, n_q, n_kv, d, d ** -0.5, 1), 8)
        tensor("prefill_attention", us, 4.0 * n_q * d * (T * (T + 1) // 2))
    return out


def kernel_tables(which: str) -> int:
    """``--only gemm``: this package's tcgen05 products against the library product at prompt-portion sizes
    (microseconds a launch, CUDA events, weights rotated so that they come from memory).  ``--only attention``: the
    tcgen05 prefill attention at several (queries, keys), with the number of key parts the engine would choose."""
    import numpy as np
    import torch

    from slipstream_b200 import ops
    from slipstream_b200.engine.context import query_tiles_longest_first_host

    dev = torch.device("cuda:0")

    def timed(fn, n: int = 16) -> float:
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(n):
            fn(i)
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) * 1e3 / n

    if which == "gemm":
        shapes = (("7b q/k/v", 4608, 3584), ("7b o", 3584, 3584), ("7b down", 3584, 18944), ("7b gate/up", 37888, 3584),
                  ("0.5b q/k/v", 1152, 896), ("0.5b gate/up", 9728, 896), ("0.5b down", 896, 4864),
                  ("14b down", 5120, 13824), ("14b q/k/v", 7168, 5120))
        for name, features, k in shapes:
            copies = max(2, min(8, int(300e6 // (features * k * 2))))
            ws = [(torch.randn(features, k, device=dev) * 0.02).bfloat16() for _ in range(copies)]
            for tokens in (128, 256, 512, 1024, 2048, 4096):
                x = torch.randn(tokens, k, device=dev).bfloat16()
                row = {"library": timed(lambda i: torch.mm(x, ws[i % copies].t()))}
                for width in (64, 128, 256):
                    if width <= features and tokens <= 1024:
                        row[f"one-SM {width}"] = timed(lambda i: ops.gemm_tcgen05(x, ws[i % copies], plan=(False, width, 1)))
                row["two-SM"] = timed(lambda i: ops.gemm_tcgen05_many(x, ws[i % copies]))
                print(json.dumps({"shape": name, "features": features, "k": k, "tokens": tokens,
                                  **{key: round(v, 1) for key, v in row.items()}}), flush=True)
        ops.check_errors(dev)
        return 0

    n_q, n_kv, d, page = SHAPE_7B["num_attention_heads"], SHAPE_7B["num_key_value_heads"], SHAPE_7B["head_dim"], 16
    tile = 128 // (n_q // n_kv)
    for queries, keys in ((2048, 2048), (2048, 8192), (8192, 8192), (1024, 1024), (512, 4096), (64, 4096)):
        pages = keys // page + 4
        copies = max(2, min(16, int(300e6 // (pages * 2 * n_kv * page * d * 2))))
        kvs = [torch.randn(pages, 2, n_kv, page, d, device=dev).bfloat16() for _ in range(copies)]
        qkv = torch.randn(queries, (n_q + 2 * n_kv) * d, device=dev).bfloat16()
        out = torch.empty(queries, n_q * d, device=dev, dtype=torch.bfloat16)
        q_lens, seq_lens = np.asarray([queries], dtype=np.int32), np.asarray([keys], dtype=np.int32)
        req, tok0 = (torch.from_numpy(a).to(dev) for a in query_tiles_longest_first_host(q_lens, seq_lens, tile))
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, -1)
        q_start = torch.tensor([0, queries], dtype=torch.int32, device=dev)
        lens = torch.tensor([keys], dtype=torch.int32, device=dev)
        parts = ops.prefill_key_parts(q_lens, seq_lens, tile, n_kv)
        us = timed(lambda i: ops.paged_attention_prefill_tcgen05(qkv, qkv.shape[1], out, kvs[i % copies], table, req, tok0,
                                                                 q_start, lens, n_q, n_kv, d, d ** -0.5, parts), 20)
        flops = 4.0 * n_q * d * sum(min(keys, keys - queries + t + 1) for t in range(queries))
        print(json.dumps({"queries": queries, "keys": keys, "key_parts": parts, "us": round(us, 1),
                          "tflops": round(flops / us / 1e6, 1)}), flush=True)
    ops.check_errors(dev)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=SHAPE_7B["num_hidden_layers"])
    ap.add_argument("--context-len", type=int, default=SHAPE_7B["max_position_embeddings"],
                    help="positions of the model (with --only: measurements at longer contexts)")
    ap.add_argument("--chunk", type=int, default=2048, help="--only prefill: tokens of the timed prompt portion")
    ap.add_argument("--prefix", type=int, default=0, help="--only prefill: tokens already cached in front of it")
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 points")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel timings")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=None,
                    help="run another measured workload end to end through the scheduler instead")
    ap.add_argument("--only", choices=["decode", "prefill", "gemm", "attention"], default=None,
                    help="run just this part and print a short line (for profiling); gemm / attention: tables of "
                         "single kernels at several sizes")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU only (this engine uses a single device); got --gpus {args.gpus}")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.workload:
        return run_workload(args.workload, args)
    if args.only in ("gemm", "attention"):
        return kernel_tables(args.only)
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np
    import torch

    from slipstream_b200 import CacheConfig, EngineConfig, SamplingParams, SchedulerConfig, ops
    from slipstream_b200.engine.llm_engine import LLMEngine, Request
    from slipstream_b200.engine.runner import StepEntry

    pk, pk_kind = peaks()
    shape = dict(SHAPE_7B, num_hidden_layers=args.layers, max_position_embeddings=args.context_len)
    folder = tempfile.mkdtemp(prefix="bench_qwen7b_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(shape, architectures=["Qwen2ForCausalLM"], model_type="qwen2"), f)
    ctx_len, page = shape["max_position_embeddings"], 16
    max_batch = max(64, args.batch)
    pages = max_batch * (args.prompt_len + args.steps + args.warmup + 2 * max_batch + 96) // page + 4096 // page + 64
    if args.only:  # one batch, or one prompt behind a prefix: the pool need not hold 64 requests
        pages = (max(args.batch * (args.prompt_len + args.steps + args.warmup + 16), args.prefix + args.chunk) + 4096) // page + 64
    engine = LLMEngine(EngineConfig.for_model(
        folder, dtype="bfloat16", load_format="random", max_model_len=ctx_len,
        cache=CacheConfig(block_size=page, num_gpu_blocks=pages),
        scheduler=SchedulerConfig(max_num_seqs=max_batch, max_num_batched_tokens=8192, prefill_chunk_size=2048),
        seed=0, use_cuda_graphs=not args.no_graphs))
    runner = engine.runner
    vocab = shape["vocab_size"]
    rng = np.random.default_rng(0)
    torch.cuda.synchronize()

    def fill(batch: int, tag: str) -> list[str]:
        """Prefill ``batch`` requests of prompt_len random tokens (untimed)."""
        ids = [f"{tag}{i}" for i in range(batch)]
        if args.prompt_len > 4096:  # long prompts go in portions of 2,048 tokens
            for r in ids:
                for at in range(0, args.prompt_len, 2048):
                    runner.step([StepEntry(r, rng.integers(0, vocab, min(2048, args.prompt_len - at)).tolist(), [])])
            return ids
        per_step = max(1, 4096 // args.prompt_len)
        for i in range(0, batch, per_step):
            runner.step([StepEntry(r, rng.integers(0, vocab, args.prompt_len).tolist(), [])
                         for r in ids[i:i + per_step]])
        return ids

    def decode_device(batch: int, steps: int, warmup: int, tag: str) -> tuple[float, float, int]:
        """(tokens/s, ms per step, own kernel launches) of ``steps`` decode steps timed on the device."""
        ids = fill(batch, tag)
        feeds = rng.integers(0, vocab, (steps + warmup, batch)).tolist()
        for w in range(warmup):
            engine.sampler.greedy(runner.step([StepEntry(r, [feeds[w][j]], [0]) for j, r in enumerate(ids)]))
        torch.cuda.synchronize()
        launches0 = ops.launch_count()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for s in range(steps):
            engine.sampler.greedy(runner.step([StepEntry(r, [feeds[warmup + s][j]], [0]) for j, r in enumerate(ids)]))
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        launches = ops.launch_count() - launches0
        for r in ids:
            runner.release(r)
        return batch * 1000.0 / ms, ms, launches

    def decode_bytes(batch: int, steps: int, warmup: int) -> float:
        mean_ctx = args.prompt_len + warmup + (steps + 1) / 2
        return runner.weight_bytes_per_step() + batch * mean_ctx * runner.kv_bytes_per_token()

    if args.only == "decode":
        value, ms_step, launches = decode_device(args.batch, args.steps, args.warmup, "d")
        print(json.dumps({"only": "decode", "batch": args.batch, "tokens_per_s": round(value, 1),
                          "ms_per_step": round(ms_step, 4), "gpu_launches": launches}))
        return 0
    if args.only == "prefill":
        T = args.chunk
        all_ms = []
        for w in range(args.warmup + args.steps):
            for at in range(0, args.prefix, 2048):  # untimed: the tokens in front of the timed portion
                runner.step([StepEntry(f"p{w}", rng.integers(0, vocab, min(2048, args.prefix - at)).tolist(), [])])
            toks = rng.integers(0, vocab, T).tolist()
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            runner.step([StepEntry(f"p{w}", toks, [T - 1])])
            stop.record()
            torch.cuda.synchronize()
            runner.release(f"p{w}")
            all_ms.append(round(start.elapsed_time(stop), 3))
        print(json.dumps({"only": "prefill", "tokens": T, "prefix": args.prefix, "ms_last": all_ms[-1], "ms_each": all_ms}))
        return 0

    # ---- prefill of one 2,048-token prompt in one step (median of five).  It is the one phase that runs at the
    # power cap: single runs of the same step vary between 21.4 and 24.8 ms with the power management's state
    T = 2048
    # warm-up until the step of this shape has been captured as a graph (the runner does that once a shape has
    # come up `mixed_graph_after` times), so that the timed steps are what a running engine repeats
    for w in range(max(3, getattr(runner, "mixed_graph_after", 0) + 2)):
        runner.step([StepEntry(f"pw{w}", rng.integers(0, vocab, T).tolist(), [T - 1])])
        runner.release(f"pw{w}")
    torch.cuda.synchronize()

    def timed_prefill(tag: str, pause: float) -> list[float]:
        out = []
        for w in range(5):
            toks = rng.integers(0, vocab, T).tolist()
            if pause:
                time.sleep(pause)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            runner.step([StepEntry(f"{tag}{w}", toks, [T - 1])])
            stop.record()
            torch.cuda.synchronize()
            out.append(start.elapsed_time(stop))
            runner.release(f"{tag}{w}")
        return out

    # A step of 2,048 prompt tokens draws the full 1,000 W: back to back, the second or third step already runs at
    # the clock the power cap sustains (1.3 to 1.5 GHz instead of 1.97).  Both figures are taken, each against the
    # peak that was measured the same way: a step by itself after a pause (median of five) against the burst
    # rate of the matmul, and five steps back to back (median) against the rate sustained under the cap.
    times = timed_prefill("p", 0.3)
    sustained = timed_prefill("q", 0.0)
    prefill_ms = sorted(times)[len(times) // 2]
    sustained_ms = sorted(sustained)[len(sustained) // 2]
    c = runner.config
    per_token_matmul = sum(e for e in [
        2 * c.hidden_size * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim,
        2 * c.num_attention_heads * c.head_dim * c.hidden_size,
        2 * c.hidden_size * 2 * c.intermediate_size,
        2 * c.intermediate_size * c.hidden_size]) * c.num_hidden_layers
    attn_flops = 4 * c.num_attention_heads * c.head_dim * (T * (T + 1) // 2) * c.num_hidden_layers
    flops = T * per_token_matmul + attn_flops + 2 * c.hidden_size * c.vocab_size
    prefill = {"value": round(T * 1000.0 / prefill_ms, 1), "tokens": T, "ms": round(prefill_ms, 3),
               "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               "tflops": round(flops / (prefill_ms * 1e-3) / 1e12, 1), "peak_tflops": pk["bf16_tflops"],
               "ms_each": [round(t, 2) for t in times],
               "sustained": {"ms": round(sustained_ms, 3), "value": round(T * 1000.0 / sustained_ms, 1),
                             "frac": round(flops / (sustained_ms * 1e-3) / (pk.get("bf16_tflops_sustained", pk["bf16_tflops"]) * 1e12), 4),
                             "peak_tflops": pk.get("bf16_tflops_sustained", pk["bf16_tflops"]),
                             "ms_each": [round(t, 2) for t in sustained]}}

    # ---- headline: decode at --batch, device-timed, with clocks sampled
    with ClockSampler() as clocks:
        value, ms_step, launches = decode_device(args.batch, args.steps, args.warmup, "d")
    clock_summary = clocks.summary()
    achieved = decode_bytes(args.batch, args.steps, args.warmup) / (ms_step * 1e-3) / 1e9

    # ---- end to end through the public engine calls: host tokens in, host tokens out, every step
    for j in range(args.batch):
        engine.add_request(Request(f"e{j}", None, rng.integers(0, vocab, args.prompt_len).tolist(),
                                   # room for the steps during which later prompts are still being admitted: no
                                   # request may finish (and no smaller batch bucket appear) inside the timed loop
                                   SamplingParams(max_tokens=args.steps + args.warmup + 2 * args.batch + 16,
                                                  temperature=0.0, ignore_eos=True), float(j)))
    while any(s.num_output_tokens == 0 for s in engine.scheduler.running) or engine.scheduler.waiting:
        engine.step()
    # The prompts of all requests went in as one step of 8,192 tokens, which runs at the GPU's power cap; for some
    # tens of milliseconds afterwards the SM clock stays at 1.3 to 1.7 GHz and a decode step takes 3.5 ms instead
    # of 2.9.  The device-timed figure above is taken at full clocks, so this one waits until they are back.
    engine.drain()
    torch.cuda.synchronize()
    time.sleep(0.5)
    for _ in range(args.warmup):
        engine.step()
    engine.drain()  # the engine launches a decode step before it has read the tokens of the step before:
    torch.cuda.synchronize()  # nothing is in flight when the clock starts, and none when it stops
    t0 = time.perf_counter()
    for _ in range(args.steps):
        engine.step()
    engine.drain()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    h2d = engine.runner.last_h2d_bytes
    while engine.scheduler.has_work():
        engine.step()

    points = {}
    if not args.no_points:
        pts_steps = max(16, args.steps // 2)
        points["decode_b1"] = round(decode_device(1, pts_steps, 3, "a")[0], 1)
        points["decode_b64"] = round(decode_device(64, pts_steps, 3, "b")[0], 1)

    kernels = {} if args.no_kernels else kernel_fractions(engine, args.batch, args.prompt_len, 2048, pk)

    line = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2048 tokens (Qwen2.5-7B bf16)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random token ids, random-init weights N(0, 0.02)",
        "config": {"model": "Qwen2.5-7B shape", "global_batch": args.batch, "seq_len": args.prompt_len,
                   "context_len": ctx_len, "parallelism": "single GPU", "layers": c.num_hidden_layers,
                   "layers_of_model": SHAPE_7B["num_hidden_layers"], "hidden": c.hidden_size,
                   "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
                   "intermediate": c.intermediate_size, "vocab": c.vocab_size, "kv_block": page,
                   "l2": "inputs larger than L2 (weights read every step)", "cuda_graphs": not args.no_graphs,
                   "order": "prefill first, then decode", "peaks": pk_kind,
                   "prefill_timing": "each step by itself after 0.3 s idle, against the burst peak; sustained: five back to back, against the sustained peak",
                   "e2e_settle": "0.5 s idle between the prompt phase and the timed decode steps"},
        "e2e": {"value": round(args.batch * 1000.0 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "kernels": kernels,
        "clocks": clock_summary,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
