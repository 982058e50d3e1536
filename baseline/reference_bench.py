"""The reference arm of bench.py: the UNMODIFIED reference engine (an offline ``pip install --no-deps --target
baseline/_ref`` of the reference checkout) run through its own public API, ``LLMEngine(EngineConfig).generate_batch``,
on the same model shape, batch, prompt length and random weights as this repository's arm.

None of this repository's models, kernels or engine is on that path; only its random-weights writer is used,
to make the model folder the reference loads (plus a one-word ``tokenizer.json``, which the reference insists
on).  Decode throughput is the difference between two ``generate_batch`` calls that differ by K generated
tokens, so that the prompt phase cancels; the step the reference runs is its stock one (eager attention over
gathered pages, one forward for the decodes, one forward per prompt portion).
"""

from __future__ import annotations

import os
import sys
import tempfile
import time


def _model_folder(shape: dict, layers: int) -> str:
    """A model folder with random weights of the shape, cached under the temporary directory."""
    root = os.path.join(tempfile.gettempdir(), f"slipstream_ref_model_{shape['hidden_size']}_{layers}_{os.getuid()}")
    if os.path.isfile(os.path.join(root, "model.safetensors")) and os.path.isfile(os.path.join(root, "tokenizer.json")):
        return root
    from slipstream_b200.config.model_config import Qwen2Config
    from slipstream_b200.weights.random_init import write_random_model

    config = Qwen2Config.from_dict(dict(shape, num_hidden_layers=layers, model_type="qwen2"))
    write_random_model(config, root, seed=0)
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel

    Tokenizer(WordLevel({"a": 0}, unk_token="a")).save(os.path.join(root, "tokenizer.json"))
    return root


def run_reference(args, shape: dict, ref_path: str) -> dict:
    sys.path.insert(0, ref_path)
    try:
        import numpy as np
        import torch
        from slipstream.core.config import CacheConfig, EngineConfig, ModelConfig, SchedulerConfig
        from slipstream.core.sampling_params import SamplingParams
        from slipstream.core.types import Request
        from slipstream.engine.llm_engine import LLMEngine
    except Exception as exc:  # the install is there but does not import here
        return {"impl": "reference", "unavailable": f"the reference does not import: {type(exc).__name__}: {exc}"[:200]}
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device"}

    layers = args.layers
    folder = _model_folder(shape, layers)
    batch, prompt_len, steps, warm = args.batch, args.prompt_len, args.steps, max(3, args.warmup)
    blocks = batch * (prompt_len + steps + warm + 64) // 16 + 64
    config = EngineConfig(
        model=ModelConfig(model_id=folder, dtype="bfloat16", max_model_len=args.context_len),
        cache=CacheConfig(block_size=16, num_gpu_blocks=blocks, enable_prefix_caching=False),
        scheduler=SchedulerConfig(max_num_seqs=max(batch, 8), max_num_batched_tokens=8192))
    engine = LLMEngine(config)
    rng = np.random.default_rng(0)
    vocab = shape["vocab_size"]

    def run(new_tokens: int) -> float:
        reqs = [Request(request_id=f"r{i}", prompt=None, prompt_token_ids=rng.integers(0, vocab, prompt_len).tolist(),
                        sampling_params=SamplingParams(max_tokens=new_tokens, temperature=0.0, ignore_eos=True),
                        arrival_ts=float(i) * 1e-6) for i in range(batch)]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = engine.generate_batch(reqs)
        torch.cuda.synchronize()
        assert all(len(o) == new_tokens for o in outs), [len(o) for o in outs]
        return time.perf_counter() - t0

    run(1 + warm)  # warm-up: allocator, library handles
    short = min(run(1 + warm) for _ in range(2))
    long = min(run(1 + warm + steps) for _ in range(2))
    ms_step = (long - short) * 1e3 / steps
    # prefill of one 2,048-token prompt (the reference cuts it into portions of 256 by default)
    engine.generate_batch([Request("p0", None, rng.integers(0, vocab, 2048).tolist(),
                                   SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True), 0.0)])
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    engine.generate_batch([Request("p1", None, rng.integers(0, vocab, 2048).tolist(),
                                   SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True), 0.0)])
    torch.cuda.synchronize()
    prefill_ms = (time.perf_counter() - t0) * 1e3
    return {
        "impl": "reference",
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2048 tokens (Qwen2.5-7B bf16)",
        "value": round(batch * 1000.0 / ms_step, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warm,
        "ms_per_step": round(ms_step, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random token ids, random-init weights N(0, 0.02)",
        "config": {"model": "Qwen2.5-7B shape", "global_batch": batch, "seq_len": prompt_len, "context_len": args.context_len,
                   "parallelism": "single GPU", "layers": layers, "layers_of_model": shape["num_hidden_layers"],
                   "kv_block": 16, "timing": "host clock around generate_batch, difference of two lengths"},
        # generate_batch takes token lists from the host and returns token lists: per decode step one new token id
        # per request comes back (the engine reads its arg-max with .tolist()) and goes in again (a [B, 1] tensor
        # built from Python lists), 8 bytes each as the reference's int64 tensors
        "e2e": {"value": round(batch * 1000.0 / ms_step, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": 8 * batch, "d2h_bytes_per_step": 8 * batch},
        "prefill": {"value": round(2048 * 1000.0 / prefill_ms, 1), "tokens": 2048, "ms": round(prefill_ms, 2)},
    }
