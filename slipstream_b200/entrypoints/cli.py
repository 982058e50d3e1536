"""Command line: generate from a model folder.

    python -m slipstream_b200.entrypoints.cli --model DIR --prompt-ids 1,2,3 --max-tokens 16

``--model`` has the meaning of the reference's only command line
(slipstream/entrypoints/api_server.py:242-252: a model folder; there it starts an
HTTP server, which is not built here).  The other options carry the names of the
reference's configuration fields (slipstream/core/config.py:25-134,
slipstream/core/sampling_params.py:16-28) with dashes for underscores.
``--write-random-model`` makes a model folder with random weights from a
config.json instead of generating.
"""

from __future__ import annotations

import argparse
import json
import sys


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="slipstream_b200", description="Qwen2.5 generation on one B200")
    p.add_argument("--model", required=True, help="folder with config.json and safetensors weights")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default=None)
    p.add_argument("--max-model-len", type=int, default=None)
    p.add_argument("--load-format", choices=["safetensors", "random"], default="safetensors")
    p.add_argument("--seed", type=int, default=0, help="engine seed (random weights, unseeded requests)")
    # cache
    p.add_argument("--block-size", type=int, default=16)
    p.add_argument("--num-gpu-blocks", type=int, default=None)
    p.add_argument("--gpu-memory-utilization", type=float, default=0.90)
    # scheduler
    p.add_argument("--max-num-seqs", type=int, default=256)
    p.add_argument("--max-num-batched-tokens", type=int, default=8192)
    p.add_argument("--prefill-chunk-size", type=int, default=256)
    p.add_argument("--disable-chunked-prefill", action="store_true")
    # request
    p.add_argument("--prompt", action="append", default=None, help="text prompt (needs tokenizer.json); repeatable")
    p.add_argument("--prompt-ids", action="append", default=None, help="comma-separated token ids; repeatable")
    p.add_argument("--max-tokens", type=int, default=16)
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--top-k", type=int, default=-1)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--min-p", type=float, default=0.0)
    p.add_argument("--repetition-penalty", type=float, default=1.0)
    p.add_argument("--stop-token-ids", default="", help="comma-separated token ids")
    p.add_argument("--stop", action="append", default=None,
                   help="stop string (needs tokenizer.json); generation ends once the output text holds it; repeatable")
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--sample-seed", type=int, default=None, help="SamplingParams.seed")
    # random-weights folder
    p.add_argument("--write-random-model", metavar="CONFIG_JSON", default=None,
                   help="write config.json + model.safetensors with random weights into --model and exit")
    return p


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    if args.write_random_model:
        from slipstream_b200.config.model_config import read_json
        from slipstream_b200.registry import resolve_architecture
        from slipstream_b200.weights.random_init import write_random_model
        from pathlib import Path

        data = read_json(Path(args.write_random_model))
        config = resolve_architecture(data).config_class.from_dict(data)
        out = write_random_model(config, args.model, seed=args.seed, dtype=args.dtype)
        print(f"wrote {out}")
        return 0

    from slipstream_b200 import SamplingParams
    from slipstream_b200.engine.llm_engine import LLM

    prompts_ids = [[int(t) for t in s.split(",") if t.strip()] for s in (args.prompt_ids or [])]
    if not prompts_ids and not args.prompt:
        print("give --prompt-ids or --prompt", file=sys.stderr)
        return 2
    if prompts_ids and args.prompt:
        print("give either --prompt-ids or --prompt, not both", file=sys.stderr)
        return 2
    params = SamplingParams(
        max_tokens=args.max_tokens, temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
        min_p=args.min_p, repetition_penalty=args.repetition_penalty,
        stop_token_ids=tuple(int(t) for t in args.stop_token_ids.split(",") if t.strip()),
        stop_strings=tuple(args.stop or ()), ignore_eos=args.ignore_eos, seed=args.sample_seed)
    llm = LLM(args.model, dtype=args.dtype, max_model_len=args.max_model_len, block_size=args.block_size,
              num_gpu_blocks=args.num_gpu_blocks, gpu_memory_utilization=args.gpu_memory_utilization,
              max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens,
              prefill_chunk_size=args.prefill_chunk_size,
              enable_chunked_prefill=not args.disable_chunked_prefill, seed=args.seed,
              load_format=args.load_format)
    if prompts_ids:
        outs = llm.generate(prompt_token_ids=prompts_ids, sampling_params=params)
    else:
        outs = llm.generate(prompts=args.prompt, sampling_params=params)
    for out in outs:
        print(json.dumps({"request_id": out.request_id, "output_token_ids": out.output_token_ids,
                          "finish_reason": out.finish_reason, "text": out.text}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
