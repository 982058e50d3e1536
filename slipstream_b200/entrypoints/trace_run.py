"""Trace replay: drives the framework's own model runner (the loader, step function,
cache manager and kernels that generation uses) with token ids given from outside
and writes the logits.  It samples nothing and has no forward pass of its own.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

``--model``: a folder with config.json and model.safetensors; the model class is
chosen by config.json.  ``--dtype bfloat16`` uses the kernels and precisions that
serving uses; ``float32`` runs everything in true 32-bit.  ``--max-tokens N``: the
most tokens live requests hold at any time, each request's count rounded up to a
multiple of 64; the page pool is made for exactly this many, so pages are reused.

Standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch.  ``want`` lists the places among the
entry's tokens whose logits are asked for; ``end`` lists requests finished after
this step, whose pages and state slot are given back.  For a step in which
something is wanted, ``<out>/<step>.f32`` holds the logits as little-endian
float32 [wanted, vocab], in the order of the entries and of ``want``.  After every
step a line ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True)
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    parser.add_argument("--out", required=True)
    parser.add_argument("--max-tokens", type=int, required=True)
    parser.add_argument("--block-size", type=int, default=16, help="tokens per cache page (divides 64)")
    parser.add_argument("--max-num-seqs", type=int, default=8)
    args = parser.parse_args(argv)
    if args.max_tokens < 1:
        parser.error("--max-tokens must be >= 1")
    if 64 % args.block_size != 0:
        parser.error("--block-size must divide 64")

    import numpy as np

    from slipstream_b200.engine.runner import ModelRunner, StepEntry
    from slipstream_b200.registry import load_config

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    num_pages = (args.max_tokens + args.block_size - 1) // args.block_size
    # a trace may run a request past the checkpoint's max_position_embeddings, as far as the pool allows
    _, config = load_config(args.model)
    runner = ModelRunner(args.model, dtype=args.dtype, page_size=args.block_size, num_pages=num_pages,
                         max_num_seqs=args.max_num_seqs,
                         max_model_len=max(config.max_position_embeddings, num_pages * args.block_size))

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = [StepEntry(e["id"], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])])
                   for e in record.get("entries", [])]
        if entries:
            logits = runner.step(entries)
            if logits.shape[0]:
                host = logits.to("cpu").numpy().astype("<f4", copy=False)
                np.ascontiguousarray(host).tofile(out_dir / f"{step}.f32")
            runner.check()
        for request_id in record.get("end", []):
            if request_id in runner.cache:
                runner.release(request_id)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
