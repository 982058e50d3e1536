"""Token selection from the step's float32 logits, on the device.

Greedy (arg-max of the raw logits) and the reference's sampling chain: repetition
penalty, temperature, top-k, top-p, min-p, then a draw
(slipstream/engine/sampler.py:36-146).  One kernel launch serves a batch in which
every row has its own parameters.  The draw is reproducible: a request's stream is
keyed by its seed, and its n-th generated token uses draw number n, whatever else
is in the batch and whether or not the request was preempted and replayed in
between.  (The reference re-seeds a generator with ``params.seed`` at every call,
:58-60, so all of a request's draws use the same random numbers.)

The tokens a request has seen (prompt and output) are kept as a bit mask in the
request's state slot, only when a request asks for a repetition penalty.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from slipstream_b200 import ops
from slipstream_b200.config.sampling_params import SamplingParams


@dataclass
class SampleRow:
    params: SamplingParams
    seed: int
    draw: int  # index of the token being drawn within the request's output
    slot: int = -1  # state slot of the request (for the seen-token mask)


class Sampler:
    def __init__(self, vocab_size: int, device: torch.device, max_num_seqs: int) -> None:
        self.vocab_size = vocab_size
        self.device = device
        self.max_num_seqs = max_num_seqs
        self.seen_words = (vocab_size + 31) // 32
        self.seen: torch.Tensor | None = None  # int32 [max_num_seqs, seen_words], made on first use

    # ------------------------------------------------------------------ history for the penalty
    def begin_request(self, slot: int, params: SamplingParams, tokens: list[int]) -> None:
        """Start (or restart after a preemption) the seen-token mask of a request."""
        if params.repetition_penalty == 1.0 or params.is_greedy:
            return
        if self.seen is None:
            self.seen = torch.zeros((self.max_num_seqs, self.seen_words), dtype=torch.int32, device=self.device)
        self.seen[slot].zero_()
        if tokens:
            ids = torch.tensor(tokens, dtype=torch.int32).to(self.device)
            ops.mark_seen(self.seen[slot], ids, self.vocab_size)

    # ------------------------------------------------------------------ selection
    def greedy(self, logits: torch.Tensor, with_status: bool = False) -> torch.Tensor:
        return ops.argmax(logits, with_status)

    def sample(self, logits: torch.Tensor, rows: list[SampleRow], with_status: bool = False) -> torch.Tensor:
        """int32 [M] token ids on the device for float32 ``logits`` [M, vocab]; ``with_status`` appends the device
        error word as element M (``ops.argmax``)."""
        if logits.shape[0] != len(rows):
            raise ValueError(f"{logits.shape[0]} logit rows but {len(rows)} sampling rows")
        if all(r.params.is_greedy for r in rows):
            return self.greedy(logits, with_status)
        m = len(rows)
        # every row's parameters in one pinned buffer and one copy: [4 float32 | 2 int32 | 2 int64] x m
        host = torch.empty(40 * m, dtype=torch.uint8, pin_memory=True)
        raw = host.numpy()
        floats = raw[: 16 * m].view(np.float32).reshape(4, m)
        ints = raw[16 * m: 24 * m].view(np.int32).reshape(2, m)
        longs = raw[24 * m:].view(np.int64).reshape(2, m)
        params = [r.params for r in rows]
        floats[0] = [0.0 if p.is_greedy else p.temperature for p in params]
        floats[1] = [p.top_p for p in params]
        floats[2] = [p.min_p for p in params]
        floats[3] = [p.repetition_penalty for p in params]
        ints[0] = [p.top_k for p in params]
        ints[1] = [r.slot if r.params.repetition_penalty != 1.0 else -1 for r in rows]
        longs[0] = [(r.seed & 0xFFFFFFFFFFFFFFFF) - (1 << 64) if (r.seed & 0x8000000000000000) else (r.seed & 0xFFFFFFFFFFFFFFFF)
                    for r in rows]
        longs[1] = [r.draw for r in rows]
        dev = host.to(self.device, non_blocking=True)
        f = dev[: 16 * m].view(torch.float32).view(4, m)
        i32 = dev[16 * m: 24 * m].view(torch.int32).view(2, m)
        i64 = dev[24 * m:].view(torch.int64).view(2, m)
        return ops.sample(logits, temperature=f[0], top_p=f[1], min_p=f[2], penalty=f[3], top_k=i32[0],
                          slots=i32[1], seeds=i64[0], draws=i64[1], seen=self.seen, with_status=with_status)
