"""Continuous batching above the step function: admit, cut prompts into portions
under a token budget, decode, finish and free.

Mechanism of the reference's scheduler with its FCFS policy
(slipstream/scheduler/scheduler.py:86-158, slipstream/scheduler/policies/fcfs.py):
each step first gives every running request that is decoding one token, then
gives running requests that still have prompt (or replay) tokens a portion of at
most ``prefill_chunk_size``, then admits waiting requests in arrival order while
tokens, ``max_num_seqs`` and pages allow.  Everything scheduled runs as ONE
step-function call (the reference runs each prompt portion as its own forward).

A sequence's tokens are ``prompt + outputs``; ``num_computed_tokens`` of them are
in the cache.  A step feeds the next ``take`` of them; when that reaches the end,
the last fed token's logits give the next output.  This one rule covers prompt
portions, decoding, and replay after a preemption
(slipstream/scheduler/replay.py:14-34).

When pages run out:
  * at admission a request waits (LATER) or, if it could never fit even in an
    empty pool, is aborted (NEVER) (slipstream/memory/block_manager.py:108-128,
    slipstream/scheduler/scheduler.py:199-202);
  * while growing, the newest running request that is not already part of this
    step is preempted by recompute: its pages and slot are given back, it goes to
    the FRONT of the waiting queue and later replays prompt + outputs
    (:169-177, :253-268); if there is nobody else to preempt, the request skips
    this step and keeps what it has (:255-257).
"""

from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field

from slipstream_b200.cache import AllocStatus, CacheManager
from slipstream_b200.config.engine_config import SchedulerConfig
from slipstream_b200.config.sampling_params import SamplingParams


class SequenceStatus(enum.IntEnum):
    """slipstream/core/types.py:37-43 without SWAPPED (preemption is by recompute only)."""

    WAITING = 0
    RUNNING = 1
    FINISHED_STOPPED = 3
    FINISHED_LENGTH = 4
    FINISHED_ABORTED = 5


@dataclass
class Sequence:
    """One generation trajectory (slipstream/core/types.py:95-147)."""

    seq_id: int
    prompt_token_ids: list[int]
    sampling_params: SamplingParams = field(default_factory=SamplingParams)
    output_token_ids: list[int] = field(default_factory=list)
    status: SequenceStatus = SequenceStatus.WAITING
    arrival_ts: float = 0.0
    request_id: str = ""
    num_computed_tokens: int = 0
    max_new_tokens: int = 16  # output cap under the context window
    seed: int = 0
    preemptions: int = 0

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_output_tokens(self) -> int:
        return len(self.output_token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def is_finished(self) -> bool:
        return self.status >= SequenceStatus.FINISHED_STOPPED

    @property
    def num_uncomputed_tokens(self) -> int:
        return self.num_tokens - self.num_computed_tokens

    @property
    def is_decoding(self) -> bool:
        """Only the last sampled token is missing from the cache."""
        return self.num_output_tokens > 0 and self.num_uncomputed_tokens == 1

    def tokens_to_feed(self, take: int) -> list[int]:
        start = self.num_computed_tokens
        n_prompt = len(self.prompt_token_ids)
        if start + take <= n_prompt:
            return self.prompt_token_ids[start:start + take]
        if start >= n_prompt:
            return self.output_token_ids[start - n_prompt:start - n_prompt + take]
        return self.prompt_token_ids[start:] + self.output_token_ids[:start + take - n_prompt]


@dataclass
class ScheduledSeq:
    seq: Sequence
    take: int

    @property
    def samples(self) -> bool:
        """This portion reaches the sequence's end, so its last logits give a new token."""
        return self.seq.num_computed_tokens + self.take == self.seq.num_tokens


@dataclass
class SchedulerOutput:
    scheduled: list[ScheduledSeq]
    num_batched_tokens: int
    preempted: list[Sequence]
    aborted: list[Sequence]

    @property
    def num_decode_tokens(self) -> int:
        return sum(1 for s in self.scheduled if s.take == 1 and s.seq.num_output_tokens > 0)


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheManager) -> None:
        self.config = config
        self.cache = cache
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self._seq_ids = 0
        self.preemptions = 0

    # ------------------------------------------------------------------ queue
    def next_seq_id(self) -> int:
        self._seq_ids += 1
        return self._seq_ids

    def add_seq(self, seq: Sequence) -> None:
        seq.status = SequenceStatus.WAITING
        self.waiting.append(seq)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    @property
    def chunk(self) -> int:
        return self.config.prefill_chunk_size if self.config.enable_chunked_prefill else 10 ** 9

    # ------------------------------------------------------------------ the decision
    def schedule(self) -> SchedulerOutput:
        budget = self.config.max_num_batched_tokens
        chunk = self.chunk
        scheduled: list[ScheduledSeq] = []
        preempted: list[Sequence] = []
        aborted: list[Sequence] = []
        protected: set[int] = set()
        tokens = 0

        def try_take(seq: Sequence, take: int) -> bool:
            """Reserve pages for ``take`` more tokens of a running sequence, preempting if needed."""
            nonlocal tokens
            while not self.cache.can_reserve(seq.seq_id, take):
                victim = self._victim(exclude=protected | {seq.seq_id})
                if victim is None:
                    return False
                self.preempt_recompute(victim)
                preempted.append(victim)
            self.cache.reserve(seq.seq_id, take)
            scheduled.append(ScheduledSeq(seq, take))
            protected.add(seq.seq_id)
            tokens += take
            return True

        # 1. decodes first, one token each
        for seq in list(self.running):
            if seq not in self.running or not seq.is_decoding:
                continue
            if tokens + 1 > budget:
                break
            try_take(seq, 1)

        # 2. running sequences with prompt or replay tokens left
        for seq in list(self.running):
            if seq not in self.running or seq.is_decoding or seq.seq_id in protected:
                continue
            take = min(seq.num_uncomputed_tokens, budget - tokens, chunk)
            if take <= 0:
                continue
            try_take(seq, take)

        # 3. admit waiting sequences, first come first served
        for seq in sorted(self.waiting, key=lambda s: (s.arrival_ts, s.seq_id)):
            if tokens >= budget or len(self.running) >= self.config.max_num_seqs:
                break
            if seq in preempted:
                continue  # it lost its pages in this very step
            take = min(seq.num_uncomputed_tokens, budget - tokens, chunk)
            total = seq.num_prompt_tokens + seq.max_new_tokens
            status = self.cache.can_admit(total, take, chunk)
            if status is AllocStatus.NEVER:
                seq.status = SequenceStatus.FINISHED_ABORTED
                self.waiting.remove(seq)
                aborted.append(seq)
                continue
            if status is AllocStatus.LATER:
                break  # keep arrival order: nobody overtakes a request that is waiting for pages
            self.waiting.remove(seq)
            seq.status = SequenceStatus.RUNNING
            self.running.append(seq)
            self.cache.admit(seq.seq_id)
            self.cache.reserve(seq.seq_id, take)
            scheduled.append(ScheduledSeq(seq, take))
            protected.add(seq.seq_id)
            tokens += take

        assert tokens <= budget, "token budget exceeded"
        return SchedulerOutput(scheduled, tokens, preempted, aborted)

    def _victim(self, exclude: set[int]) -> Sequence | None:
        """Newest running sequence outside ``exclude`` (slipstream/scheduler/policies/fcfs.py:22-25)."""
        others = [s for s in self.running if s.seq_id not in exclude]
        if not others:
            return None
        return max(others, key=lambda s: (s.arrival_ts, s.seq_id))

    # ------------------------------------------------------------------ transitions
    def preempt_recompute(self, seq: Sequence) -> None:
        self.running.remove(seq)
        self.cache.release(seq.seq_id)
        seq.num_computed_tokens = 0
        seq.status = SequenceStatus.WAITING
        seq.preemptions += 1
        self.waiting.appendleft(seq)
        self.preemptions += 1

    def finish(self, seq: Sequence) -> None:
        """Remove a finished (or aborted) sequence and give back what it holds."""
        if seq in self.running:
            self.running.remove(seq)
        if seq in self.waiting:
            self.waiting.remove(seq)
        if seq.seq_id in self.cache:
            self.cache.release(seq.seq_id)

    def abort(self, seq_id: int) -> None:
        for seq in list(self.running) + list(self.waiting):
            if seq.seq_id == seq_id:
                seq.status = SequenceStatus.FINISHED_ABORTED
                self.finish(seq)
                return
