"""The Python entry point, in the reference's manner:

    engine = LLMEngine(EngineConfig.for_model(folder))
    tokens = engine.generate(Request("r0", None, [1, 2, 3], SamplingParams(max_tokens=8), 0.0))
    outs   = engine.generate_batch([...])         # continuous batching; inject="arrival" releases each
    for t in engine.stream(request): ...          # request when the wall clock reaches its arrival_ts

(slipstream/engine/llm_engine.py:66-127).  ``generate`` and ``stream`` are
``generate_batch`` with one request.  Every step is ONE call of the step function
with whatever the scheduler chose: decoded tokens beside prompt portions.
``LLM`` is a thin convenience wrapper that returns ``RequestOutput`` records.

Token ids in, token ids out; text prompts need a ``tokenizer.json`` in the model
folder (slipstream/models/tokenizer.py:11-57), which random-weight folders lack.
"""

from __future__ import annotations

import time
from collections.abc import Iterator
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np
import torch

from slipstream_b200.config.engine_config import CacheConfig, EngineConfig, SchedulerConfig
from slipstream_b200.config.sampling_params import SamplingParams
from slipstream_b200 import ops
from slipstream_b200.sampling.sampler import SampleRow, Sampler

from .context import StepEntry
from .runner import ModelRunner
from .scheduler import ScheduledSeq, Scheduler, Sequence, SequenceStatus


@dataclass
class Request:
    """slipstream/core/types.py:73-87.  The two latency targets are carried for callers that set them; the
    first-come-first-served policy, the only one built, does not read them."""

    request_id: str
    prompt: str | None
    prompt_token_ids: list[int] | None
    sampling_params: SamplingParams = field(default_factory=SamplingParams)
    arrival_ts: float = 0.0
    slo_ttft_ms: float = 2000.0
    slo_tpot_ms: float = 100.0

    def __post_init__(self) -> None:
        if self.prompt is None and self.prompt_token_ids is None:
            raise ValueError("Request needs prompt or prompt_token_ids")


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: list[int]
    output_token_ids: list[int]
    finish_reason: str  # stop | length | abort
    text: str | None = None


@dataclass
class StepStats:
    """Counters of the last step (slipstream/observability/metrics.py:29-95, reduced)."""

    step: int = 0
    num_running: int = 0
    num_waiting: int = 0
    num_batched_tokens: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    free_pages: int = 0
    preemptions: int = 0
    step_time_ms: float = 0.0


PENDING = -1  # placeholder in a sequence's output for a token that was sampled but not yet read by the host


@dataclass
class InFlight:
    """A decode step whose sampled tokens are still on their way to the host."""

    seqs: list[Sequence]
    where: list[int]  # index into each sequence's output of the placeholder this step fills
    tokens_dev: torch.Tensor  # int32 [len(seqs) + 1] on the device: the tokens, then the device error word
    tokens_host: torch.Tensor  # pinned copy, valid once ``ready`` has happened
    ready: torch.cuda.Event


def absolute_arrival(ts: float, now: float) -> float:
    """An arrival time on the wall clock: small values are offsets from ``now``, values from 1e9 are wall-clock
    seconds already (slipstream/engine/llm_engine.py:38-42)."""
    return ts if ts >= 1_000_000_000.0 else now + ts


def capped_new_tokens(prompt_len: int, max_tokens: int, max_model_len: int) -> int:
    """New tokens that fit under the context window (slipstream/engine/llm_engine.py:56-63)."""
    if max_tokens < 1:
        return 0
    return max(0, min(max_tokens, max_model_len - prompt_len))


_FINISH = {SequenceStatus.FINISHED_STOPPED: "stop", SequenceStatus.FINISHED_LENGTH: "length",
           SequenceStatus.FINISHED_ABORTED: "abort"}


class LLMEngine:
    def __init__(self, config: EngineConfig) -> None:
        self.config = config
        m, c, s = config.model, config.cache, config.scheduler
        self.runner = ModelRunner(
            m.model_id, dtype=m.dtype, page_size=c.block_size, num_pages=c.num_gpu_blocks,
            gpu_memory_utilization=c.gpu_memory_utilization, max_num_seqs=s.max_num_seqs,
            max_model_len=m.max_model_len, load_format=m.load_format, seed=config.seed,
            use_cuda_graphs=config.use_cuda_graphs,
            max_step_tokens=min(s.max_num_batched_tokens,
                                s.prefill_chunk_size if s.enable_chunked_prefill else s.max_num_batched_tokens))
        self.model_config = self.runner.config
        self.max_model_len = self.runner.max_model_len
        self.scheduler = Scheduler(s, self.runner.cache)
        self.sampler = Sampler(self.model_config.vocab_size, self.runner.device, s.max_num_seqs)
        self.tokenizer = None
        folder = Path(m.model_id)
        if (folder / "tokenizer.json").is_file():
            from tokenizers import Tokenizer

            self.tokenizer = Tokenizer.from_file(str(folder / "tokenizer.json"))
        self.stats = StepStats()
        # wall-clock latencies of the last generate_batch, in seconds: time to the first token of every request
        # (from enqueue, or from its arrival with inject="arrival") and the gaps between a request's tokens, as
        # the host comes to know them (slipstream/engine/llm_engine.py:89-90,577-598)
        self.last_ttft_s: list[float] = []
        self.last_itl_s: list[float] = []
        self._started_at: dict[int, float] = {}
        self._last_emit: dict[int, float] = {}
        self._requests_seen = 0
        self._inflight: InFlight | None = None
        self._zombies: list[Sequence] = []  # stopped while their next token was already being computed
        self.run_ahead = True  # decode steps are launched before the tokens of the step before reach the host
        # pinned buffers and events of the steps in flight, made once (a step in flight and the one being launched)
        self._token_ring = [torch.empty(s.max_num_seqs + 1, dtype=torch.int32, pin_memory=True) for _ in range(3)]
        self._event_ring = [torch.cuda.Event() for _ in range(3)]
        self._ring_turn = 0

    # ------------------------------------------------------------------ public calls
    def generate(self, request: Request) -> list[int]:
        """Blocking generation of one request; returns the output token ids only."""
        return self.generate_batch([request])[0]

    def stream(self, request: Request) -> Iterator[int]:
        """Token iterator with the same tokens as ``generate``."""
        seq = self._make_sequence(request)
        self._started_at[seq.seq_id] = time.perf_counter()
        self.scheduler.add_seq(seq)
        emitted = 0
        while self.scheduler.has_work():
            if not self._step():
                break
            while emitted < seq.num_output_tokens and seq.output_token_ids[emitted] != PENDING:
                yield seq.output_token_ids[emitted]
                emitted += 1
        self.drain()
        while emitted < seq.num_output_tokens:
            yield seq.output_token_ids[emitted]
            emitted += 1

    def warm_up(self, max_requests: int | None = None) -> int:
        """Capture the decode graphs of all batch sizes up to ``max_requests`` (default ``max_num_seqs``) before
        the first request, so that no request ever waits for a capture.  Returns the number captured."""
        return self.runner.capture_decode_graphs(max_requests)

    def add_request(self, request: Request) -> Sequence:
        """Queue a request; ``step`` then advances everything queued by one engine step."""
        seq = self._make_sequence(request)
        self.scheduler.add_seq(seq)
        return seq

    def step(self) -> bool:
        """One engine step: schedule, one step-function call, sample, finish.  False when idle."""
        return self._step()

    def generate_batch(self, requests: list[Request], *, inject: str = "all") -> list[list[int]]:
        """Continuous batching of several requests (slipstream/engine/llm_engine.py:107-119).  ``inject="all"``
        queues every request at once; ``inject="arrival"`` releases a request when the wall clock reaches its
        ``arrival_ts`` (an offset from the call, or wall-clock seconds) and sleeps while nothing is due."""
        if inject not in ("all", "arrival"):
            raise ValueError("inject must be 'all' or 'arrival'")
        seqs = [self._make_sequence(r) for r in requests]
        wall, perf = time.time(), time.perf_counter()
        self.last_ttft_s.clear()
        self.last_itl_s.clear()
        self._started_at.clear()
        self._last_emit.clear()
        pending: list[Sequence] = []
        for seq in seqs:
            if inject == "all":
                self._started_at[seq.seq_id] = perf
                self.scheduler.add_seq(seq)
            else:
                seq.arrival_ts = absolute_arrival(seq.arrival_ts, wall)
                self._started_at[seq.seq_id] = perf + (seq.arrival_ts - wall)
                pending.append(seq)
        pending.sort(key=lambda q: (q.arrival_ts, q.seq_id))
        self.run_until_done(seqs, pending)
        return [list(q.output_token_ids) for q in seqs]

    def run_until_done(self, seqs: list[Sequence], pending: list[Sequence] | None = None) -> None:
        """Step until the scheduler is idle.  ``pending``: sequences not yet queued, sorted by their wall-clock
        arrival; each is queued when its time has come."""
        pending = pending if pending is not None else []
        # the reference's bound on replay storms (slipstream/engine/llm_engine.py:423-429)
        limit = 1 + 8 * sum(q.num_prompt_tokens + q.max_new_tokens for q in seqs)
        steps = 0
        while (self.scheduler.has_work() or pending) and steps < limit:
            if pending:
                now = time.time()
                due = 0
                while due < len(pending) and pending[due].arrival_ts <= now:
                    self.scheduler.add_seq(pending[due])
                    due += 1
                del pending[:due]
                if not self.scheduler.has_work():
                    self.drain()
                    time.sleep(max(0.0, min(pending[0].arrival_ts - time.time(), 0.02)))
                    continue
            steps += 1
            if not self._step():
                if not pending:
                    break
                self.drain()
                time.sleep(max(0.0, min(pending[0].arrival_ts - time.time(), 0.02)))
        self.drain()
        for seq in seqs:
            if not seq.is_finished:
                seq.status = SequenceStatus.FINISHED_ABORTED
                self.scheduler.finish(seq)

    def tokenize(self, request: Request) -> list[int]:
        if request.prompt_token_ids is not None:
            return [int(t) for t in request.prompt_token_ids]
        if self.tokenizer is None:
            raise ValueError("a text prompt needs tokenizer.json in the model folder; pass prompt_token_ids")
        return list(self.tokenizer.encode(request.prompt, add_special_tokens=False).ids)

    # ------------------------------------------------------------------ internals
    def _make_sequence(self, request: Request) -> Sequence:
        ids = self.tokenize(request)
        if not ids:
            raise ValueError("empty prompt")
        if len(ids) >= self.max_model_len:
            raise ValueError(f"prompt length {len(ids)} exceeds max_model_len {self.max_model_len}")
        vocab = self.model_config.vocab_size
        if min(ids) < 0 or max(ids) >= vocab:
            raise ValueError(f"a prompt token id is outside [0, {vocab})")
        params = request.sampling_params
        if params.stop_strings and self.tokenizer is None:
            raise ValueError("stop_strings need tokenizer.json in the model folder")
        max_new = capped_new_tokens(len(ids), params.max_tokens, self.max_model_len)
        self._requests_seen += 1
        seed = params.seed if params.seed is not None else (self.config.seed * 1000003 + self._requests_seen)
        return Sequence(seq_id=self.scheduler.next_seq_id(), prompt_token_ids=ids, sampling_params=params,
                        arrival_ts=request.arrival_ts, request_id=request.request_id, max_new_tokens=max_new,
                        seed=seed)

    def _mark_emit(self, seq: Sequence, now: float) -> None:
        """The host has just learnt a token of ``seq``: its first one gives the time to first token, every other
        one a gap between tokens (slipstream/engine/llm_engine.py:577-598)."""
        prev = self._last_emit.get(seq.seq_id)
        if prev is None:
            self.last_ttft_s.append(max(0.0, now - self._started_at.get(seq.seq_id, now)))
        else:
            self.last_itl_s.append(now - prev)
        self._last_emit[seq.seq_id] = now

    def _is_stop(self, seq: Sequence, token: int) -> bool:
        """slipstream/engine/llm_engine.py:223-234; the stop token stays in the output."""
        params = seq.sampling_params
        if token in params.stop_token_ids:
            return True
        eos = self.model_config.eos_token_id
        if not params.ignore_eos and eos is not None and token == eos:
            return True
        if params.stop_strings and self.tokenizer is not None:
            text = self.tokenizer.decode(seq.output_token_ids)
            return any(stop and stop in text for stop in params.stop_strings)
        return False

    # ------------------------------------------------------------------ decode steps that run ahead of the host
    def _collect(self, flight: InFlight) -> None:
        """Read the tokens of a launched step, put them in place of their placeholders, finish what is done."""
        flight.ready.synchronize()
        tokens = flight.tokens_host.tolist()
        self._check_status(tokens.pop(), flight.seqs)
        now = time.perf_counter()
        for seq, at, token in zip(flight.seqs, flight.where, tokens):
            if seq in self._zombies:  # stopped one token earlier; this token was computed for nothing
                self._zombies.remove(seq)
                self.scheduler.finish(seq)
                continue
            seq.output_token_ids[at] = int(token)
            self._mark_emit(seq, now)
            ahead = at + 1 < len(seq.output_token_ids)  # its next token is already being computed
            if self._is_stop(seq, int(token)):
                seq.status = SequenceStatus.FINISHED_STOPPED
                if ahead:
                    del seq.output_token_ids[at + 1:]
                    self._zombies.append(seq)  # keeps its pages until that step has run
                else:
                    self.scheduler.finish(seq)
            elif not ahead and (seq.num_output_tokens >= seq.max_new_tokens or seq.num_tokens >= self.max_model_len):
                seq.status = SequenceStatus.FINISHED_LENGTH
                self.scheduler.finish(seq)

    def _check_status(self, status: int, seqs: list[Sequence]) -> None:
        """``status`` is the device error word as the step's sampling kernel saw it.  Non-zero: a kernel met a
        token id, cache slot or block-table entry out of range, or a bounded wait inside a kernel gave up; the
        tokens of that step cannot be trusted.  Everything that was running is aborted (its pages go back) and
        ``KernelError`` is raised."""
        if not status:
            return
        self._inflight = None
        for seq in list(self.scheduler.running) + [s for s in seqs if s not in self.scheduler.running]:
            if not seq.is_finished:
                seq.status = SequenceStatus.FINISHED_ABORTED
            self.scheduler.finish(seq)
        self._zombies.clear()
        ops.raise_for_status(status, self.runner.device)

    def drain(self) -> None:
        """Wait for the tokens of the decode step that is still running, if one is, and put them in place."""
        if self._inflight is not None:
            flight, self._inflight = self._inflight, None
            self._collect(flight)

    def _run_ahead_candidates(self) -> list[Sequence] | None:
        """The sequences of a steady decode step, or None when the next step is not one: somebody waits to be
        admitted, or still has prompt to run, or needs its text (stop strings), or pages are short."""
        sched = self.scheduler
        if not self.run_ahead or sched.waiting or not sched.running:
            return None
        live = [s for s in sched.running if not s.is_finished]
        if not live or len(live) > sched.config.max_num_batched_tokens:
            return None
        for seq in live:
            if not seq.is_decoding or seq.sampling_params.stop_strings:
                return None
        # a sequence whose last allowed token is already being computed takes no further step
        todo = [s for s in live if s.num_output_tokens < s.max_new_tokens and s.num_tokens < self.max_model_len]
        if not todo or not self.runner.can_run_ahead(len(todo)):
            return None
        if not self.runner.cache.can_reserve_all([(s.seq_id, 1) for s in todo]):
            return None  # growing needs a preemption: the ordinary path decides that
        return todo

    def _step_run_ahead(self, todo: list[Sequence]) -> bool:
        """Launch the next decode step with token ids taken on the device from the step before, then read the
        tokens of the step before while the new one runs."""
        started = time.perf_counter()
        prev = self._inflight
        index = {id(s): i for i, s in enumerate(prev.seqs)} if prev is not None else {}
        entries, src_rows, rows, where = [], [], [], []
        for seq in todo:
            last = seq.output_token_ids[-1]
            src_rows.append(index[id(seq)] if last == PENDING else -1)
            entries.append(StepEntry(seq.seq_id, [0 if last == PENDING else last], [0]))
            rows.append(SampleRow(seq.sampling_params, seq.seed, seq.num_output_tokens,
                                  self.runner.cache.get(seq.seq_id).slot))
        for seq in todo:
            self.runner.cache.reserve(seq.seq_id, 1)
        logits = self.runner.step_decode(entries, prev.tokens_dev if prev is not None else None,
                                         np.asarray(src_rows, dtype=np.int32))
        tokens_dev = self.sampler.sample(logits, rows, with_status=True)
        turn = self._ring_turn = (self._ring_turn + 1) % len(self._token_ring)
        tokens_host = self._token_ring[turn][: len(todo) + 1]
        tokens_host.copy_(tokens_dev, non_blocking=True)
        ready = self._event_ring[turn]
        ready.record()
        for seq in todo:  # the host's view moves on at once; the token's value follows
            seq.num_computed_tokens += 1
            where.append(len(seq.output_token_ids))
            seq.output_token_ids.append(PENDING)
        self._inflight = InFlight(todo, where, tokens_dev, tokens_host, ready)
        if prev is not None:
            self._collect(prev)
        st = self.stats
        st.step += 1
        st.num_running, st.num_waiting = len(self.scheduler.running), len(self.scheduler.waiting)
        st.num_batched_tokens = st.decode_tokens = len(todo)
        st.prefill_tokens = 0
        st.free_pages = self.runner.cache.min_free_pages()
        st.preemptions = self.scheduler.preemptions
        st.step_time_ms = (time.perf_counter() - started) * 1e3
        return True

    def _step(self) -> bool:
        """Schedule, run one step-function call, sample, finish.  False when nothing can run."""
        todo = self._run_ahead_candidates()
        if todo is not None:
            return self._step_run_ahead(todo)
        self.drain()
        if not self.scheduler.has_work():
            return False
        started = time.perf_counter()
        plan = self.scheduler.schedule()
        if not plan.scheduled:
            # nothing fits: whoever is still waiting can never run (slipstream/engine/llm_engine.py:467-474)
            for stuck in list(self.scheduler.waiting):
                stuck.status = SequenceStatus.FINISHED_ABORTED
                self.scheduler.finish(stuck)
            return False
        entries: list[StepEntry] = []
        sampling: list[ScheduledSeq] = []
        for item in plan.scheduled:
            seq = item.seq
            if seq.num_computed_tokens == 0:
                slot = self.runner.cache.get(seq.seq_id).slot
                self.runner.reset_state(slot)
                self.sampler.begin_request(slot, seq.sampling_params,
                                           seq.prompt_token_ids + seq.output_token_ids)
            want = [item.take - 1] if item.samples else []
            entries.append(StepEntry(seq.seq_id, seq.tokens_to_feed(item.take), want))
            if item.samples:
                sampling.append(item)
        decode_tokens = plan.num_decode_tokens
        logits = self.runner.step(entries)
        tokens: list[int] = []
        if sampling:
            rows = [SampleRow(i.seq.sampling_params, i.seq.seed, i.seq.num_output_tokens,
                              self.runner.cache.get(i.seq.seq_id).slot) for i in sampling]
            # the step's one device-to-host copy: the tokens and, behind them, the device error word
            tokens = self.sampler.sample(logits, rows, with_status=True).tolist()
            self._check_status(tokens.pop(), [i.seq for i in plan.scheduled])
        for item in plan.scheduled:
            item.seq.num_computed_tokens += item.take
        now = time.perf_counter()
        for item, token in zip(sampling, tokens):
            seq = item.seq
            seq.output_token_ids.append(int(token))
            self._mark_emit(seq, now)
            if self._is_stop(seq, int(token)):
                seq.status = SequenceStatus.FINISHED_STOPPED
            elif seq.num_output_tokens >= seq.max_new_tokens or seq.num_tokens >= self.max_model_len:
                seq.status = SequenceStatus.FINISHED_LENGTH
            if seq.is_finished:
                self.scheduler.finish(seq)
        st = self.stats
        st.step += 1
        st.num_running, st.num_waiting = len(self.scheduler.running), len(self.scheduler.waiting)
        st.num_batched_tokens = plan.num_batched_tokens
        st.decode_tokens = decode_tokens
        st.prefill_tokens = plan.num_batched_tokens - st.decode_tokens
        st.free_pages = self.runner.cache.min_free_pages()
        st.preemptions = self.scheduler.preemptions
        st.step_time_ms = (time.perf_counter() - started) * 1e3
        return True


class LLM:
    """Convenience wrapper: keyword options instead of an ``EngineConfig``; lists in, records out."""

    def __init__(self, model: str, *, dtype: str | None = None, max_model_len: int | None = None,
                 block_size: int = 16, num_gpu_blocks: int | None = None, gpu_memory_utilization: float = 0.9,
                 max_num_seqs: int = 256, max_num_batched_tokens: int = 8192, prefill_chunk_size: int = 256,
                 enable_chunked_prefill: bool = True, seed: int = 0, load_format: str = "safetensors",
                 use_cuda_graphs: bool = True) -> None:
        self.engine = LLMEngine(EngineConfig.for_model(
            model, dtype=dtype, max_model_len=max_model_len, load_format=load_format,
            cache=CacheConfig(block_size=block_size, gpu_memory_utilization=gpu_memory_utilization,
                              num_gpu_blocks=num_gpu_blocks),
            scheduler=SchedulerConfig(max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens,
                                      enable_chunked_prefill=enable_chunked_prefill,
                                      prefill_chunk_size=prefill_chunk_size),
            seed=seed, use_cuda_graphs=use_cuda_graphs))

    def generate(self, prompts: list[str] | None = None, sampling_params: SamplingParams | list[SamplingParams] | None = None,
                 *, prompt_token_ids: list[list[int]] | None = None) -> list[RequestOutput]:
        n = len(prompt_token_ids) if prompt_token_ids is not None else len(prompts or [])
        if isinstance(sampling_params, list):
            params = sampling_params
        else:
            params = [sampling_params or SamplingParams()] * n
        requests = [Request(f"req-{i}", None if prompts is None else prompts[i],
                            None if prompt_token_ids is None else prompt_token_ids[i], params[i], float(i) * 1e-6)
                    for i in range(n)]
        engine = self.engine
        seqs = [engine._make_sequence(r) for r in requests]
        for seq in seqs:
            engine._started_at[seq.seq_id] = time.perf_counter()
            engine.scheduler.add_seq(seq)
        engine.run_until_done(seqs)
        outs = []
        for seq in seqs:
            text = engine.tokenizer.decode(seq.output_token_ids) if engine.tokenizer is not None else None
            outs.append(RequestOutput(seq.request_id, seq.prompt_token_ids, list(seq.output_token_ids),
                                      _FINISH.get(seq.status, "abort"), text))
        return outs
