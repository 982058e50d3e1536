"""The model runner: a loaded model, its cache, and the one step function.

``ModelRunner.step(entries)`` takes a batch of (request, its next tokens, wanted
places): portions of prompts beside single decoded tokens, cut anywhere.  It runs
only those tokens, as one ragged batch, against the pages earlier steps left,
and returns float32 logits at the wanted places.  The reference runs decodes as
one dense ``[B, 1]`` forward and every prompt portion as its own ``[1, take]``
forward (slipstream/engine/llm_engine.py:476-484,508-567) and returns logits for
every position (slipstream/models/causal_lm.py:140).

Generation (``LLMEngine``) and trace replay (``bin/trace_run``) both drive this
class; neither has a forward pass, cache or loader of its own.
"""

from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from slipstream_b200 import ops
from slipstream_b200.cache import CacheManager, PagedStore, pool_sizes, tokens_that_fit
from slipstream_b200.parts.base import Runtime
from slipstream_b200.registry import load_config
from slipstream_b200.weights.loader import load_weights
from slipstream_b200.weights.random_init import random_weights_on_device

from .context import StepContext, StepEntry, StepInputError, plan_step, to_device
from .graphs import BUCKETS, DecodeGraph, MixedGraph, bucket_for, mixed_bucket

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class ModelRunner:
    def __init__(self, model_dir: str | Path, *, dtype: str | None = None, page_size: int = 16,
                 num_pages: "int | list[int] | None" = None, gpu_memory_utilization: float = 0.9,
                 max_num_seqs: int = 256, max_model_len: int | None = None, load_format: str = "safetensors",
                 seed: int = 0, device: str | torch.device = "cuda:0", use_cuda_graphs: bool = True,
                 max_step_tokens: int | None = None) -> None:
        """``page_size``: tokens per page for cache groups whose mixers do not ask for a size of their own.
        ``num_pages``: pages of that size the cache should hold (groups with another page size get as many pages
        as hold the same tokens; a windowed group at most what ``max_num_seqs`` requests can keep of their windows
        when a step feeds up to ``max_step_tokens`` tokens of a request), or one count per cache group, or None
        to size the pools from the free device memory."""
        ops.require_cuda()
        self.device = torch.device(device)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        self.architecture, self.config = load_config(model_dir)
        dtype_name = dtype or self.config.torch_dtype
        if dtype_name not in _DTYPES:
            raise ValueError(f"unsupported dtype: {dtype_name} (bfloat16 or float32)")
        self.dtype_name = dtype_name
        self.runtime = Runtime(self.device, _DTYPES[dtype_name])
        self.max_model_len = max_model_len or self.config.max_position_embeddings
        self.page_size = page_size
        self.max_num_seqs = max_num_seqs

        self.model = self.architecture.build(self.config)
        specs = self.model.weight_specs()
        if load_format == "random":
            weights = random_weights_on_device(specs, self.runtime, seed)
        else:
            weights = load_weights(model_dir, specs, self.runtime)
        self.model.bind(weights, self.runtime)
        del weights

        layouts = self.model.group_layouts
        page_sizes = [layout.spec.page_size or page_size for layout in layouts]
        step_tokens = max_step_tokens or self.max_model_len
        if isinstance(num_pages, (list, tuple)):
            pools = [int(n) for n in num_pages]
        else:
            if num_pages is None:
                torch.cuda.synchronize(self.device)
                torch.cuda.empty_cache()
                free, _total = torch.cuda.mem_get_info(self.device)
                per_token = [PagedStore.bytes_per_token(layout, self.runtime.dtype) for layout in layouts]
                # leave room for activations of the largest step beside the pages
                tokens = tokens_that_fit(layouts, page_sizes, per_token, int(free * gpu_memory_utilization * 0.9),
                                         max_num_seqs, self.max_model_len, step_tokens)
            else:
                tokens = int(num_pages) * page_size
            pools = pool_sizes(layouts, page_sizes, tokens, max_num_seqs, self.max_model_len, step_tokens)
        self.cache = CacheManager(layouts, pools, page_sizes, max_num_seqs, self.max_model_len)
        self.num_pages = self.cache.num_pages
        self.store = PagedStore(layouts, self.runtime.dtype, self.device, self.model.entry_state, max_num_seqs)
        self.model.attach_store(self.store)
        self.has_state = any(self.model.entry_state)
        self.steps_run = 0
        self.last_h2d_bytes = 0
        self.use_cuda_graphs = (use_cuda_graphs and self.device.type == "cuda"
                                and all(getattr(p, "cuda_graph_safe", False) for p in self.model.parts()))
        # parts whose captured form depends on the lengths of a step (``Part.capture_variant``)
        from slipstream_b200.parts.base import Part
        seen: set[object] = set()
        self.variant_parts = []
        for part in self.model.parts():
            if type(part).capture_variant is not Part.capture_variant and part.capture_group() not in seen:
                seen.add(part.capture_group())
                self.variant_parts.append(part)
        self._graphs: dict[tuple, DecodeGraph] = {}  # (batch bucket, the parts' variants)
        # steps with prompt portions: (token bucket, request bucket, logits per token?, variants) -> graph, or the
        # number of times the bucket has come up so far.  A capture costs tens to hundreds of milliseconds (0.25 s
        # for a 48-layer model), so a bucket is captured only when it keeps coming up: at its seventh step.
        self._mixed_graphs: dict[tuple, "MixedGraph | int"] = {}
        self.mixed_graph_after = 6  # steps of a bucket that run kernel by kernel before it is captured
        self.max_mixed_graphs = 24

    # ------------------------------------------------------------------ requests
    def admit(self, request_id: object) -> None:
        """Give a new request its state slot (zeroed) and empty block tables."""
        req = self.cache.admit(request_id)
        if self.has_state:
            self.store.zero_state(req.slot)

    def reset_state(self, slot: int) -> None:
        """Zero the fixed-size state rows of a slot (a request starts, or restarts after a preemption)."""
        if self.has_state:
            self.store.zero_state(slot)

    def release(self, request_id: object) -> None:
        self.cache.release(request_id)

    # ------------------------------------------------------------------ the step function
    @torch.inference_mode()
    def step(self, entries: list[StepEntry]) -> torch.Tensor:
        for e in entries:
            if e.request_id not in self.cache:
                self.admit(e.request_id)
        decode_only = all(len(e.tokens) == 1 for e in entries)
        bucket = self._graph_bucket(len(entries)) if decode_only else None
        plan = plan_step(entries, self.cache, self.config.vocab_size, with_tables=bucket is None)
        mixed = None if bucket is not None else self._mixed_graph(plan)
        if bucket is not None:
            graph = self._decode_graph(bucket, plan)
            self.last_h2d_bytes = graph.h2d_bytes
            logits = graph.run(plan)
        elif mixed is not None:
            self.last_h2d_bytes = mixed.h2d_bytes
            logits = mixed.run(plan)
        else:
            ctx = to_device(plan, self.device)
            self.last_h2d_bytes = ctx.extras["host_buffer"].numel() * 4
            logits = self.run(ctx)
        for e in entries:
            self.cache.commit(e.request_id, len(e.tokens))
        self.steps_run += 1
        return logits

    def _decode_graph(self, bucket: int, plan) -> DecodeGraph:
        """The captured step for this bucket and for the form each part wants at these lengths (a decode
        attention, say, cuts the keys of few long requests into more slices than those of many short ones, and
        the number of slices is fixed when a graph is captured)."""
        longest = int(plan.seq_lens.max())
        variants = tuple(part.capture_variant(longest, plan) for part in self.variant_parts)
        graph = self._graphs.get((bucket, variants))
        if graph is None:
            graph = self._graphs[(bucket, variants)] = DecodeGraph(self, bucket, variants)
        return graph

    def _mixed_graph(self, plan) -> "MixedGraph | None":
        """The captured step that serves this plan (prompt portions beside decoded tokens), once its bucket has come
        up often enough to be worth a capture; None: run the step kernel by kernel."""
        if not self.use_cuda_graphs:
            return None
        sizes = mixed_bucket(plan.num_tokens, plan.num_requests)
        if sizes is None:
            return None
        per_token = plan.logit_rows.size > sizes[1]
        if per_token and plan.logit_rows.size > sizes[0]:
            return None
        variants = tuple(part.capture_variant(int(plan.seq_lens.max()), plan) for part in self.variant_parts)
        key = (*sizes, per_token, variants)
        seen = self._mixed_graphs.get(key, 0)
        if isinstance(seen, MixedGraph):
            return seen
        if seen < self.mixed_graph_after:
            self._mixed_graphs[key] = seen + 1
            return None
        if sum(isinstance(g, MixedGraph) for g in self._mixed_graphs.values()) >= self.max_mixed_graphs:
            return None
        graph = self._mixed_graphs[key] = MixedGraph(self, sizes[0], sizes[1], sizes[0] if per_token else sizes[1], variants)
        return graph

    def _graph_bucket(self, n_requests: int) -> int | None:
        bucket = bucket_for(n_requests) if self.use_cuda_graphs else None
        return bucket if bucket is not None and bucket <= max(self.max_num_seqs, 1) * 2 else None

    def capture_decode_graphs(self, max_requests: int | None = None) -> int:
        """Capture the decode graph of every batch bucket up to ``max_requests`` (default: the most requests
        the cache manager admits) now, instead of at the first step that needs it: a capture takes tens of
        milliseconds, during which every running request waits.  Returns how many graphs were captured."""
        if not self.use_cuda_graphs:
            return 0
        limit = self.max_num_seqs if max_requests is None else max_requests
        made = 0
        for bucket in BUCKETS:
            variants = tuple(part.capture_variant(1) for part in self.variant_parts)  # the form for short requests
            if self._graph_bucket(bucket) != bucket or (bucket, variants) in self._graphs:
                continue
            self._graphs[(bucket, variants)] = DecodeGraph(self, bucket, variants)
            made += 1
            if bucket >= limit:
                break
        return made

    def can_run_ahead(self, n_requests: int) -> bool:
        """Whether a decode-only step of this many requests goes through a captured graph (the only kind of
        step that can take token ids straight from the device)."""
        return self._graph_bucket(n_requests) is not None

    @torch.inference_mode()
    def step_decode(self, entries: list[StepEntry], pending: torch.Tensor | None,
                    src_rows: "np.ndarray | None") -> torch.Tensor:
        """A decode-only step whose token ids may still be on the device: row r takes
        ``pending[src_rows[r]]`` where ``src_rows[r] >= 0`` (its entry's token is then a placeholder).
        Returns logits of every row as a view that is valid until the next step."""
        if any(len(e.tokens) != 1 for e in entries) or not self.can_run_ahead(len(entries)):
            raise StepInputError("step_decode takes decode-only steps that fit a captured graph")
        plan = plan_step(entries, self.cache, self.config.vocab_size, with_tables=False)
        graph = self._decode_graph(self._graph_bucket(plan.num_requests), plan)
        self.last_h2d_bytes = graph.h2d_bytes
        logits = graph.run(plan, pending=pending, src_rows=src_rows, keep=False)
        for e in entries:
            self.cache.commit(e.request_id, len(e.tokens))
        self.steps_run += 1
        return logits

    def run(self, ctx: StepContext) -> torch.Tensor:
        return self.model.forward(ctx)

    def check(self) -> None:
        """Raise if a kernel flagged an out-of-range id, slot or page (synchronises)."""
        ops.check_errors(self.device)

    # ------------------------------------------------------------------ accounting
    def weight_bytes_per_step(self) -> int:
        return self.model.weight_bytes_per_step()

    def kv_bytes_per_token(self) -> int:
        return self.store.kv_bytes_per_token()


__all__ = ["ModelRunner", "StepEntry", "StepInputError"]
