"""CUDA graphs for decode steps.

A step in which every request brings one token launches a few hundred small
kernels; at batch 1 the launches cost more than the kernels.  For such steps the
runner captures the whole forward once per batch-size bucket and replays it.
The captured step reads its metadata (token ids, positions, lengths, block
tables, slot mapping) from a static device buffer that is refilled by one copy
before each replay; rows beyond the live requests are padding (length 0, slot
-1), which every kernel skips.  The split of the decode attention over the keys
is fixed per bucket, so grids do not depend on the lengths.

The reference has a ``CudaGraphPool`` keyed by batch size that was never wired
into its serving loop (slipstream/engine/cuda_graph.py:1-93).
"""

from __future__ import annotations

import gc

import numpy as np
import torch

from slipstream_b200 import ops

from .context import GroupMeta, HostPlan, StepContext

BUCKETS = [1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512]
HOST_RING = 4


def bucket_for(n: int) -> int | None:
    for b in BUCKETS:
        if n <= b:
            return b
    return None


class DecodeGraph:
    def __init__(self, runner, bucket: int, wide: bool = False) -> None:
        self.runner = runner
        self.bucket = bucket
        self.wide = wide  # captured for long contexts: attention may cut the keys into more than 8 slices
        cache = runner.cache
        self.n_groups = len(cache.groups)
        self.max_blocks = max(1, (runner.max_model_len + cache.page_size - 1) // cache.page_size)
        B, G, MB = bucket, self.n_groups, self.max_blocks
        names = ["token_ids", "positions", "q_start", "seq_lens", "slots", "first", "logit_rows", "src_rows",
                 "tables", "slot_maps"]
        sizes = [B, B, B + 1, B, B, B, B, B, G * B * MB, G * B]
        self.offsets = dict(zip(names, np.concatenate([[0], np.cumsum(sizes)])[:-1].tolist()))
        self.sizes = dict(zip(names, sizes))
        total = int(sum(sizes))
        device = runner.device
        self.static = torch.zeros(total, dtype=torch.int32, device=device)
        self.hosts = [torch.zeros(total, dtype=torch.int32, pin_memory=True) for _ in range(HOST_RING)]
        self.events: list[torch.cuda.Event | None] = [None] * HOST_RING
        self.turn = 0

        def view(name: str) -> torch.Tensor:
            o = self.offsets[name]
            return self.static[o: o + self.sizes[name]]

        groups = []
        for g in range(G):
            groups.append(GroupMeta(block_tables=view("tables")[g * B * MB: (g + 1) * B * MB].view(B, MB),
                                    slot_mapping=view("slot_maps")[g * B: (g + 1) * B],
                                    page_size=cache.page_size, max_blocks=MB))
        ones = np.ones(B, dtype=np.int32)
        self.ctx = StepContext(num_tokens=B, num_requests=B, token_ids=view("token_ids"),
                               positions=view("positions"), q_start=view("q_start"), seq_lens=view("seq_lens"),
                               state_slots=view("slots"), first_chunk=view("first"), logit_rows=view("logit_rows"),
                               groups=groups, q_lens_host=ones, seq_lens_host=ones, request_ids=[], device=device,
                               num_logits=B)
        self.ctx.extras["static_max_seq_len"] = runner.max_model_len
        self.ctx.extras["decode_wide"] = wide
        arange = torch.arange(B, dtype=torch.int32, device=device)
        self.ctx._tiles[(16, 1)] = (arange, torch.zeros(B, dtype=torch.int32, device=device))
        self._fill(self.hosts[0].numpy(), None)
        self.static.copy_(self.hosts[0])
        # warm up outside the capture (library handles, lazily compiled kernels), then capture
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            runner.model.forward(self.ctx)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(device)
        self.graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        # Python's collector must not run inside the capture: if it frees a dead object that owns pinned memory
        # or another graph (an engine that is no longer used), the calls that frees make invalidate the capture
        gc.collect()
        collector_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph):
                self.logits = runner.model.forward(self.ctx)
        finally:
            if collector_was_on:
                gc.enable()
        self.kernels = ops.launch_count() - before

    def _fill(self, host: np.ndarray, plan: HostPlan | None) -> None:
        B, MB, G = self.bucket, self.max_blocks, self.n_groups
        o = self.offsets
        host[:] = 0
        host[o["q_start"]: o["q_start"] + B + 1] = np.arange(B + 1, dtype=np.int32)
        host[o["logit_rows"]: o["logit_rows"] + B] = np.arange(B, dtype=np.int32)
        host[o["tables"]: o["tables"] + G * B * MB] = -1
        host[o["slot_maps"]: o["slot_maps"] + G * B] = -1
        host[o["src_rows"]: o["src_rows"] + B] = -1
        if plan is None:
            return
        R = plan.num_requests
        for name, arr in (("token_ids", plan.token_ids), ("positions", plan.positions),
                          ("seq_lens", plan.seq_lens), ("slots", plan.slots), ("first", plan.first)):
            host[o[name]: o[name] + R] = arr
        mb = plan.tables.shape[2]
        tables = host[o["tables"]: o["tables"] + G * B * MB].reshape(G, B, MB)
        tables[:, :R, :mb] = plan.tables
        host[o["slot_maps"]: o["slot_maps"] + G * B].reshape(G, B)[:, :R] = plan.slot_maps

    def run(self, plan: HostPlan, pending: torch.Tensor | None = None, src_rows: np.ndarray | None = None,
            keep: bool = True) -> torch.Tensor:
        """Refill the static metadata, replay the step, return the logits of the wanted rows.

        ``pending`` / ``src_rows``: token ids that are still on the device (sampled by the step before): row r
        takes ``pending[src_rows[r]]`` where ``src_rows[r] >= 0``.  ``keep`` False returns a view of the static
        logits buffer, valid until the next replay."""
        i = self.turn
        self.turn = (i + 1) % HOST_RING
        if self.events[i] is not None:
            self.events[i].synchronize()  # the copy that last used this host buffer has run
        host = self.hosts[i].numpy()
        self._fill(host, plan)
        if src_rows is not None:
            o = self.offsets["src_rows"]
            host[o: o + src_rows.size] = src_rows
        self.static.copy_(self.hosts[i], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.events[i] = event
        if pending is not None:
            o = self.offsets
            ops.gather_tokens(self.static[o["token_ids"]: o["token_ids"] + self.bucket],
                              self.static[o["src_rows"]: o["src_rows"] + self.bucket], pending)
        self.graph.replay()
        ops.count_launches(self.kernels)
        R = plan.num_requests
        if not keep and plan.logit_rows.size == R and bool((plan.logit_rows == np.arange(R)).all()):
            return self.logits[:R]
        if plan.logit_rows.size == R and bool((plan.logit_rows == np.arange(R)).all()):
            return self.logits[:R].clone()
        if plan.logit_rows.size == 0:
            return self.logits[:0].clone()
        rows = torch.from_numpy(plan.logit_rows.astype(np.int64)).to(self.runner.device)
        return self.logits.index_select(0, rows)

    @property
    def h2d_bytes(self) -> int:
        return self.static.numel() * 4
