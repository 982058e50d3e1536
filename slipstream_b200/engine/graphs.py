"""CUDA graphs for decode steps.

A step in which every request brings one token launches a few hundred small
kernels; at batch 1 the launches cost more than the kernels.  For such steps the
runner captures the whole forward once per batch-size bucket and replays it.
The captured step reads its metadata (token ids, positions, lengths, slot
mapping) from a small static device buffer that is refilled by one copy before
each replay; rows beyond the live requests are padding (length 0, slot -1), which
every kernel skips.

The block tables stay on the device from step to step.  A decode step changes at
most one entry per request and cache group (a newly reserved page; in a windowed
group also the pages the window has passed), so the host sends only those changes
as (index, value) patches inside the same small copy, and the kernel in front of
the replay applies them.  When a row of the batch goes to another request its whole
row is patched; a step with more changes than the patch area holds (many requests
arriving at once) copies the host's mirror of the tables instead.

What a part's forward would take from the host-side lengths of a step (how many
slices the decode attention cuts the keys into, say) is fixed when the graph is
captured: every part gets ``prepare_capture`` on the static context, and parts whose
best form depends on the lengths say so through ``capture_variant``; the runner keeps
one graph per bucket and combination of variants.

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
    def __init__(self, runner, bucket: int, variants: tuple = ()) -> None:
        self.runner = runner
        self.bucket = bucket
        self.variants = variants
        cache = runner.cache
        G = self.n_groups = len(cache.groups)
        B = bucket
        self.max_blocks = [max(1, (runner.max_model_len + ps - 1) // ps) for ps in cache.page_sizes]
        self.table_offsets = np.concatenate([[0], np.cumsum([B * mb for mb in self.max_blocks])]).astype(np.int64)
        self.max_patches = max(64, 4 * B * max(G, 1))
        P = self.max_patches
        names = ["token_ids", "positions", "q_start", "seq_lens", "slots", "first", "logit_rows", "src_rows",
                 "slot_maps", "n_patches", "patch_idx", "patch_val"]
        sizes = [B, B, B + 1, B, B, B, B, B, G * B, 1, P, P]
        self.offsets = dict(zip(names, np.concatenate([[0], np.cumsum(sizes)])[:-1].tolist()))
        self.sizes = dict(zip(names, sizes))
        total = int(sum(sizes))
        device = runner.device
        self.static = torch.zeros(total, dtype=torch.int32, device=device)
        self.hosts = [torch.zeros(total, dtype=torch.int32, pin_memory=True) for _ in range(HOST_RING)]
        self.events: list[torch.cuda.Event] = [torch.cuda.Event() for _ in range(HOST_RING)]
        self.used = [False] * HOST_RING
        self.turn = 0
        # block tables: on the device for good, mirrored on the host
        n_table = max(1, int(self.table_offsets[-1]))
        self.tables_dev = torch.full((n_table,), -1, dtype=torch.int32, device=device)
        self.tables_host = torch.full((n_table,), -1, dtype=torch.int32, pin_memory=True)
        self.mirror = self.tables_host.numpy()
        self.mirror_event: torch.cuda.Event | None = None  # a copy of the whole mirror that may still be running
        self.row_owner: list[object] = [None] * B  # the cache manager's record of the request whose table each row holds
        self.row_synced = [[0] * B for _ in range(G)]  # entries of the request's table that the row holds
        self.row_first = [[0] * B for _ in range(G)]  # first block not yet given back, as the row knows it
        self.full_copies = 0

        def view(name: str) -> torch.Tensor:
            o = self.offsets[name]
            return self.static[o: o + self.sizes[name]]

        groups = []
        for g in range(G):
            mb, o = self.max_blocks[g], int(self.table_offsets[g])
            groups.append(GroupMeta(block_tables=self.tables_dev[o: o + B * mb].view(B, mb),
                                    slot_mapping=view("slot_maps")[g * B: (g + 1) * B],
                                    page_size=cache.page_sizes[g], max_blocks=mb))
        ones = np.ones(B, dtype=np.int32)
        self.ctx = StepContext(num_tokens=B, num_requests=B, token_ids=view("token_ids"),
                               positions=view("positions"), q_start=view("q_start"), seq_lens=view("seq_lens"),
                               state_slots=view("slots"), first_chunk=view("first"), logit_rows=view("logit_rows"),
                               groups=groups, q_lens_host=ones, seq_lens_host=ones, request_ids=[], device=device,
                               num_logits=B)
        self.ctx.extras["every_row_wanted"] = True  # logit_rows is 0 .. B - 1 in every replay
        self._views = {name: view(name) for name in ("token_ids", "src_rows", "n_patches", "patch_idx", "patch_val")}
        # what the parts want fixed for this bucket and these variants
        variant_of = {part.capture_group(): variant for part, variant in zip(runner.variant_parts, variants)}
        for part in runner.model.parts():
            part.prepare_capture(self.ctx, variant_of.get(part.capture_group()), runner.max_model_len)
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

    # ------------------------------------------------------------------ per step
    def _fill(self, host: np.ndarray, plan: HostPlan | None) -> None:
        B, G = self.bucket, self.n_groups
        o = self.offsets
        host[: o["patch_idx"]] = 0
        host[o["q_start"]: o["q_start"] + B + 1] = np.arange(B + 1, dtype=np.int32)
        host[o["logit_rows"]: o["logit_rows"] + B] = np.arange(B, dtype=np.int32)
        host[o["slot_maps"]: o["slot_maps"] + G * B] = -1
        host[o["src_rows"]: o["src_rows"] + B] = -1
        if plan is None:
            return
        R = plan.num_requests
        for name, arr in (("token_ids", plan.token_ids), ("positions", plan.positions),
                          ("seq_lens", plan.seq_lens), ("slots", plan.slots), ("first", plan.first)):
            host[o[name]: o[name] + R] = arr
        host[o["slot_maps"]: o["slot_maps"] + G * B].reshape(G, B)[:, :R] = plan.slot_maps

    def _table_changes(self, plan: HostPlan) -> tuple[list[int], list[int]]:
        """Bring the host's mirror of the block tables up to this step and return what changed as (flat index,
        value) lists.  Row i of the batch holds the table of ``plan.requests[i]``."""
        idx: list[int] = []
        val: list[int] = []
        if self.mirror_event is not None:  # the mirror must not change under a copy of it
            self.mirror_event.synchronize()
            self.mirror_event = None
        mirror = self.mirror
        for i, req in enumerate(plan.requests):
            # the manager's record itself, not the request's name: a request that was preempted and admitted again
            # keeps its name but starts a new table
            fresh = self.row_owner[i] is not req
            if fresh:
                self.row_owner[i] = req
            for g in range(self.n_groups):
                table = req.tables[g]
                base = int(self.table_offsets[g]) + i * self.max_blocks[g]
                synced = 0 if fresh else self.row_synced[g][i]
                first_known = 0 if fresh else self.row_first[g][i]
                first = req.first_block[g]
                if first > first_known and not fresh:  # pages a window has passed
                    for b in range(first_known, min(first, synced)):
                        idx.append(base + b)
                        val.append(-1)
                        mirror[base + b] = -1
                if len(table) > synced:
                    new = table[synced:]
                    idx.extend(range(base + synced, base + len(table)))
                    val.extend(new)
                    mirror[base + synced: base + len(table)] = new
                self.row_synced[g][i] = len(table)
                self.row_first[g][i] = first
        return idx, val

    def run(self, plan: HostPlan, pending: torch.Tensor | None = None, src_rows: np.ndarray | None = None,
            keep: bool = True) -> torch.Tensor:
        """Refill the static metadata, patch the tables, replay the step, return the logits of the wanted rows.

        ``pending`` / ``src_rows``: token ids that are still on the device (sampled by the step before): row r
        takes ``pending[src_rows[r]]`` where ``src_rows[r] >= 0``.  ``keep`` False returns a view of the static
        logits buffer, valid until the next replay."""
        i = self.turn
        self.turn = (i + 1) % HOST_RING
        if self.used[i]:
            self.events[i].synchronize()  # the copy that last used this host buffer has run
        host = self.hosts[i].numpy()
        self._fill(host, plan)
        o = self.offsets
        if src_rows is not None:
            host[o["src_rows"]: o["src_rows"] + src_rows.size] = src_rows
        idx, val = self._table_changes(plan)
        if len(idx) <= self.max_patches:
            host[o["n_patches"]] = len(idx)
            host[o["patch_idx"]: o["patch_idx"] + len(idx)] = idx
            host[o["patch_val"]: o["patch_val"] + len(idx)] = val
        else:  # too many changes for the patch area: send the whole mirror
            self.tables_dev.copy_(self.tables_host, non_blocking=True)
            self.mirror_event = torch.cuda.Event()
            self.mirror_event.record()
            self.full_copies += 1
        self.static.copy_(self.hosts[i], non_blocking=True)
        self.events[i].record()
        self.used[i] = True
        v = self._views
        ops.prepare_decode(v["token_ids"], v["src_rows"], pending, self.tables_dev, v["patch_idx"], v["patch_val"],
                           v["n_patches"])
        self.graph.replay()
        ops.count_launches(self.kernels)
        R = plan.num_requests
        in_order = plan.logit_rows.size == R and bool((plan.logit_rows == np.arange(R)).all())
        if in_order:
            return self.logits[:R] if not keep else self.logits[:R].clone()
        if plan.logit_rows.size == 0:
            return self.logits[:0].clone()
        rows = torch.from_numpy(plan.logit_rows.astype(np.int64)).to(self.runner.device)
        return self.logits.index_select(0, rows)

    @property
    def h2d_bytes(self) -> int:
        """Bytes the host sends per replay (the small static buffer; the tables travel as patches inside it)."""
        return self.static.numel() * 4


# =========================================================================== steps with prompt portions
TOKEN_BUCKETS = ([16, 32] + [64 * k for k in range(1, 11)] + [768, 896, 1024, 1152, 1280, 1536, 1792, 2048, 2304])
REQUEST_BUCKETS = [4, 8, 16, 32, 64, 128, 256]
PADDING_TILE_FIRST = 1 << 24  # "first row" of a tile that holds no row: every kernel returns at once on such a tile


def mixed_bucket(n_tokens: int, n_requests: int) -> tuple[int, int] | None:
    tokens = next((b for b in TOKEN_BUCKETS if n_tokens <= b), None)
    requests = next((b for b in REQUEST_BUCKETS if n_requests <= b), None)
    return None if tokens is None or requests is None else (tokens, requests)


class MixedGraph:
    """A captured step of up to ``n_tokens`` tokens of up to ``n_requests`` requests, prompt portions beside
    decoded tokens.  A step of a small model launches a few hundred kernels that the host needs longer to launch
    than the GPU to run (a 24-layer model: 3.4 ms of launches for under 1 ms of work); replayed from a graph it
    costs the host one copy and one launch.

    The captured step always runs ``n_tokens`` rows and ``n_requests`` requests.  Rows beyond the live tokens are
    padding (token 0, slot -1: nothing is written to the cache; their activations are computed and never read),
    requests beyond the live ones are empty, and the lists of query tiles the attention kernels walk are padded
    with tiles that hold no row.  All metadata, the block tables and the tile lists lie in one static device buffer
    that one copy refills before each replay."""

    def __init__(self, runner, n_tokens: int, n_requests: int, n_logits: int, variants: tuple = ()) -> None:
        """``n_logits``: rows whose logits a step may ask for (a serving step wants one per request at most, a
        replayed trace up to one per token)."""
        self.runner = runner
        self.n_tokens, self.n_requests, self.n_logits = N, R, L = n_tokens, n_requests, n_logits
        cache = runner.cache
        G = self.n_groups = len(cache.groups)
        self.max_blocks = [max(1, (runner.max_model_len + ps - 1) // ps) for ps in cache.page_sizes]
        self.tile_capacity = 2 * N + R  # entries per list: the most tiles a step has while a tile holds 64 rows of a
        # group of up to 128 heads, or 16 tokens
        self.max_tile_lists = 4
        names = ["token_ids", "positions", "q_start", "seq_lens", "slots", "first", "logit_rows", "slot_maps"]
        sizes = [N, N, R + 1, R, R, R, L, G * N]
        names += [f"table{g}" for g in range(G)]
        sizes += [R * mb for mb in self.max_blocks]
        names += ["tiles"]
        sizes += [self.max_tile_lists * 2 * self.tile_capacity]
        self.offsets = dict(zip(names, np.concatenate([[0], np.cumsum(sizes)])[:-1].tolist()))
        self.sizes = dict(zip(names, sizes))
        total = int(sum(sizes))
        device = runner.device
        self.static = torch.zeros(total, dtype=torch.int32, device=device)
        self.hosts = [torch.zeros(total, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.events = [torch.cuda.Event() for _ in range(2)]
        self.used = [False, False]
        self.turn = 0
        self.tile_keys: list[tuple] = []  # (kind, rows, group) of every tile list the parts asked for

        def view(name: str) -> torch.Tensor:
            o = self.offsets[name]
            return self.static[o: o + self.sizes[name]]

        groups = [GroupMeta(block_tables=view(f"table{g}").view(R, self.max_blocks[g]),
                            slot_mapping=view("slot_maps")[g * N: (g + 1) * N], page_size=cache.page_sizes[g],
                            max_blocks=self.max_blocks[g]) for g in range(G)]
        self.ctx = StepContext(num_tokens=N, num_requests=R, token_ids=view("token_ids"), positions=view("positions"),
                               q_start=view("q_start"), seq_lens=view("seq_lens"), state_slots=view("slots"),
                               first_chunk=view("first"), logit_rows=view("logit_rows"), groups=groups,
                               # lengths are not known on the host inside a replay; 2 only says "not one token each"
                               q_lens_host=np.full(R, 2, dtype=np.int32), seq_lens_host=np.zeros(R, dtype=np.int32),
                               request_ids=[], device=device, num_logits=L, static_tiles=self._static_tiles)
        variant_of = {part.capture_group(): variant for part, variant in zip(runner.variant_parts, variants)}
        for part in runner.model.parts():
            part.prepare_capture(self.ctx, variant_of.get(part.capture_group()), runner.max_model_len)
        self._fill(self.hosts[0].numpy(), None)
        self.static.copy_(self.hosts[0])
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            runner.model.forward(self.ctx)  # also tells which tile lists the parts want
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(device)
        self.graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
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

    def _static_tiles(self, key: tuple) -> tuple[torch.Tensor, torch.Tensor]:
        if key not in self.tile_keys:
            if len(self.tile_keys) == self.max_tile_lists:
                raise RuntimeError("a captured step has room for four lists of query tiles")
            self.tile_keys.append(key)
        o = self.offsets["tiles"] + self.tile_keys.index(key) * 2 * self.tile_capacity
        _kind, rows, group = key
        count = (self.n_tokens * group + rows - 1) // rows + self.n_requests  # the most tiles a step can have
        if count > self.tile_capacity:
            raise RuntimeError("the tile list of a captured step is too long for its buffer")
        return self.static[o: o + count], self.static[o + self.tile_capacity: o + self.tile_capacity + count]

    def _fill(self, host: np.ndarray, plan: HostPlan | None) -> None:
        N, R, G = self.n_tokens, self.n_requests, self.n_groups
        o = self.offsets
        host[: o["table0"] if G else o["tiles"]] = 0
        host[o["slot_maps"]: o["slot_maps"] + G * N] = -1
        tiles = host[o["tiles"]: o["tiles"] + self.sizes["tiles"]].reshape(self.max_tile_lists, 2, self.tile_capacity)
        tiles[:, 0, :] = 0
        tiles[:, 1, :] = PADDING_TILE_FIRST
        if plan is None:
            return
        n, r = plan.num_tokens, plan.num_requests
        host[o["token_ids"]: o["token_ids"] + n] = plan.token_ids
        host[o["positions"]: o["positions"] + n] = plan.positions
        host[o["q_start"]: o["q_start"] + r + 1] = plan.q_start
        host[o["q_start"] + r + 1: o["q_start"] + R + 1] = n  # the requests behind the live ones are empty
        for name, arr in (("seq_lens", plan.seq_lens), ("slots", plan.slots), ("first", plan.first)):
            host[o[name]: o[name] + r] = arr
        host[o["logit_rows"]: o["logit_rows"] + plan.logit_rows.size] = plan.logit_rows
        host[o["slot_maps"]: o["slot_maps"] + G * N].reshape(G, N)[:, :n] = plan.slot_maps
        for g in range(G):
            table = plan.tables[g]
            host[o[f"table{g}"]: o[f"table{g}"] + R * self.max_blocks[g]].reshape(R, self.max_blocks[g])[:r, : table.shape[1]] = table
        from .context import query_tiles_host, query_tiles_longest_first_host
        for i, (kind, rows, group) in enumerate(self.tile_keys):
            if kind == "longest_first":
                req, first = query_tiles_longest_first_host(plan.q_lens, plan.seq_lens, rows)
            else:
                req, first = query_tiles_host(plan.q_lens * group, rows)
            tiles[i, 0, : req.size] = req
            tiles[i, 1, : req.size] = first

    def run(self, plan: HostPlan) -> torch.Tensor:
        i = self.turn
        self.turn ^= 1
        if self.used[i]:
            self.events[i].synchronize()
        self._fill(self.hosts[i].numpy(), plan)
        self.static.copy_(self.hosts[i], non_blocking=True)
        self.events[i].record()
        self.used[i] = True
        self.graph.replay()
        ops.count_launches(self.kernels)
        return self.logits[: plan.logit_rows.size].clone()

    @property
    def h2d_bytes(self) -> int:
        return self.static.numel() * 4
