"""What one step hands to the model: a token-major ragged batch and its metadata.

``StepEntry`` is (request, its next tokens, the places among them whose logits
are wanted).  ``build_context`` reserves pages for every entry, lays all step
metadata out in one host buffer (token ids, positions, row ranges, lengths, and
per cache group the block tables and slot mapping) and moves it to the device
with one copy.  The reference rebuilds five small device tensors per forward
from Python lists instead (slipstream/memory/paged_cache.py:71-109) and needs the
same number of new tokens for every row of a forward.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from slipstream_b200.cache import CacheManager

ATTN_TILE_ROWS = 16  # query tokens per tile of the SIMT attention kernel


@dataclass
class StepEntry:
    request_id: object
    tokens: list[int]
    want: list[int] = field(default_factory=list)


@dataclass
class GroupMeta:
    block_tables: torch.Tensor  # int32 [R, max_blocks] on the device, -1 where no page
    slot_mapping: torch.Tensor  # int32 [N]: page * page_size + offset of each new token
    page_size: int
    max_blocks: int


@dataclass
class StepContext:
    num_tokens: int
    num_requests: int
    token_ids: torch.Tensor  # int32 [N]
    positions: torch.Tensor  # int32 [N]
    q_start: torch.Tensor  # int32 [R + 1]: rows of request r are q_start[r] .. q_start[r+1]
    seq_lens: torch.Tensor  # int32 [R]: tokens of the request in the cache after this step
    state_slots: torch.Tensor  # int32 [R]: row of the state pool
    first_chunk: torch.Tensor  # int32 [R]: 1 when the request had nothing cached before this step
    logit_rows: torch.Tensor  # int32 [M]: rows whose logits are wanted
    groups: list[GroupMeta]
    q_lens_host: np.ndarray
    seq_lens_host: np.ndarray
    request_ids: list[object]
    device: torch.device
    num_logits: int = 0
    _tiles: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = field(default_factory=dict)
    extras: dict[str, object] = field(default_factory=dict)
    # the static context of a captured step: a function that hands out static device buffers for a list of tiles
    # ((kind, rows, group) -> (requests, first rows)), which the graph refills before every replay
    static_tiles: object = None

    @property
    def max_q_len(self) -> int:
        return int(self.q_lens_host.max()) if self.num_requests else 0

    @property
    def max_seq_len(self) -> int:
        return int(self.seq_lens_host.max()) if self.num_requests else 0

    @property
    def is_decode_only(self) -> bool:
        return self.num_requests > 0 and self.max_q_len == 1

    def query_tiles(self, rows: int = ATTN_TILE_ROWS, group: int = 1) -> tuple[torch.Tensor, torch.Tensor]:
        """(request index, first row within the request) of every tile of ``rows`` consecutive rows, as
        int32 device tensors.  A request has ``q_len * group`` rows: with ``group`` 1 a row is a query
        token; with the size of a kv group it is a (token, head of the group) pair."""
        key = (rows, group)
        cached = self._tiles.get(key)
        if cached is None and self.static_tiles is not None:  # the context of a captured step
            cached = self._tiles[key] = self.static_tiles(("in_order", rows, group))
        if cached is None:
            req, q0 = query_tiles_host(self.q_lens_host * group, rows)
            # through pinned memory: a copy from pageable memory would hold the host until every kernel queued
            # before it has run, and the first layer of the step would be launched one kernel at a time
            if self.device.type == "cuda":
                staged = torch.empty(2 * req.size, dtype=torch.int32, pin_memory=True)
                staged.numpy()[: req.size] = req
                staged.numpy()[req.size:] = q0
            else:
                staged = torch.from_numpy(np.concatenate([req, q0]))
            both = staged.to(self.device, non_blocking=True)
            cached = (both[: req.size], both[req.size:])
            self._tiles[key] = cached
        return cached

    def query_tiles_longest_first(self, rows: int) -> tuple[torch.Tensor, torch.Tensor]:
        """``query_tiles(rows)`` ordered by falling number of keys a tile sees (its last token's position): a kernel
        whose blocks take one tile each and start in index order then starts its longest blocks first."""
        key = ("longest_first", rows)
        cached = self._tiles.get(key)
        if cached is None and self.static_tiles is not None:
            cached = self._tiles[key] = self.static_tiles(("longest_first", rows, 1))
        if cached is None:
            req, q0 = query_tiles_longest_first_host(self.q_lens_host, self.seq_lens_host, rows)
            staged = torch.empty(2 * req.size, dtype=torch.int32, pin_memory=self.device.type == "cuda")
            staged.numpy()[: req.size] = req
            staged.numpy()[req.size:] = q0
            both = staged.to(self.device, non_blocking=True)
            cached = self._tiles[key] = (both[: req.size], both[req.size:])
        return cached

    def set_query_tiles(self, rows: int, group: int, tile_req: torch.Tensor, tile_first: torch.Tensor) -> None:
        """Fix the answer of ``query_tiles(rows, group)`` (a part does this for the static context of a graph)."""
        self._tiles[(rows, group)] = (tile_req, tile_first)


def query_tiles_host(q_lens: np.ndarray, rows: int) -> tuple[np.ndarray, np.ndarray]:
    counts = (q_lens + rows - 1) // rows
    req = np.repeat(np.arange(q_lens.size, dtype=np.int32), counts)
    first = np.cumsum(counts) - counts
    q0 = (np.arange(int(counts.sum()), dtype=np.int32) - np.repeat(first, counts).astype(np.int32)) * rows
    return req.astype(np.int32), q0.astype(np.int32)


def query_tiles_longest_first_host(q_lens: np.ndarray, seq_lens: np.ndarray, rows: int) -> tuple[np.ndarray, np.ndarray]:
    """The tiles of ``query_tiles_host`` by falling position of their last token (the number of keys they see)."""
    req, q0 = query_tiles_host(q_lens, rows)
    q_lens = np.asarray(q_lens, dtype=np.int64)
    last = (np.asarray(seq_lens, dtype=np.int64) - q_lens)[req] + np.minimum(q0 + rows, q_lens[req]) - 1
    order = np.argsort(-last, kind="stable")
    return req[order], q0[order]


class StepInputError(ValueError):
    """A step was asked for something it cannot run (checked on the host before any launch)."""


@dataclass
class HostPlan:
    """The step's metadata as host arrays, before it goes to the device."""

    entries: list[StepEntry]
    q_lens: np.ndarray
    token_ids: np.ndarray
    positions: np.ndarray
    q_start: np.ndarray
    seq_lens: np.ndarray
    slots: np.ndarray
    first: np.ndarray
    logit_rows: np.ndarray
    tables: list[np.ndarray]  # per cache group [R, max_blocks of that group]
    slot_maps: np.ndarray  # [groups, N]
    page_sizes: list[int]  # per cache group
    requests: list = field(default_factory=list)  # the cache manager's record of each entry's request

    @property
    def num_requests(self) -> int:
        return self.q_lens.size

    @property
    def num_tokens(self) -> int:
        return self.token_ids.size

    @property
    def is_decode_only(self) -> bool:
        return bool((self.q_lens == 1).all())


def plan_step(entries: list[StepEntry], cache: CacheManager, vocab_size: int, reserve: bool = True,
              with_tables: bool = True) -> HostPlan:
    """Check the entries, reserve their pages and lay the step's metadata out in host arrays.  ``with_tables``
    False leaves the block tables out (``plan.tables`` is empty and ``plan.requests`` holds the cache manager's
    records instead): a replayed decode graph keeps its tables on the device and only patches them."""
    if not entries:
        raise StepInputError("a step needs at least one entry")
    seen: set[object] = set()
    for e in entries:
        if e.request_id in seen:
            raise StepInputError(f"request {e.request_id!r} appears twice in one step")
        seen.add(e.request_id)
        if len(e.tokens) < 1:
            raise StepInputError(f"request {e.request_id!r} brings no tokens")
        for w in e.want:
            if not 0 <= w < len(e.tokens):
                raise StepInputError(f"request {e.request_id!r}: wanted place {w} is outside its "
                                     f"{len(e.tokens)} tokens")
    R = len(entries)
    q_lens = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=R)
    N = int(q_lens.sum())
    token_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
    if token_ids.min() < 0 or token_ids.max() >= vocab_size:
        raise StepInputError(f"a token id is outside [0, {vocab_size})")
    if reserve:
        for e in entries:
            cache.reserve(e.request_id, len(e.tokens))
    reqs = [cache.get(e.request_id) for e in entries]
    before = np.fromiter((r.length for r in reqs), dtype=np.int32, count=R)
    seq_lens = (before + q_lens).astype(np.int32)
    q_start = np.zeros(R + 1, dtype=np.int32)
    np.cumsum(q_lens, out=q_start[1:])
    row_req = np.repeat(np.arange(R, dtype=np.int32), q_lens)
    positions = (np.arange(N, dtype=np.int32) - q_start[:-1][row_req] + before[row_req]).astype(np.int32)
    logit_rows = np.fromiter((q_start[i] + w for i, e in enumerate(entries) for w in e.want), dtype=np.int32)
    slots = np.fromiter((r.slot for r in reqs), dtype=np.int32, count=R)
    first = (before == 0).astype(np.int32)

    n_groups = len(cache.groups)
    longest = int(seq_lens.max())
    tables = []
    slot_maps = np.empty((n_groups, N), dtype=np.int32)
    for g in range(n_groups):
        ps = cache.page_sizes[g]
        if not with_tables:  # one token per request, or few: look the pages up directly
            try:
                pages = np.fromiter((reqs[i].tables[g][p // ps] for i, p in zip(row_req.tolist(), positions.tolist())),
                                    dtype=np.int32, count=N)
            except IndexError:
                raise StepInputError("a new token falls on a block without a page") from None
            if (pages < 0).any():
                raise StepInputError("a new token falls on a block without a page")
            slot_maps[g] = pages * ps + positions % ps
            continue
        max_blocks = max(1, (longest + ps - 1) // ps)
        table = np.full((R, max_blocks), -1, dtype=np.int32)
        for i, r in enumerate(reqs):
            t = r.tables[g][:max_blocks]
            table[i, : len(t)] = t
        pages = table[row_req, positions // ps]
        if (pages < 0).any():
            raise StepInputError("a new token falls on a block without a page")
        slot_maps[g] = pages * ps + positions % ps
        tables.append(table)
    return HostPlan(entries, q_lens, token_ids.astype(np.int32), positions, q_start, seq_lens, slots, first,
                    logit_rows, tables, slot_maps, list(cache.page_sizes), reqs)


def to_device(plan: HostPlan, device: torch.device) -> StepContext:
    """One host buffer, one copy, then views of it."""
    R, N = plan.num_requests, plan.num_tokens
    n_groups = len(plan.tables)
    parts = [plan.token_ids, plan.positions, plan.q_start, plan.seq_lens, plan.slots, plan.first,
             plan.logit_rows, plan.slot_maps.reshape(-1)] + [t.reshape(-1) for t in plan.tables]
    sizes = [p.size for p in parts]
    host = torch.empty(int(sum(sizes)), dtype=torch.int32, pin_memory=torch.cuda.is_available())
    np.concatenate(parts, out=host.numpy())
    dev = host.to(device, non_blocking=True)
    offs = np.concatenate([[0], np.cumsum(sizes)])
    cut = [dev[offs[i]: offs[i + 1]] for i in range(len(parts))]
    groups = []
    for g in range(n_groups):
        max_blocks = plan.tables[g].shape[1]
        groups.append(GroupMeta(block_tables=cut[8 + g].view(R, max_blocks), slot_mapping=cut[7][g * N: (g + 1) * N],
                                page_size=plan.page_sizes[g], max_blocks=max_blocks))
    ctx = StepContext(num_tokens=N, num_requests=R, token_ids=cut[0], positions=cut[1], q_start=cut[2],
                      seq_lens=cut[3], state_slots=cut[4], first_chunk=cut[5], logit_rows=cut[6],
                      groups=groups, q_lens_host=plan.q_lens, seq_lens_host=plan.seq_lens,
                      request_ids=[e.request_id for e in plan.entries], device=device,
                      num_logits=plan.logit_rows.size)
    ctx.extras["host_buffer"] = host  # keep the pinned buffer alive until the copy has run
    # every row's logits, in order: the final norm needs no selection of rows
    ctx.extras["every_row_wanted"] = plan.logit_rows.size == N and bool((plan.logit_rows == np.arange(N)).all())
    return ctx


def build_context(entries: list[StepEntry], cache: CacheManager, vocab_size: int, device: torch.device,
                  reserve: bool = True) -> StepContext:
    return to_device(plan_step(entries, cache, vocab_size, reserve), device)
