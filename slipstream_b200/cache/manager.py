"""Cache manager: pages of keys and values, block tables, fixed-size state slots.

Layers are grouped by what they need from the cache (``CacheSpec``: key/value
heads, head size, window, page size).  Each group has its own page pool, with its
own page size and number of pages, and each request has one block table per group;
a page id is valid for every layer of its group, as in the reference's single pool
(slipstream/memory/paged_cache.py:13-28).  Pages
come from a LIFO free list (slipstream/memory/block_manager.py:42,272-280), so a
page given back is the next one handed out.  Pages return when a request is
released (:169-181) or, in a windowed group, as soon as no later query can see
any key in them.  Beside the pages, every live request owns one slot of the
fixed-size state pool.

The manager is host-side bookkeeping only (no tensors) so that it can be tested
without a device; ``PagedStore`` holds the device memory.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

from slipstream_b200.parts.base import CacheSpec


class AllocStatus(Enum):
    """slipstream/core/types.py:55-60."""

    OK = "ok"
    LATER = "later"
    NEVER = "never"


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    pass


@dataclass
class GroupLayout:
    """One cache group: the spec its layers share, how many of them write pages, and (once the runner has sized
    the pools) its page size and number of pages."""

    spec: CacheSpec
    num_entries: int = 0
    page_size: int = 0
    num_pages: int = 0


class PagePool:
    """Page ids of one group with a LIFO free list and a holder per page."""

    def __init__(self, num_pages: int) -> None:
        if num_pages < 1:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))  # page 0 is handed out first
        self._holder: list[object | None] = [None] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, holder: object) -> int:
        if not self._free:
            raise OutOfPages("out of KV pages")
        page = self._free.pop()
        if self._holder[page] is not None:
            raise CacheError(f"page {page} on the free list is held by {self._holder[page]!r}")
        self._holder[page] = holder
        return page

    def give_back(self, page: int, holder: object) -> None:
        if not 0 <= page < self.num_pages:
            raise CacheError(f"page {page} is outside the pool")
        if self._holder[page] is None:
            raise CacheError(f"double free of page {page}")
        if self._holder[page] != holder:
            raise CacheError(f"page {page} is held by {self._holder[page]!r}, not {holder!r}")
        self._holder[page] = None
        self._free.append(page)

    def holder(self, page: int) -> object | None:
        return self._holder[page]


@dataclass
class RequestPages:
    """What the manager keeps per live request."""

    request_id: object
    slot: int
    length: int = 0  # tokens whose keys and values are in the cache
    reserved: int = 0  # tokens covered by pages (>= length)
    tables: list[list[int]] = field(default_factory=list)  # per group: logical block -> page or -1
    first_block: list[int] = field(default_factory=list)  # per group: first block still held


def pool_sizes(groups: list[GroupLayout], page_sizes: list[int], tokens: int, max_num_seqs: int,
               max_model_len: int, max_step_tokens: int) -> list[int]:
    """Pages each group needs so that the cache holds ``tokens`` tokens of live requests.  A group that keeps every
    key gets ``tokens / page size`` pages.  A windowed group never holds more of a request than its window plus
    the tokens of one step (pages are reserved for a whole step before the window moves on), so it gets at most
    that for ``max_num_seqs`` requests: its pool is smaller than its neighbours'."""
    sizes = []
    for layout, page in zip(groups, page_sizes):
        pages = max(1, -(-tokens // page))
        window = layout.spec.window
        if window is not None:
            span = min(max_model_len, window + max(1, max_step_tokens))
            pages = min(pages, max_num_seqs * (-(-span // page) + 1))
        sizes.append(pages)
    return sizes


def tokens_that_fit(groups: list[GroupLayout], page_sizes: list[int], bytes_per_token: list[int], budget: int,
                    max_num_seqs: int, max_model_len: int, max_step_tokens: int) -> int:
    """The most tokens whose pools (``pool_sizes``) fit into ``budget`` bytes, at most what ``max_num_seqs``
    requests of ``max_model_len`` tokens need."""
    def cost(tokens: int) -> int:
        pools = pool_sizes(groups, page_sizes, tokens, max_num_seqs, max_model_len, max_step_tokens)
        return sum(n * page * per for n, page, per in zip(pools, page_sizes, bytes_per_token))

    low, high = 1, max_num_seqs * (max_model_len + max(page_sizes, default=1))
    if cost(high) <= budget:
        return high
    while low < high:
        mid = (low + high + 1) // 2
        if cost(mid) <= budget:
            low = mid
        else:
            high = mid - 1
    return low


def _per_group(value, n: int, what: str) -> list[int]:
    values = [int(v) for v in value] if isinstance(value, (list, tuple)) else [int(value)] * n
    if len(values) != n:
        raise ValueError(f"{what}: {len(values)} values for {n} cache groups")
    return values


class CacheManager:
    def __init__(self, groups: list[GroupLayout], num_pages: "int | list[int]", page_size: "int | list[int]",
                 max_num_seqs: int, max_model_len: int) -> None:
        """``num_pages`` and ``page_size``: one value for every group, or one per group."""
        self.groups = groups
        self.page_sizes = _per_group(page_size, len(groups), "page_size")
        counts = _per_group(num_pages, len(groups), "num_pages")
        if any(p < 1 for p in self.page_sizes):
            raise ValueError("page_size must be >= 1")
        if max_num_seqs < 1:
            raise ValueError("max_num_seqs must be >= 1")
        for layout, size, count in zip(groups, self.page_sizes, counts):
            layout.page_size, layout.num_pages = size, count
        self.max_num_seqs = max_num_seqs
        self.max_model_len = max_model_len
        self.pools = [PagePool(count) for count in counts]
        self._free_slots = list(range(max_num_seqs - 1, -1, -1))
        self._requests: dict[object, RequestPages] = {}

    # ------------------------------------------------------------------ queries
    def __contains__(self, request_id: object) -> bool:
        return request_id in self._requests

    def get(self, request_id: object) -> RequestPages:
        try:
            return self._requests[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not live") from None

    def live_requests(self) -> list[object]:
        return list(self._requests)

    def length(self, request_id: object) -> int:
        return self.get(request_id).length

    @property
    def page_size(self) -> int:
        """Page size of the first group (the only one of a model whose layers all need the same)."""
        return self.page_sizes[0] if self.page_sizes else 1

    @property
    def num_pages(self) -> int:
        return self.pools[0].num_pages if self.pools else 0

    def num_free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free if self.pools else 0

    def free_pages(self) -> list[int]:
        return [pool.num_free for pool in self.pools]

    def all_pages_free(self) -> bool:
        return all(pool.num_free == pool.num_pages for pool in self.pools)

    def min_free_pages(self) -> int:
        return min((p.num_free for p in self.pools), default=0)

    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def blocks_for(self, tokens: int, group: int = 0) -> int:
        size = self.page_sizes[group]
        return 0 if tokens <= 0 else (tokens + size - 1) // size

    def _first_needed_block(self, group: int, length: int) -> int:
        """First block that a query at position >= ``length`` can still see."""
        window = self.groups[group].spec.window
        if window is None:
            return 0
        return max(0, length - window + 1) // self.page_sizes[group]

    def pages_needed(self, request_id: object, new_tokens: int) -> list[int]:
        """Pages each group must still hand out to cover ``new_tokens`` more tokens."""
        req = self.get(request_id)
        target = req.length + new_tokens
        if target <= req.reserved:
            return [0] * len(self.groups)
        return [self.blocks_for(target, g) - len(table) for g, table in enumerate(req.tables)]

    def peak_pages(self, group: int, total_tokens: int, chunk: int) -> int:
        """Most pages of ``group`` a request of ``total_tokens`` holds at any time when it is fed
        at most ``chunk`` tokens a step."""
        window = self.groups[group].spec.window
        if window is None:
            return self.blocks_for(total_tokens, group)
        span = min(total_tokens, window + max(chunk, 1))
        return min(self.blocks_for(total_tokens, group), self.blocks_for(span, group) + 1)

    def can_admit(self, total_tokens: int, first_tokens: int, chunk: int) -> AllocStatus:
        """Three-way answer of slipstream/memory/block_manager.py:108-128: NEVER when the request at
        its full length (``total_tokens`` = prompt + output cap, capped by the context) cannot fit in
        an empty pool of some group; LATER when pages of some group or a slot for its first
        ``first_tokens`` are missing now."""
        total = min(total_tokens, self.max_model_len)
        for g, pool in enumerate(self.pools):
            if self.peak_pages(g, total, chunk) > pool.num_pages:
                return AllocStatus.NEVER
        if not self._free_slots:
            return AllocStatus.LATER
        if any(self.blocks_for(first_tokens, g) > pool.num_free for g, pool in enumerate(self.pools)):
            return AllocStatus.LATER
        return AllocStatus.OK

    def can_reserve(self, request_id: object, new_tokens: int) -> bool:
        return all(n <= pool.num_free for n, pool in zip(self.pages_needed(request_id, new_tokens), self.pools))

    def can_reserve_all(self, wanted: "list[tuple[object, int]]") -> bool:
        """Whether every (request, new tokens) of ``wanted`` can be served together from what is free now."""
        left = [pool.num_free for pool in self.pools]
        for request_id, new_tokens in wanted:
            for g, need in enumerate(self.pages_needed(request_id, new_tokens)):
                left[g] -= need
                if left[g] < 0:
                    return False
        return True

    # ------------------------------------------------------------------ changes
    def admit(self, request_id: object) -> RequestPages:
        if request_id in self._requests:
            raise CacheError(f"request {request_id!r} is already live")
        if not self._free_slots:
            raise CacheError("no free state slot")
        req = RequestPages(request_id, self._free_slots.pop(), tables=[[] for _ in self.groups],
                           first_block=[0] * len(self.groups))
        self._requests[request_id] = req
        return req

    def reserve(self, request_id: object, new_tokens: int) -> None:
        """Hand out the pages that positions [length, length + new_tokens) fall into."""
        req = self.get(request_id)
        target = req.length + new_tokens
        if target > self.max_model_len:
            raise CacheError(f"request {request_id!r} would reach {target} tokens, beyond max_model_len "
                             f"{self.max_model_len}")
        needs = self.pages_needed(request_id, new_tokens)
        for need, pool in zip(needs, self.pools):
            if need > pool.num_free:
                raise OutOfPages(f"request {request_id!r} needs {need} pages, {pool.num_free} are free")
        for g, need in enumerate(needs):
            for _ in range(need):
                req.tables[g].append(self.pools[g].take(request_id))
        req.reserved = max(req.reserved, target)

    def commit(self, request_id: object, new_tokens: int) -> None:
        """The step wrote ``new_tokens`` more tokens; pages a window has passed go back."""
        req = self.get(request_id)
        if req.length + new_tokens > req.reserved:
            raise CacheError(f"request {request_id!r}: commit past the reserved pages")
        req.length += new_tokens
        for g in range(len(self.groups)):
            first = self._first_needed_block(g, req.length)
            table = req.tables[g]
            for b in range(req.first_block[g], min(first, len(table))):
                if table[b] >= 0:
                    self.pools[g].give_back(table[b], request_id)
                    table[b] = -1
            req.first_block[g] = max(req.first_block[g], min(first, len(table)))

    def release(self, request_id: object) -> None:
        """Everything the request holds goes back (finished, aborted or preempted)."""
        req = self._requests.pop(request_id, None)
        if req is None:
            raise CacheError(f"release of request {request_id!r}, which is not live")
        for g, table in enumerate(req.tables):
            for page in reversed(table):
                if page >= 0:
                    self.pools[g].give_back(page, request_id)
        self._free_slots.append(req.slot)

    # ------------------------------------------------------------------ checks
    def utilization(self) -> float:
        """Useful tokens / token slots in held pages (slipstream/memory/block_manager.py:246-258)."""
        held = useful = 0
        for req in self._requests.values():
            for g, table in enumerate(req.tables):
                pages = sum(1 for p in table if p >= 0)
                size = self.page_sizes[g]
                held += pages * size
                useful += min(req.length - req.first_block[g] * size, pages * size)
        return 1.0 if held == 0 else useful / held

    def check_invariants(self) -> None:
        """No page lost, held twice or free while held; slots likewise
        (slipstream/memory/block_manager.py:303-325)."""
        for g, pool in enumerate(self.pools):
            free = pool._free
            if len(set(free)) != len(free):
                raise AssertionError(f"group {g}: a page is on the free list twice")
            held: dict[int, object] = {}
            for rid, req in self._requests.items():
                for page in req.tables[g]:
                    if page < 0:
                        continue
                    if page in held:
                        raise AssertionError(f"group {g}: page {page} is held by {held[page]!r} and {rid!r}")
                    held[page] = rid
            if set(held) & set(free):
                raise AssertionError(f"group {g}: a held page is on the free list")
            if len(held) + len(free) != pool.num_pages:
                raise AssertionError(f"group {g}: {pool.num_pages - len(held) - len(free)} pages lost")
            for page, rid in held.items():
                if pool.holder(page) != rid:
                    raise AssertionError(f"group {g}: page {page} holder mismatch")
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise AssertionError("a state slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_num_seqs:
            raise AssertionError("a state slot was lost")
