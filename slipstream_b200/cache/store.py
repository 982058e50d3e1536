"""Device memory behind the cache manager: one page tensor per cache group and one
tensor per fixed-size state a part declared.

Page tensor of a group: ``[entries, pages, 2, kv_heads, page_size, head_dim]`` in
the compute dtype: an entry is one place in the execution order that writes
pages; keys are index 0 and values index 1 of the third axis; one (page, head)
tile of ``page_size x head_dim`` is contiguous so that a kernel can fetch it with
one bulk copy.  The reference keeps ``[layers, 2, blocks, block_size, kv_heads,
head_dim]`` (slipstream/core/types.py:25-29).
"""

from __future__ import annotations

import torch

from slipstream_b200.parts.base import StateSpec

from .manager import GroupLayout


class PagedStore:
    def __init__(self, layouts: list[GroupLayout], dtype: torch.dtype, device: torch.device,
                 state_specs: list[list[StateSpec]], max_num_seqs: int) -> None:
        """``layouts`` carry each group's page size and number of pages (the cache manager fills them in)."""
        self.dtype = dtype
        self.kv: list[torch.Tensor] = []
        for layout in layouts:
            spec = layout.spec
            if layout.page_size < 1 or layout.num_pages < 1:
                raise ValueError("a cache group has no page size or number of pages yet")
            self.kv.append(torch.zeros(
                (max(layout.num_entries, 1), layout.num_pages, 2, spec.num_kv_heads, layout.page_size, spec.head_dim),
                dtype=dtype, device=device))
        self.state: list[dict[str, torch.Tensor]] = []
        for specs in state_specs:
            self.state.append({s.name: torch.zeros((max_num_seqs, *s.shape), dtype=s.dtype, device=device)
                               for s in specs})

    def kv_bytes_per_token(self) -> int:
        """Bytes one cached token takes over all groups and entries
        (slipstream/core/config.py:10-22 for a single group)."""
        total = 0
        for t in self.kv:
            entries, _, _, heads, _, dim = t.shape
            total += entries * 2 * heads * dim * t.element_size()
        return total

    @staticmethod
    def bytes_per_token(layout: GroupLayout, dtype: torch.dtype) -> int:
        """Bytes of one cached token in one group, over the group's entries."""
        size = torch.empty((), dtype=dtype).element_size()
        return max(layout.num_entries, 1) * 2 * layout.spec.num_kv_heads * layout.spec.head_dim * size

    def zero_state(self, slot: int) -> None:
        for entry in self.state:
            for tensor in entry.values():
                tensor[slot].zero_()
