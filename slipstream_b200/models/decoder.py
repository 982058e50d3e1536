"""A decoder-only language model as data: parts, and the order in which layers run.

``DecoderLM`` holds an embedding, a list of blocks, a final norm, an LM head and
``order``: the list of ``ExecEntry`` that says which block runs when.  The order
may name a block twice (each occurrence has pages and state of its own) or let
an occurrence read the pages another occurrence wrote (``cache_of``).  For the
Qwen2.5 decoder the order is simply every block once
(slipstream/models/causal_lm.py:95-96).  The class knows no architecture; model
builders (``slipstream_b200/models/qwen2.py``) fill it from a configuration.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from slipstream_b200.cache import GroupLayout
from slipstream_b200.parts.base import (Block, CacheSpec, Embedding, Head, LayerBinding, Norm, Part,
                                        PositionEncoding, Runtime, StateSpec, WeightSpec, settle)


@dataclass(frozen=True)
class ExecEntry:
    """One place in the execution order.  ``block``: index of the block whose weights run.
    ``cache_of``: index (into the order) of an earlier entry whose pages this one reads
    instead of writing its own."""

    block: int
    cache_of: int | None = None


def _walk(part: Part) -> list[Part]:
    out = [part]
    children = getattr(part, "children", None)
    if callable(children):
        for child in children():
            out.extend(_walk(child))
    return out


class DecoderLM:
    def __init__(self, config, embedding: Embedding, blocks: list[Block], final_norm: Norm,
                 lm_head: Head, order: list[ExecEntry] | None = None,
                 position_encoding: PositionEncoding | None = None) -> None:
        self.config = config
        self.embedding = embedding
        self.blocks = blocks
        self.final_norm = final_norm
        self.lm_head = lm_head
        self.position_encoding = position_encoding
        self.order = order if order is not None else [ExecEntry(i) for i in range(len(blocks))]
        self.bindings: list[LayerBinding] = []
        self._plan_cache()

    # ------------------------------------------------------------------ structure
    def parts(self) -> list[Part]:
        out: list[Part] = [self.embedding]
        for block in self.blocks:
            out.extend(_walk(block))
        out.extend([self.final_norm, self.lm_head])
        if self.position_encoding is not None:
            out.append(self.position_encoding)
        return out

    def weight_specs(self) -> list[WeightSpec]:
        specs: dict[str, WeightSpec] = {}
        for part in self.parts():
            for spec in part.weight_specs():
                if spec.name in specs and specs[spec.name] != spec:
                    raise ValueError(f"two parts claim the tensor {spec.name!r} differently")
                specs[spec.name] = spec
        return list(specs.values())

    def _plan_cache(self) -> None:
        """Group the order's entries by what their mixers need from the cache."""
        self.group_layouts: list[GroupLayout] = []
        self.entry_group: list[int] = []  # per order entry: group index or -1
        self.entry_index: list[int] = []  # per order entry: index within its group's page tensor
        self.entry_state: list[list[StateSpec]] = []
        by_spec: dict[CacheSpec, int] = {}
        for pos, entry in enumerate(self.order):
            if not 0 <= entry.block < len(self.blocks):
                raise ValueError(f"order[{pos}] names block {entry.block}, which does not exist")
            mixer = self.blocks[entry.block].mixer
            spec = mixer.cache_spec()
            self.entry_state.append(list(mixer.state_specs()))
            if spec is None:
                if entry.cache_of is not None:
                    raise ValueError(f"order[{pos}] reads another entry's cache but its mixer has none")
                self.entry_group.append(-1)
                self.entry_index.append(-1)
                continue
            if entry.cache_of is not None:
                src = entry.cache_of
                if not 0 <= src < pos or self.order[src].cache_of is not None:
                    raise ValueError(f"order[{pos}].cache_of must name an earlier entry that writes its own pages")
                if self.blocks[self.order[src].block].mixer.cache_spec() != spec:
                    raise ValueError(f"order[{pos}] and order[{src}] need different pages and cannot share them")
                self.entry_group.append(self.entry_group[src])
                self.entry_index.append(self.entry_index[src])
                continue
            g = by_spec.setdefault(spec, len(self.group_layouts))
            if g == len(self.group_layouts):
                self.group_layouts.append(GroupLayout(spec))
            self.entry_group.append(g)
            self.entry_index.append(self.group_layouts[g].num_entries)
            self.group_layouts[g].num_entries += 1

    # ------------------------------------------------------------------ binding
    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        for part in self.parts():
            part.bind(weights, runtime)

    def attach_store(self, store) -> None:
        """Give every entry of the order its pages and its rows of the state pool."""
        self.bindings = []
        for pos, entry in enumerate(self.order):
            g = self.entry_group[pos]
            kv = store.kv[g][self.entry_index[pos]] if g >= 0 else None
            self.bindings.append(LayerBinding(kv=kv, group=g, writes_cache=entry.cache_of is None,
                                              state=store.state[pos]))

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one step reads: every entry of the order reads its block's weights,
        plus the LM head (the embedding gather is negligible)."""
        per_block = [sum(p.weight_bytes() for p in _walk(b)) for b in self.blocks]
        return sum(per_block[e.block] for e in self.order) + self.final_norm.weight_bytes() + self.lm_head.weight_bytes()

    # ------------------------------------------------------------------ forward
    def forward(self, ctx) -> torch.Tensor:
        """Run the step's tokens through the order; float32 logits [wanted rows, vocab]."""
        residual = self.embedding.forward(ctx.token_ids)
        if self.position_encoding is not None:
            self.position_encoding.on_embedding(residual, ctx)
        pending = normed = None
        # the last block may end in the final norm when that norm needs no selection of rows
        closing = self.final_norm if ctx.extras.get("every_row_wanted") and ctx.num_logits else None
        for pos, (entry, binding) in enumerate(zip(self.order, self.bindings)):
            # a block's last projection may end in the first norm of the block that runs next
            following = self.blocks[self.order[pos + 1].block].first_norm() if pos + 1 < len(self.order) else closing
            residual, pending, normed = self.blocks[entry.block].forward_chained(residual, pending, normed, following,
                                                                                 ctx, binding)
        if ctx.num_logits == 0:
            return torch.empty((0, self.lm_head.vocab_size), dtype=torch.float32, device=residual.device)
        if normed is not None:
            return self.lm_head.forward(settle(normed, self.lm_head))
        x = self.final_norm.add_norm(residual, pending, rows=ctx.logit_rows)
        return self.lm_head.forward(x)
