"""Grouped-query attention over the paged key/value cache.

Biased q/k/v projections (stacked into one product at load), rotary encoding of
queries and keys, the write of keys and values to their pages, causal attention
of the step's rows over each request's pages, and the output projection
(slipstream/models/layers/attention.py:98-191).  ``window`` None attends over all
earlier keys; an integer W over the last W.  ``page_size`` asks for cache pages of
that many tokens for this layer (layers that ask alike share a pool).  Every size is
a constructor parameter; the part does not know which model it is in.
"""

from __future__ import annotations

import torch

from slipstream_b200 import ops

from .base import MIXERS, CacheSpec, IntoNorm, LayerBinding, Mixer, PositionEncoding, Runtime, WeightSpec


@MIXERS.register("paged_attention")
class PagedAttention(Mixer):
    cuda_graph_safe = True
    takes_into = True
    takes_pending_norm = True

    def __init__(self, name: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position_encoding: PositionEncoding, qkv_bias: bool = True, out_bias: bool = False,
                 window: int | None = None, scale: float | None = None, page_size: int | None = None) -> None:
        if num_heads % num_kv_heads != 0:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({num_kv_heads})")
        if head_dim % 16 != 0 or not 16 <= head_dim <= 256:
            raise ValueError(f"the attention kernels take head sizes that are multiples of 16 up to 256, not {head_dim}")
        if window is not None and window < 1:
            raise ValueError("window must be >= 1")
        self.name = name
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.position_encoding = position_encoding
        self.qkv_bias = qkv_bias
        self.out_bias = out_bias
        self.window = window
        self.page_size = page_size  # tokens per cache page this layer wants; None: the engine's default
        self.scale = head_dim ** -0.5 if scale is None else float(scale)

    def weight_specs(self) -> list[WeightSpec]:
        h, d, n = self.hidden_size, self.head_dim, self.name
        specs = [WeightSpec(f"{n}.q_proj.weight", (self.num_heads * d, h)),
                 WeightSpec(f"{n}.k_proj.weight", (self.num_kv_heads * d, h)),
                 WeightSpec(f"{n}.v_proj.weight", (self.num_kv_heads * d, h)),
                 WeightSpec(f"{n}.o_proj.weight", (h, self.num_heads * d))]
        if self.qkv_bias:
            specs += [WeightSpec(f"{n}.q_proj.bias", (self.num_heads * d,), kind="vector"),
                      WeightSpec(f"{n}.k_proj.bias", (self.num_kv_heads * d,), kind="vector"),
                      WeightSpec(f"{n}.v_proj.bias", (self.num_kv_heads * d,), kind="vector")]
        if self.out_bias:
            specs.append(WeightSpec(f"{n}.o_proj.bias", (h,), kind="vector"))
        return specs

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(self.num_kv_heads, self.head_dim, self.window, self.page_size)

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        n = self.name
        self.qkv_weight = torch.cat([weights[f"{n}.{p}_proj.weight"] for p in "qkv"], dim=0).contiguous()
        self.qkv_b = None
        if self.qkv_bias:
            self.qkv_b = torch.cat([weights[f"{n}.{p}_proj.bias"] for p in "qkv"]).to(runtime.dtype).contiguous()
        self.o_weight = weights[f"{n}.o_proj.weight"]
        self.o_b = weights[f"{n}.o_proj.bias"].to(runtime.dtype) if self.out_bias else None
        self.position_encoding.bind(weights, runtime)
        ops.attention_library(self.head_dim)  # compile now, not inside the first step

    # ------------------------------------------------------------------ decode steps replayed from a graph
    def capture_variant(self, longest: int, plan: object = None) -> object:
        """Decode steps: long contexts of few requests want the keys cut into more slices than fit one thread-block
        cluster (``ops.decode_slices``).  Steps with prompt portions: into how many parts the tcgen05 prefill kernel
        cuts the keys of a query tile (``ops.prefill_key_parts``).  Each form is captured as a graph of its own."""
        bf16 = self.runtime.dtype == torch.bfloat16
        if plan is None or plan.is_decode_only:
            return bool(bf16 and ops.is_long_context(longest))
        group = self.num_heads // self.num_kv_heads
        if not bf16 or not ops.tcgen05_attention_fits(self.head_dim, self.num_heads, self.num_kv_heads, self.page_size or 16,
                                          self.window or 0):
            return None
        return int(ops.prefill_key_parts(plan.q_lens, plan.seq_lens, 128 // group, self.num_kv_heads,
                                         ops.sm_count(self.runtime.device)))

    def capture_group(self) -> object:
        return "paged_attention"

    def prepare_capture(self, ctx, variant: object, max_model_len: int) -> None:
        if not ctx.is_decode_only:
            # a captured step with prompt portions: the number of key parts is the variant's (the choice follows the
            # lengths of the step, which a replay does not know on the host)
            ctx.extras[("prefill_key_parts", 128 // (self.num_heads // self.num_kv_heads), self.num_kv_heads)] = int(variant or 1)
            return
        # the number of slices must not follow the lengths of the step that happens to be captured
        ctx.extras["static_max_seq_len"] = max_model_len
        ctx.extras["decode_wide"] = bool(variant)
        # the float32 kernel's list of query tiles: one tile per row of the batch
        rows = ctx.num_requests
        ctx.set_query_tiles(16, 1, torch.arange(rows, dtype=torch.int32, device=ctx.device),
                            torch.zeros(rows, dtype=torch.int32, device=ctx.device))

    def weight_bytes(self) -> int:
        return (self.qkv_weight.numel() + self.o_weight.numel()) * self.o_weight.element_size()

    def after_projection(self, qkv: torch.Tensor, ctx) -> None:
        """Hook for subclasses: change the stacked projection output [N, (n_q + 2 n_kv) * D] in place before
        queries and keys are rotated and keys and values go to their pages (a norm over each query and key head,
        say).  A subclass that overrides it keeps every attention kernel; only the fusion of rotation and page
        write into the decode kernel is off for it, since that kernel takes the projection output as it is."""
        return None

    def forward(self, x: torch.Tensor, ctx, layer: LayerBinding, into: IntoNorm | None = None) -> torch.Tensor:
        meta = ctx.groups[layer.group]
        qkv = ops.linear(x, self.qkv_weight, self.qkv_b)
        plain_projection = type(self).after_projection is PagedAttention.after_projection
        if not plain_projection:
            self.after_projection(qkv, ctx)
        inv_freq, rotary_dim = self.position_encoding.rotary_table()
        # a decode step's attention kernel rotates and writes the newest key and value itself
        fused = (plain_projection and layer.writes_cache
                 and ops.fuses_rope(qkv, ctx, self.head_dim, self.num_heads, self.num_kv_heads, layer.kv.shape[3]))
        if not fused:
            ops.rope_and_cache(qkv, ctx.positions, meta.slot_mapping, inv_freq, layer.kv, self.num_heads,
                               self.num_kv_heads, self.head_dim, rotary_dim, write_cache=layer.writes_cache)
        out = torch.empty((x.shape[0], self.num_heads * self.head_dim), dtype=x.dtype, device=x.device)
        ops.paged_attention(qkv, out, layer.kv, meta.block_tables, ctx, self.num_heads, self.num_kv_heads,
                            self.head_dim, self.scale, self.window or 0,
                            rope=(inv_freq, rotary_dim) if fused else None)
        if into is not None:
            return into.close(out, self.o_weight, self.o_b)
        return ops.linear(out, self.o_weight, self.o_b)
