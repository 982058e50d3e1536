"""Interfaces of the parts a model is put together from, and their registries.

A part knows its own sizes and constants (constructor parameters), the
checkpoint tensors it owns (``weight_specs``), what it needs from the cache
manager (``cache_spec`` for pages of keys and values, ``state_specs`` for
fixed-size per-request state), and how to run on a token-major batch.  No part
knows which model it is in: a model builder picks parts layer by layer from the
configuration and hands them their tensor-name prefixes.

Token-major means activations are ``[num_tokens, width]`` for all tokens of the
step, whatever request they belong to; ``StepContext`` says which rows belong to
which request.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import TYPE_CHECKING, Any, Callable

import torch

if TYPE_CHECKING:
    from slipstream_b200.engine.context import StepContext


# --------------------------------------------------------------------------- specs

@dataclass(frozen=True)
class WeightSpec:
    """One checkpoint tensor a part reads.

    ``kind`` decides the dtype it is kept in: ``matrix`` tensors go to the compute
    dtype (bfloat16 or float32); ``vector`` tensors do too unless the checkpoint
    stores them in 32-bit, which is kept; ``index`` tensors become int32.
    ``init`` is used by the random-weights mode: ("normal", std) or
    ("one_plus_normal", std).  ``alias_of`` names the tensor that stands in when
    this one is absent (tied embeddings).
    """

    name: str
    shape: tuple[int, ...]
    kind: str = "matrix"
    init: tuple[str, float] = ("normal", 0.02)
    alias_of: str | None = None


@dataclass(frozen=True)
class CacheSpec:
    """Pages of keys and values one mixer needs per token.  ``window`` None means
    every earlier key stays visible; an integer W means only the last W keys are,
    so pages wholly before the window are given back.  ``page_size``: tokens per page this mixer's kernels
    want; None takes the engine's default.  Mixers whose specs are equal share a cache group (one page pool, one
    block table per request); a group has its own page size and its own number of pages."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None
    page_size: int | None = None


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state a part keeps in the slot pool (one row per
    live request); zeroed when a request is admitted."""

    name: str
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class Runtime:
    """Device and precision the parts are bound to."""

    device: torch.device
    dtype: torch.dtype  # torch.bfloat16 or torch.float32

    @property
    def is_fp32(self) -> bool:
        return self.dtype == torch.float32


# --------------------------------------------------------------------------- parts

class Part:
    """Base of all parts.  ``bind`` receives the loaded tensors by full name.

    ``cuda_graph_safe``: the part's forward launches the same kernels with the same grids for every
    decode step of a given batch size and never synchronises with the host, so a decode step through
    it may be captured in a CUDA graph.  Parts that do not say so run eagerly."""

    cuda_graph_safe = False

    def weight_specs(self) -> list[WeightSpec]:
        return []

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime

    def weight_bytes(self) -> int:
        """Bytes of weights one step reads from this part (for the roofline)."""
        return 0

    # -- decode steps replayed from a CUDA graph.  Inside a replay nothing is known on the host about the step
    # -- but its bucket (the number of rows), so whatever a part's forward derives from the step's lengths has to
    # -- be fixed when the graph is captured.  A part that needs this overrides the two methods below.
    def capture_variant(self, longest: int, plan: object = None) -> object:
        """Which captured form of this part a step whose longest request holds ``longest`` tokens should run
        (any hashable; None: there is only one form).  ``plan`` is the step's host-side metadata
        (``engine.context.HostPlan``: ``q_lens``, ``seq_lens``, ``is_decode_only``) or None.  The runner keeps one
        graph per bucket and combination of variants."""
        return None

    def capture_group(self) -> object:
        """Parts that return the same value here always answer ``capture_variant`` alike (every attention layer
        of a model, say), so the runner asks one of them per step."""
        return id(self)

    def prepare_capture(self, ctx: "StepContext", variant: object, max_model_len: int) -> None:
        """Called once on the static context of a decode graph before it is captured: store in ``ctx.extras``
        (or through ``ctx.set_query_tiles``) what the forward must not take from the host-side lengths of the
        step, for the form ``variant`` (the value ``capture_variant`` returned)."""
        return None


class Norm(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_norm(self, residual: torch.Tensor, delta: torch.Tensor | None,
                 rows: torch.Tensor | None = None) -> torch.Tensor:
        """``residual += delta`` (float32, in place) and return ``norm(residual)``
        in the compute dtype.  With ``rows`` only those rows are normalised and
        returned, and ``residual`` is left untouched."""
        raise NotImplementedError

    def add_norm_of_linear(self, residual: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
                           bias: torch.Tensor | None):
        """``add_norm(residual, x @ weight.T + bias)``: a branch's last projection with the add and the norm
        that follow it.  A norm that can be split between the projection in front and the product behind it
        overrides this and may return an ``ops.PendingNorm`` instead of a tensor; the block hands that only to a
        part whose ``takes_pending_norm`` is True (its first product accepts it) and otherwise calls its
        ``materialize()``."""
        from slipstream_b200 import ops
        return self.add_norm(residual, ops.linear(x, weight, bias))


@dataclass
class IntoNorm:
    """Handed to a mixer or feed-forward whose ``takes_into`` is True: instead of returning its output it ends
    with ``into.close(x, weight, bias)``, its last projection, and returns what that returns, the norm of the
    stream with its output added (the add is done: the caller adds nothing), as a tensor or a pending norm."""

    norm: Norm
    residual: torch.Tensor

    def close(self, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None):
        return self.norm.add_norm_of_linear(self.residual, x, weight, bias)


def settle(x, part: Part) -> torch.Tensor:
    """``x`` as ``part`` can take it: a pending norm is computed now unless the part's first product accepts it."""
    if isinstance(x, torch.Tensor) or getattr(part, "takes_pending_norm", False):
        return x
    return x.materialize()


class PositionEncoding(Part):
    """Where positions enter.  ``on_embedding`` may add to the residual stream;
    ``on_query_key`` rotates (or otherwise marks) queries and keys inside a mixer.
    Both default to doing nothing."""

    def on_embedding(self, residual: torch.Tensor, ctx: "StepContext") -> None:
        return None

    def rotary_table(self) -> tuple[torch.Tensor | None, int]:
        """(inverse frequencies float32 [rotary_dim/2] on the device, rotary_dim),
        or (None, 0) when queries and keys are not rotated."""
        return None, 0


class Mixer(Part):
    """Mixes information across the tokens of a request (attention here).  A mixer that ends in a projection may
    set ``takes_into`` and accept ``forward(x, ctx, layer, into=None)`` (see `IntoNorm`); one that hands ``x``
    to ``ops.linear`` first and otherwise only asks its shape, dtype and device may set ``takes_pending_norm``."""

    takes_into = False
    takes_pending_norm = False

    def cache_spec(self) -> CacheSpec | None:
        return None

    def state_specs(self) -> list[StateSpec]:
        return []

    def forward(self, x: torch.Tensor, ctx: "StepContext", layer: "LayerBinding") -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    """A feed-forward that ends in a projection may set ``takes_into`` and accept ``forward(x, ctx, into=None)``
    (see `IntoNorm`); one that hands ``x`` to ``ops.linear`` or ``ops.gate_up_swiglu`` first may set
    ``takes_pending_norm``."""

    takes_into = False
    takes_pending_norm = False

    def forward(self, x: torch.Tensor, ctx: "StepContext") -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    """Token ids (int32 [N] on the device) into the float32 residual stream [N, hidden]."""

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    """Normalised rows of the stream (compute dtype [M, hidden]) into float32 logits [M, vocab_size].  A head
    that hands ``x`` to ``ops.linear`` first may set ``takes_pending_norm`` (see `IntoNorm`): when every row's
    logits are wanted, the last block then ends in the final norm."""

    vocab_size: int
    takes_pending_norm = False

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arrangement of a mixer, a feed-forward and their norms around the float32
    residual stream.  ``forward`` takes the stream and a branch output that has
    not been added yet, and returns the same pair, so that the add fuses with the
    next norm wherever it stands."""

    mixer: Mixer

    def forward(self, residual: torch.Tensor, pending: torch.Tensor | None,
                ctx: "StepContext", layer: "LayerBinding") -> tuple[torch.Tensor, torch.Tensor | None]:
        raise NotImplementedError

    def first_norm(self) -> Norm | None:
        """The norm this block applies first to (stream + pending), if it can take that norm's result instead
        (``forward_chained``'s ``normed``); None: the block wants the stream and the pending output."""
        return None

    def forward_chained(self, residual: torch.Tensor, pending: torch.Tensor | None, normed: torch.Tensor | None,
                        following: Norm | None, ctx: "StepContext",
                        layer: "LayerBinding") -> tuple[torch.Tensor, torch.Tensor | None, torch.Tensor | None]:
        """``forward`` for a model that lets a block's last projection end in the next block's first norm.
        ``normed``: ``first_norm()`` of the stream, already computed by the block before, as a tensor or a pending
        norm (then ``pending`` is None and added).  ``following``: the next block's first norm, or None.  Returns
        (stream, pending, normed): either a pending output, or, if it applied ``following``, that norm's result.
        The default chains nothing."""
        assert normed is None
        residual, pending = self.forward(residual, pending, ctx, layer)
        return residual, pending, None


@dataclass
class LayerBinding:
    """What one entry of the execution order hands to the mixer: which pages and
    which state rows are its own.  ``kv`` is this entry's page tensor
    ``[num_pages, 2, num_kv_heads, page_size, head_dim]`` (or None), ``group`` the
    index of the cache group whose block tables address it, ``writes_cache``
    False when the entry only reads pages that another entry wrote."""

    kv: torch.Tensor | None = None
    group: int = -1
    writes_cache: bool = True
    state: dict[str, torch.Tensor] = field(default_factory=dict)


# --------------------------------------------------------------------------- registries

class Registry:
    """Name -> class (or builder) table with a decorator to add entries."""

    def __init__(self, what: str) -> None:
        self.what = what
        self._entries: dict[str, Any] = {}

    def register(self, name: str) -> Callable[[Any], Any]:
        def add(obj: Any) -> Any:
            if name in self._entries and self._entries[name] is not obj:
                raise KeyError(f"{self.what} {name!r} is already registered")
            self._entries[name] = obj
            return obj
        return add

    def unregister(self, name: str) -> None:
        self._entries.pop(name, None)

    def get(self, name: str) -> Any:
        try:
            return self._entries[name]
        except KeyError:
            known = ", ".join(sorted(self._entries)) or "none"
            raise KeyError(f"unknown {self.what} {name!r} (registered: {known})") from None

    def names(self) -> list[str]:
        return sorted(self._entries)

    def __contains__(self, name: str) -> bool:
        return name in self._entries


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block arrangement")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")
