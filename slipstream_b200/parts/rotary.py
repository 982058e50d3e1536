"""Rotary position encoding (half-split pairing: element d pairs with d + D/2).

Inverse frequencies ``1 / theta**(2i/D)`` are formed in float32 on the host
exactly as the reference does (slipstream/models/layers/rope.py:39-42); angles,
cosines and sines are float32 inside the kernel (:93-106), which also writes the
rotated keys and the values to their cache pages.
"""

from __future__ import annotations

import torch

from .base import POSITION_ENCODINGS, PositionEncoding, Runtime


@POSITION_ENCODINGS.register("rotary")
class RotaryEncoding(PositionEncoding):
    cuda_graph_safe = True

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None) -> None:
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim must be even and in (0, {head_dim}], got {self.rotary_dim}")
        self.inv_freq: torch.Tensor | None = None

    def inverse_frequencies(self) -> torch.Tensor:
        dims = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
        return 1.0 / (self.theta ** (dims / self.rotary_dim))

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        self.inv_freq = self.inverse_frequencies().to(runtime.device)

    def rotary_table(self) -> tuple[torch.Tensor | None, int]:
        return self.inv_freq, self.rotary_dim


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    """Queries and keys are used as projected."""

    cuda_graph_safe = True
