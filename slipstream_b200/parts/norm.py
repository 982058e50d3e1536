"""RMSNorm, fused with the residual add that precedes it.

``y = weight * round(x * rsqrt(mean(x^2) + eps))`` with the statistics in
float32 (slipstream/models/layers/rmsnorm.py:28-34).  The residual stream is kept
in float32; the branch output that has not been added yet comes in as ``delta``.
"""

from __future__ import annotations

import torch

from slipstream_b200 import ops

from .base import NORMS, Norm, Runtime, WeightSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    cuda_graph_safe = True

    def __init__(self, name: str, size: int, eps: float) -> None:
        self.name = name
        self.size = size
        self.eps = float(eps)
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(f"{self.name}.weight", (self.size,), kind="vector",
                           init=("one_plus_normal", 0.1))]

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        self.weight = weights[f"{self.name}.weight"]

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def add_norm(self, residual: torch.Tensor, delta: torch.Tensor | None,
                 rows: torch.Tensor | None = None) -> torch.Tensor:
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, self.runtime.dtype, rows=rows)

    def add_norm_of_linear(self, residual: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
                           bias: torch.Tensor | None) -> torch.Tensor:
        return ops.linear_add_rmsnorm(x, weight, bias, residual, self.weight, self.eps, self.runtime.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.add_norm(x, None)
