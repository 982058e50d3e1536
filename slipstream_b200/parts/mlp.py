"""Dense SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))``
(slipstream/models/layers/mlp.py:33-40).  The gate and up matrices are stacked at
load so that one product feeds the activation kernel."""

from __future__ import annotations

import torch

from slipstream_b200 import ops

from .base import FEED_FORWARDS, FeedForward, IntoNorm, Runtime, WeightSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLUFeedForward(FeedForward):
    cuda_graph_safe = True
    takes_into = True
    takes_pending_norm = True

    def __init__(self, name: str, hidden_size: int, intermediate_size: int, bias: bool = False) -> None:
        self.name = name
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.bias = bias

    def weight_specs(self) -> list[WeightSpec]:
        h, i = self.hidden_size, self.intermediate_size
        specs = [WeightSpec(f"{self.name}.gate_proj.weight", (i, h)),
                 WeightSpec(f"{self.name}.up_proj.weight", (i, h)),
                 WeightSpec(f"{self.name}.down_proj.weight", (h, i))]
        if self.bias:
            specs += [WeightSpec(f"{self.name}.gate_proj.bias", (i,), kind="vector"),
                      WeightSpec(f"{self.name}.up_proj.bias", (i,), kind="vector"),
                      WeightSpec(f"{self.name}.down_proj.bias", (h,), kind="vector")]
        return specs

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        n = self.name
        # gate and up rows alternate in runs of `block`, so that one 128-row tile of the stacked product holds
        # 64 gate features and the 64 matching up features (the fused epilogue needs both in one block)
        i = self.intermediate_size
        self.block = 64 if i % 64 == 0 else i

        def interleave(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
            g = gate.reshape(i // self.block, self.block, *gate.shape[1:])
            u = up.reshape(i // self.block, self.block, *up.shape[1:])
            return torch.stack([g, u], dim=1).reshape(2 * i, *gate.shape[1:]).contiguous()

        self.gate_up = interleave(weights[f"{n}.gate_proj.weight"], weights[f"{n}.up_proj.weight"])
        self.down = weights[f"{n}.down_proj.weight"]
        self.gate_up_bias = self.down_bias = None
        if self.bias:
            self.gate_up_bias = interleave(weights[f"{n}.gate_proj.bias"], weights[f"{n}.up_proj.bias"]).to(runtime.dtype)
            self.down_bias = weights[f"{n}.down_proj.bias"].to(runtime.dtype)

    def weight_bytes(self) -> int:
        return (self.gate_up.numel() + self.down.numel()) * self.down.element_size()

    def forward(self, x: torch.Tensor, ctx, into: IntoNorm | None = None) -> torch.Tensor:
        hidden = ops.gate_up_swiglu(x, self.gate_up, self.gate_up_bias, self.block)
        if into is not None:
            return into.close(hidden, self.down, self.down_bias)
        return ops.linear(hidden, self.down, self.down_bias)
