"""Pre-norm residual block: ``x + mixer(norm(x))`` then ``x + ffn(norm(x))``
(slipstream/models/causal_lm.py:47-48,58-61), on a float32 residual stream with
each add fused into the norm that follows it, and that norm handed to the branch
before it (`IntoNorm`), whose last projection may do both in its own launch."""

from __future__ import annotations

import torch

from .base import BLOCKS, Block, FeedForward, IntoNorm, LayerBinding, Mixer, Norm, Part, settle


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    cuda_graph_safe = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, ffn_norm: Norm) -> None:
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.ffn_norm = ffn_norm

    def children(self) -> list[Part]:
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward]

    def forward(self, residual: torch.Tensor, pending: torch.Tensor | None, ctx,
                layer: LayerBinding) -> tuple[torch.Tensor, torch.Tensor | None]:
        residual, pending, _ = self.forward_chained(residual, pending, None, None, ctx, layer)
        return residual, pending

    def first_norm(self) -> Norm:
        return self.mixer_norm

    def forward_chained(self, residual: torch.Tensor, pending: torch.Tensor | None, normed: torch.Tensor | None,
                        following: Norm | None, ctx, layer: LayerBinding):
        x = settle(normed, self.mixer) if normed is not None else self.mixer_norm.add_norm(residual, pending)
        if self.mixer.takes_into:
            x = settle(self.mixer.forward(x, ctx, layer, into=IntoNorm(self.ffn_norm, residual)), self.feed_forward)
        else:
            x = self.ffn_norm.add_norm(residual, self.mixer.forward(x, ctx, layer))
        if following is not None and self.feed_forward.takes_into:
            return residual, None, self.feed_forward.forward(x, ctx, into=IntoNorm(following, residual))
        return residual, self.feed_forward.forward(x, ctx), None
