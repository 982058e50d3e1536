"""Pre-norm residual block: ``x + mixer(norm(x))`` then ``x + ffn(norm(x))``
(slipstream/models/causal_lm.py:47-48,58-61), on a float32 residual stream with
each add fused into the norm that follows it."""

from __future__ import annotations

import torch

from .base import BLOCKS, Block, FeedForward, LayerBinding, Mixer, Norm, Part


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
        x = self.mixer_norm.add_norm(residual, pending)
        mixed = self.mixer.forward(x, ctx, layer)
        x = self.ffn_norm.add_norm(residual, mixed)
        return residual, self.feed_forward.forward(x, ctx)
