"""Builder of the Qwen2.5 dense decoder from ``Qwen2Config``: which parts stand in
which layer, with which constants and tensor names.

Structure and names follow slipstream/models/causal_lm.py:31-141: per layer
``input_layernorm``, ``self_attn`` (biased q/k/v, unbiased o_proj:
slipstream/models/layers/attention.py:91-95), ``post_attention_layernorm``,
``mlp``; then ``model.norm`` and ``lm_head`` (the embedding matrix when tied).
"""

from __future__ import annotations

from slipstream_b200.config.model_config import Qwen2Config
from slipstream_b200.parts import (LMHead, PagedAttention, PreNormBlock, RMSNorm, RotaryEncoding,
                                   SwiGLUFeedForward, TokenEmbedding)

from .decoder import DecoderLM


def build_qwen2(config: Qwen2Config) -> DecoderLM:
    c = config
    blocks = []
    rotary = RotaryEncoding(c.head_dim, c.rope_theta)  # one table of frequencies for all layers
    for i in range(c.num_hidden_layers):
        prefix = f"model.layers.{i}"
        attention = PagedAttention(
            f"{prefix}.self_attn", c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
            rotary, qkv_bias=c.attention_bias, out_bias=False, window=None)
        ffn = SwiGLUFeedForward(f"{prefix}.mlp", c.hidden_size, c.intermediate_size, bias=c.mlp_bias)
        blocks.append(PreNormBlock(
            attention, ffn,
            RMSNorm(f"{prefix}.input_layernorm", c.hidden_size, c.rms_norm_eps),
            RMSNorm(f"{prefix}.post_attention_layernorm", c.hidden_size, c.rms_norm_eps)))
    return DecoderLM(
        c,
        TokenEmbedding("model.embed_tokens", c.vocab_size, c.hidden_size),
        blocks,
        RMSNorm("model.norm", c.hidden_size, c.rms_norm_eps),
        LMHead("lm_head", c.vocab_size, c.hidden_size,
               tied_to="model.embed_tokens.weight" if c.tie_word_embeddings else None))
