"""Plain, slow restatement of the Qwen2.5 dense decoder, used as the oracle in tests.

Whole sequences, no cache, one function for each part, and no code shared with
the product package: it reads ``config.json`` and ``model.safetensors`` by
itself and works on plain tensors on the CPU.  Each function cites the reference
lines whose formula it restates.  ``tests/golden/make_golden.py`` compares it
once with the reference's own model code on a tiny random model; the stored
outputs are checked by ``tests/test_plain_reference.py``.

Arithmetic runs in ``dtype`` (float32 by default, float64 for a tighter oracle);
where the reference casts to float32 inside a bfloat16 model, this code is
already at least that wide.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# --------------------------------------------------------------------------- loading

def read_model_folder(folder, dtype=torch.float32):
    """Return (config dict, {tensor name: tensor in ``dtype``}) of a model folder."""
    from safetensors import safe_open

    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    weights = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as handle:
        for key in handle.keys():
            weights[key] = handle.get_tensor(key).to(dtype)
    return config, weights


def sizes(config):
    """The constants of slipstream/models/hf_config.py:60-153 with its defaults."""
    hidden = config["hidden_size"]
    n_q = config["num_attention_heads"]
    return {
        "hidden": hidden,
        "n_q": n_q,
        "n_kv": config.get("num_key_value_heads") or n_q,
        "head_dim": config.get("head_dim") or hidden // n_q,
        "layers": config["num_hidden_layers"],
        "eps": config.get("rms_norm_eps", 1e-6),
        "theta": config.get("rope_theta", 10000.0),
        "tied": bool(config.get("tie_word_embeddings", False)),
    }


# --------------------------------------------------------------------------- parts

def rms_norm(x, weight, eps):
    """slipstream/models/layers/rmsnorm.py:28-34: variance over the last axis,
    ``x * rsqrt(mean(x^2) + eps)``, then the weight."""
    x_hat = x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return weight * x_hat


def inverse_frequencies(head_dim, theta):
    """slipstream/models/layers/rope.py:39-42: ``1 / theta**(i/head_dim)`` for even
    i, formed in float32 as the reference does."""
    dims = torch.arange(0, head_dim, 2, dtype=torch.float32)
    return 1.0 / (theta ** (dims / head_dim))


def rotary_tables(positions, head_dim, theta, dtype):
    """slipstream/models/layers/rope.py:93-106: angles = position * inv_freq in
    float32, duplicated over both halves; cos and sin of them.  The reference takes
    cosine and sine in float32; here each float32 angle goes through ``math.cos`` /
    ``math.sin`` (double precision, one value at a time), which differs from that by
    at most the rounding of the result to float32.  A vectorised float32 cosine
    of a CPU math library may be less exact than that on some inputs (errors of 1e-4 have
    been seen); going through double precision keeps the oracle independent of it."""
    inv_freq = inverse_frequencies(head_dim, theta)
    freqs = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    angles = [[float(a) for a in row] for row in freqs.tolist()]
    cos = torch.tensor([[math.cos(a) for a in row] for row in angles], dtype=torch.float64).reshape(freqs.shape)
    sin = torch.tensor([[math.sin(a) for a in row] for row in angles], dtype=torch.float64).reshape(freqs.shape)
    return torch.cat((cos, cos), dim=-1).to(dtype), torch.cat((sin, sin), dim=-1).to(dtype)


def rotate_half(x):
    """slipstream/models/layers/rope.py:13-17."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rotary(x, cos, sin):
    """slipstream/models/layers/rope.py:20-36 for one of q or k; ``x`` is
    [tokens, heads, head_dim], cos/sin are [tokens, head_dim]."""
    return x * cos[:, None, :] + rotate_half(x) * sin[:, None, :]


def causal_attention(q, k, v, scale):
    """slipstream/models/layers/attention.py:20-29 (each group of query heads
    shares a key/value head), :46-51 (key j visible to query i iff j <= i),
    :64-88 (scores * scale, softmax, weighted sum).  q is [T, n_q, D]; k and v
    are [T, n_kv, D]; returns [T, n_q * D]."""
    tokens, n_q, head_dim = q.shape
    group = n_q // k.shape[1]
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    allowed = torch.arange(tokens)[None, :] <= torch.arange(tokens)[:, None]
    scores = scores.masked_fill(~allowed[None, :, :], float("-inf"))
    weights = torch.softmax(scores, dim=-1)
    out = torch.einsum("hij,jhd->ihd", weights, v)
    return out.reshape(tokens, n_q * head_dim)


def attention_block(x, positions, weights, prefix, s):
    """slipstream/models/layers/attention.py:130-135,148-190: biased q/k/v
    projections, rotary on q and k, attention, unbiased output projection."""
    def proj(name):
        out = x @ weights[f"{prefix}.{name}.weight"].T
        bias = weights.get(f"{prefix}.{name}.bias")
        return out if bias is None else out + bias

    tokens = x.shape[0]
    q = proj("q_proj").view(tokens, s["n_q"], s["head_dim"])
    k = proj("k_proj").view(tokens, s["n_kv"], s["head_dim"])
    v = proj("v_proj").view(tokens, s["n_kv"], s["head_dim"])
    cos, sin = rotary_tables(positions, s["head_dim"], s["theta"], x.dtype)
    q = apply_rotary(q, cos, sin)
    k = apply_rotary(k, cos, sin)
    attn = causal_attention(q, k, v, s["head_dim"] ** -0.5)
    return proj_out(attn, weights, prefix)


def proj_out(attn, weights, prefix):
    out = attn @ weights[f"{prefix}.o_proj.weight"].T
    bias = weights.get(f"{prefix}.o_proj.bias")
    return out if bias is None else out + bias


def swiglu_mlp(x, weights, prefix):
    """slipstream/models/layers/mlp.py:33-40: ``down(silu(gate(x)) * up(x))``."""
    def proj(name, inp):
        out = inp @ weights[f"{prefix}.{name}.weight"].T
        bias = weights.get(f"{prefix}.{name}.bias")
        return out if bias is None else out + bias

    gate = proj("gate_proj", x)
    return proj("down_proj", gate * torch.sigmoid(gate) * proj("up_proj", x))


def decoder_layer(x, positions, weights, index, s):
    """slipstream/models/causal_lm.py:47-48,58-61: ``x + attn(norm(x))`` then
    ``x + mlp(norm(x))``."""
    prefix = f"model.layers.{index}"
    x = x + attention_block(
        rms_norm(x, weights[f"{prefix}.input_layernorm.weight"], s["eps"]),
        positions, weights, f"{prefix}.self_attn", s)
    x = x + swiglu_mlp(
        rms_norm(x, weights[f"{prefix}.post_attention_layernorm.weight"], s["eps"]),
        weights, f"{prefix}.mlp")
    return x


def forward_logits(config, weights, token_ids, return_hidden=False, rows=None):
    """slipstream/models/causal_lm.py:93-97,140: embedding lookup, the layers,
    final norm, LM head (the embedding matrix when tied and no head is stored,
    slipstream/models/loader.py:91-93).  Returns logits [T, vocab] for the whole
    sequence of ``token_ids`` at positions 0..T-1; with ``rows`` only for those positions (the layers still run
    over the whole sequence)."""
    s = sizes(config)
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(ids.numel())
    x = weights["model.embed_tokens.weight"][ids]
    for index in range(s["layers"]):
        x = decoder_layer(x, positions, weights, index, s)
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long)]
    x = rms_norm(x, weights["model.norm.weight"], s["eps"])
    head = weights.get("lm_head.weight")
    if head is None:
        if not s["tied"]:
            raise KeyError("lm_head.weight is absent and tie_word_embeddings is false")
        head = weights["model.embed_tokens.weight"]
    logits = x @ head.T
    return (logits, x) if return_hidden else logits


# --------------------------------------------------------------------------- sampling

def filtered_logits(logits, *, temperature, top_k=-1, top_p=1.0, min_p=0.0,
                    repetition_penalty=1.0, history=()):
    """slipstream/engine/sampler.py:87-104 with :107-146, for one row of logits:
    repetition penalty, temperature, top-k, top-p, min-p, in that order; removed
    tokens become -inf.  Float64 throughout so it can judge a float32 kernel."""
    out = logits.to(torch.float64).clone()
    if repetition_penalty != 1.0 and len(history):
        idx = torch.as_tensor(sorted(set(int(t) for t in history)), dtype=torch.long)
        picked = out[idx]
        out[idx] = torch.where(picked < 0, picked * repetition_penalty,
                               picked / repetition_penalty)
    out = out / temperature
    if top_k > 0 and top_k < out.numel():
        kth = torch.topk(out, top_k).values[-1]
        out = out.masked_fill(out < kth, float("-inf"))
    if top_p < 1.0:
        probs = torch.softmax(out, dim=-1)
        sorted_probs, sorted_idx = torch.sort(probs, descending=True)
        before = torch.cumsum(sorted_probs, dim=-1) - sorted_probs
        remove = torch.zeros_like(probs, dtype=torch.bool)
        remove[sorted_idx] = before >= top_p
        out = out.masked_fill(remove, float("-inf"))
    if min_p > 0.0:
        probs = torch.softmax(out, dim=-1)
        out = out.masked_fill(probs < min_p * probs.max(), float("-inf"))
    return out


def greedy_token(logits):
    """slipstream/engine/sampler.py:55-56; the lowest index wins a tie."""
    return int(torch.argmax(logits.to(torch.float64)).item())


def generate_greedy(config, weights, prompt, max_tokens):
    """Greedy continuation by re-running the whole sequence each step."""
    tokens = list(prompt)
    out = []
    for _ in range(max_tokens):
        logits = forward_logits(config, weights, tokens)
        nxt = greedy_token(logits[-1])
        out.append(nxt)
        tokens.append(nxt)
    return out


def kv_bytes_per_token(config, dtype_bytes):
    """slipstream/core/config.py:10-22."""
    s = sizes(config)
    return 2 * s["layers"] * s["n_kv"] * s["head_dim"] * dtype_bytes


__all__ = [name for name in dir() if not name.startswith("_") and name not in ("json", "math", "Path", "torch")]
