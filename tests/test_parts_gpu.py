"""Each part of the model alone, built with sizes of its own and random tensors, against the plain
functions of tests/plain_qwen2.py."""
import pytest
import torch

import plain_qwen2 as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


def runtime(dtype):
    from slipstream_b200.parts import Runtime
    return Runtime(DEV, dtype)


def rel(got, ref):
    return ((got.double().cpu() - ref.double()).abs().max() / ref.double().abs().max()).item()


def draw(part, dtype, seed=0, scale=1.0):
    """Random tensors for a part's weight specs: (device tensors in the compute dtype, float64 copies of them)."""
    g = torch.Generator().manual_seed(seed)
    dev, ref = {}, {}
    for spec in part.weight_specs():
        t = torch.randn(spec.shape, generator=g) * (0.3 * scale if len(spec.shape) == 2 else 0.2)
        if spec.init[0] == "one_plus_normal":
            t = t + 1
        dev[spec.name] = t.to(dtype).to(DEV)
        ref[spec.name] = dev[spec.name].double().cpu()
    return dev, ref


def single_request_ctx(cache, request_id, tokens_or_n, vocab=10 ** 6):
    from slipstream_b200.engine.context import StepEntry, build_context
    n = tokens_or_n if isinstance(tokens_or_n, int) else len(tokens_or_n)
    tokens = list(range(n)) if isinstance(tokens_or_n, int) else tokens_or_n
    if request_id not in cache:
        cache.admit(request_id)
    ctx = build_context([StepEntry(request_id, tokens, [])], cache, vocab, DEV)
    cache.commit(request_id, n)
    return ctx


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from slipstream_b200.parts import RMSNorm
    part = RMSNorm("n", 200, 1e-4)
    dev, ref = draw(part, dtype)
    part.bind(dev, runtime(dtype))
    x = torch.randn(7, 200)
    got = part.forward(x.to(DEV))
    assert got.dtype == dtype and rel(got, plain.rms_norm(x.double(), ref["n.weight"], 1e-4)) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_feed_forward_part(dtype):
    from slipstream_b200.parts import SwiGLUFeedForward
    for bias, inter, tokens in ((False, 200, 11), (True, 200, 11), (True, 192, 5), (False, 320, 100)):
        part = SwiGLUFeedForward("m", 72, inter, bias=bias)
        dev, ref = draw(part, dtype, seed=3)
        part.bind(dev, runtime(dtype))
        assert part.block == (64 if inter % 64 == 0 else inter)
        x = torch.randn(tokens, 72).to(dtype)
        got = part.forward(x.to(DEV), None)
        assert rel(got, plain.swiglu_mlp(x.double(), ref, "m")) < TOL[dtype]
        assert part.weight_bytes() == 3 * 72 * inter * (4 if dtype == torch.float32 else 2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_lm_head_parts(dtype):
    from slipstream_b200.parts import LMHead, TokenEmbedding
    emb, head = TokenEmbedding("e", 301, 40), LMHead("h", 301, 40, tied_to="e.weight")
    dev, ref = draw(emb, dtype)
    dev["h.weight"] = dev["e.weight"]
    emb.bind(dev, runtime(dtype)); head.bind(dev, runtime(dtype))
    ids = torch.tensor([0, 300, 5, 5], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids).cpu(), ref["e.weight"][ids.long().cpu()].float())
    x = torch.randn(3, 40).to(dtype)
    logits = head.forward(x.to(DEV))
    assert logits.dtype == torch.float32 and rel(logits, x.double() @ ref["e.weight"].T) < TOL[dtype] / 2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, d, page, bias", [(6, 2, 32, 8, True), (5, 1, 16, 4, False), (4, 4, 64, 16, True)])
def test_attention_part_in_two_portions_and_decoding(dtype, heads, kv_heads, d, page, bias):
    """The mixer alone: a prompt portion, a second portion, then single tokens, against the plain
    attention over the whole sequence."""
    from slipstream_b200.cache import CacheManager, GroupLayout, PagedStore
    from slipstream_b200.parts import LayerBinding, PagedAttention, RotaryEncoding
    hidden, theta, n = 56, 30000.0, 45
    part = PagedAttention("a", hidden, heads, kv_heads, d, RotaryEncoding(d, theta), qkv_bias=bias)
    dev, ref = draw(part, dtype, seed=d, scale=0.5)  # scores of order one: keys matter, but no hard arg-max
    part.bind(dev, runtime(dtype))
    layouts = [GroupLayout(part.cache_spec(), 1)]
    cache = CacheManager(layouts, 16, page, 2, 256)
    store = PagedStore(layouts, dtype, DEV, [[]], 2)
    binding = LayerBinding(kv=store.kv[0][0], group=0)
    x = torch.randn(n, hidden).to(dtype)
    s = {"n_q": heads, "n_kv": kv_heads, "head_dim": d, "theta": theta}
    want = plain.attention_block(x.double(), torch.arange(n), ref, "a", s)
    outs, i = [], 0
    for take in (20, 13, 1, 1, 2, 1, 7):
        ctx = single_request_ctx(cache, "r", take)
        outs.append(part.forward(x[i:i + take].to(DEV).contiguous(), ctx, binding))
        i += take
    assert i == n and rel(torch.cat(outs), want) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_an_attention_subclass_that_normalises_heads_before_the_rotation(dtype):
    """A mixer that puts something between projection and rotation (here: every query and key head scaled to unit
    root-mean-square) overrides one hook of the attention part and keeps its kernels: prompt portions through the
    tiled kernels, single tokens through the split decode kernel (head size 64 and pages of 16 would otherwise
    take the kernel that rotates by itself)."""
    from slipstream_b200.cache import CacheManager, GroupLayout, PagedStore
    from slipstream_b200.parts import LayerBinding, PagedAttention, RotaryEncoding
    hidden, heads, kv_heads, d, theta, n, eps = 56, 4, 2, 64, 30000.0, 45, 1e-6

    class HeadNormAttention(PagedAttention):
        def after_projection(self, qkv, ctx):
            qk = qkv[:, : (heads + kv_heads) * d].view(qkv.shape[0], heads + kv_heads, d)
            qk.copy_((qk.float() * torch.rsqrt(qk.float().pow(2).mean(-1, keepdim=True) + eps)).to(qkv.dtype))

    part = HeadNormAttention("a", hidden, heads, kv_heads, d, RotaryEncoding(d, theta), qkv_bias=True)
    dev, ref = draw(part, dtype, seed=3, scale=0.5)
    part.bind(dev, runtime(dtype))
    layouts = [GroupLayout(part.cache_spec(), 1)]
    cache = CacheManager(layouts, 16, 16, 2, 256)
    store = PagedStore(layouts, dtype, DEV, [[]], 2)
    binding = LayerBinding(kv=store.kv[0][0], group=0)
    x = torch.randn(n, hidden).to(dtype)
    # the plain restatement: plain.attention_block with the norm between projection and rotation
    xd = x.double()
    proj = {p: xd @ ref[f"a.{p}_proj.weight"].T + ref[f"a.{p}_proj.bias"] for p in "qkv"}
    q, k, v = proj["q"].view(n, heads, d), proj["k"].view(n, kv_heads, d), proj["v"].view(n, kv_heads, d)
    q, k = (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) for t in (q, k))
    cos, sin = plain.rotary_tables(torch.arange(n), d, theta, torch.float64)
    attn = plain.causal_attention(plain.apply_rotary(q, cos, sin), plain.apply_rotary(k, cos, sin), v, d ** -0.5)
    want = plain.proj_out(attn, ref, "a")
    outs, i = [], 0
    for take in (20, 13, 1, 1, 2, 1, 7):
        ctx = single_request_ctx(cache, "r", take)
        outs.append(part.forward(x[i:i + take].to(DEV).contiguous(), ctx, binding))
        i += take
    assert i == n and rel(torch.cat(outs), want) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_pre_norm_block(dtype):
    from slipstream_b200.cache import CacheManager, GroupLayout, PagedStore
    from slipstream_b200.parts import (LayerBinding, PagedAttention, PreNormBlock, RMSNorm, RotaryEncoding,
                                       SwiGLUFeedForward)
    hidden, heads, kv_heads, d, inter, eps, theta, n = 48, 3, 1, 16, 100, 1e-5, 1e4, 19
    prefix = "model.layers.0"
    block = PreNormBlock(PagedAttention(f"{prefix}.self_attn", hidden, heads, kv_heads, d, RotaryEncoding(d, theta)),
                         SwiGLUFeedForward(f"{prefix}.mlp", hidden, inter),
                         RMSNorm(f"{prefix}.input_layernorm", hidden, eps),
                         RMSNorm(f"{prefix}.post_attention_layernorm", hidden, eps))
    dev, ref = {}, {}
    for k, child in enumerate(block.children()):
        a, b = draw(child, dtype, seed=k, scale=0.5)  # scores of order one: with larger ones bfloat16's rounding
        dev.update(a); ref.update(b)                  # of queries and keys alone moves the softmax by percents
    for child in block.children():
        child.bind(dev, runtime(dtype))
    layouts = [GroupLayout(block.mixer.cache_spec(), 1)]
    cache = CacheManager(layouts, 8, 4, 2, 64)
    store = PagedStore(layouts, dtype, DEV, [[]], 2)
    x = torch.randn(n, hidden, generator=torch.Generator().manual_seed(5))
    s = {"n_q": heads, "n_kv": kv_heads, "head_dim": d, "theta": theta, "eps": eps}
    want = plain.decoder_layer(x.double(), torch.arange(n), ref, 0, s)
    ctx = single_request_ctx(cache, "r", n)
    residual, pending = block.forward(x.to(DEV).clone(), None, ctx, LayerBinding(kv=store.kv[0][0], group=0))
    got = residual.double().cpu() + pending.double().cpu()  # the last add is left to the next norm
    assert rel(got, want) < TOL[dtype]


@pytest.mark.parametrize("n, fused", [(7, True), (40, False)])
def test_pre_norm_block_chained_into_the_next_norm(n, fused):
    """`forward_chained` with the first norm of the block that runs next: with few bfloat16 tokens and a width in
    steps of 128 the branches' last projections add themselves to the stream and the norms come back pending (no
    norm kernel but the first: 5 launches); with more tokens the same call runs product, add + norm (7 launches).
    Both against the plain layer followed by the plain norm."""
    from slipstream_b200 import ops
    from slipstream_b200.cache import CacheManager, GroupLayout, PagedStore
    from slipstream_b200.parts import (LayerBinding, PagedAttention, PreNormBlock, RMSNorm, RotaryEncoding,
                                       SwiGLUFeedForward)
    dtype = torch.bfloat16
    hidden, heads, kv_heads, d, inter, eps, theta = 256, 4, 2, 64, 320, 1e-6, 1e4
    prefix = "model.layers.0"
    block = PreNormBlock(PagedAttention(f"{prefix}.self_attn", hidden, heads, kv_heads, d, RotaryEncoding(d, theta)),
                         SwiGLUFeedForward(f"{prefix}.mlp", hidden, inter),
                         RMSNorm(f"{prefix}.input_layernorm", hidden, eps),
                         RMSNorm(f"{prefix}.post_attention_layernorm", hidden, eps))
    following = RMSNorm("model.layers.1.input_layernorm", hidden, eps)
    dev, ref = {}, {}
    for k, child in enumerate(block.children() + [following]):
        a, b = draw(child, dtype, seed=k, scale=0.2)  # sums over 256 and 320 terms of order one, as in the narrow block
        dev.update(a); ref.update(b)
    for child in block.children() + [following]:
        child.bind(dev, runtime(dtype))
    layouts = [GroupLayout(block.mixer.cache_spec(), 1)]
    cache = CacheManager(layouts, 8, 8, 2, 64)
    store = PagedStore(layouts, dtype, DEV, [[]], 2)
    x = torch.randn(n, hidden, generator=torch.Generator().manual_seed(5))
    s = {"n_q": heads, "n_kv": kv_heads, "head_dim": d, "theta": theta, "eps": eps}
    out = plain.decoder_layer(x.double(), torch.arange(n), ref, 0, s)
    want = plain.rms_norm(out, ref["model.layers.1.input_layernorm.weight"].double(), eps)
    ctx = single_request_ctx(cache, "r", n)
    launches = ops.launch_count()
    residual, pending, normed = block.forward_chained(x.to(DEV).clone(), None, None, following, ctx,
                                                      LayerBinding(kv=store.kv[0][0], group=0))
    used = ops.launch_count() - launches
    assert pending is None and normed is not None
    assert isinstance(normed, ops.PendingNorm) == fused
    if fused:
        # norm, q/k/v, (rotation + pages), attention, o, gate/up, down: no norm kernel behind the first
        assert used <= 7 and normed.stream.data_ptr() == residual.data_ptr()
        got_norm = normed.materialize()
        scaled_way = normed.scaled.double() * torch.rsqrt(normed.squares.double().sum(1, keepdim=True) / hidden + eps)
        assert rel(scaled_way.cpu(), want) < TOL[dtype]
    else:
        got_norm = normed
    errors = rel(residual.double().cpu(), out), rel(got_norm.double().cpu(), want)
    assert errors[0] < TOL[dtype], errors  # the add is done: the stream is the layer's output
    assert errors[1] < TOL[dtype], errors
