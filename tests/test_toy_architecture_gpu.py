"""A toy architecture defined HERE, registered, built and stepped without a change to the package:
a mixer with fixed-size state of its own (a running mean), an attention layer with a window, a block
that the execution order names twice, and an entry that reads another entry's cache.  It is checked
against a plain whole-sequence restatement written in this file, under several ways of cutting."""
from dataclasses import asdict, dataclass
from typing import ClassVar

import pytest
import torch

import plain_qwen2 as plain
from conftest import random_tokens

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@dataclass(frozen=True)
class ToyConfig:
    architecture: ClassVar[str] = "ToyMixForCausalLM"
    vocab_size: int = 97
    hidden_size: int = 40
    num_hidden_layers: int = 4
    max_position_embeddings: int = 512
    torch_dtype: str = "float32"
    eos_token_id: int | None = None
    heads: int = 5
    kv_heads: int = 1
    head_dim: int = 16
    inter: int = 72
    eps: float = 1e-5
    theta: float = 2000.0
    window: int = 9
    window_page: int | None = None  # tokens per cache page of the windowed layer; None: the engine's default

    @classmethod
    def from_dict(cls, data, generation=None):
        return cls(**{k: v for k, v in data.items() if k in cls.__dataclass_fields__})

    def to_dict(self):
        return dict(asdict(self), architectures=[self.architecture])


def define_toy():
    """Everything a user would write to add a mixer and an architecture."""
    from slipstream_b200.models.decoder import DecoderLM, ExecEntry
    from slipstream_b200.parts import (MIXERS, LMHead, Mixer, PagedAttention, PreNormBlock, RMSNorm, RotaryEncoding,
                                       StateSpec, SwiGLUFeedForward, TokenEmbedding, WeightSpec)
    from slipstream_b200.registry import register_architecture, unregister_architecture

    MIXERS.unregister("running_mean")

    @MIXERS.register("running_mean")
    class RunningMean(Mixer):
        """y_t = W * mean(x_0 .. x_t): needs the sum and the count of what it has seen, per request."""

        def __init__(self, name, hidden):
            self.name, self.hidden = name, hidden

        def weight_specs(self):
            return [WeightSpec(f"{self.name}.mix.weight", (self.hidden, self.hidden), init=("normal", 0.3))]

        def state_specs(self):
            return [StateSpec("sum", (self.hidden,), torch.float32), StateSpec("count", (1,), torch.float32)]

        def bind(self, weights, runtime):
            super().bind(weights, runtime)
            self.weight = weights[f"{self.name}.mix.weight"]

        def forward(self, x, ctx, layer):
            out = torch.empty_like(x)
            starts = ctx.q_start.tolist()
            for r, slot in enumerate(ctx.state_slots.tolist()):
                rows = x[starts[r]: starts[r + 1]].float()
                total = layer.state["sum"][slot] + rows.cumsum(0)
                count = layer.state["count"][slot] + torch.arange(1, rows.shape[0] + 1, device=x.device)[:, None]
                out[starts[r]: starts[r + 1]] = ((total / count) @ self.weight.float().T).to(x.dtype)
                layer.state["sum"][slot] = total[-1]
                layer.state["count"][slot] = count[-1]
            return out

    def build(c: ToyConfig):
        rotary = RotaryEncoding(c.head_dim, c.theta)

        def block(i, mixer):
            p = f"toy.layers.{i}"
            return PreNormBlock(mixer, SwiGLUFeedForward(f"{p}.mlp", c.hidden_size, c.inter),
                                RMSNorm(f"{p}.norm1", c.hidden_size, c.eps), RMSNorm(f"{p}.norm2", c.hidden_size, c.eps))

        def attention(i, window):
            return PagedAttention(f"toy.layers.{i}.attn", c.hidden_size, c.heads, c.kv_heads, c.head_dim, rotary,
                                  qkv_bias=False, window=window, page_size=c.window_page if window else None)

        blocks = [block(0, attention(0, None)), block(1, MIXERS.get("running_mean")("toy.layers.1", c.hidden_size)),
                  block(2, attention(2, c.window)), block(3, attention(3, None))]
        # block 0 runs twice (pages of its own each time); the last entry reads the pages entry 0 wrote
        order = [ExecEntry(0), ExecEntry(1), ExecEntry(2), ExecEntry(0), ExecEntry(3, cache_of=0)]
        return DecoderLM(c, TokenEmbedding("toy.embed", c.vocab_size, c.hidden_size), blocks,
                         RMSNorm("toy.norm", c.hidden_size, c.eps), LMHead("toy.head", c.vocab_size, c.hidden_size, None),
                         order=order)

    unregister_architecture("ToyMixForCausalLM")
    register_architecture("ToyMixForCausalLM", ToyConfig, build)
    return build


# --------------------------------------------------------------------------- plain restatement

def plain_attention(x, w, prefix, c, window, kv_from=None):
    T = x.shape[0]
    q = (x @ w[f"{prefix}.q_proj.weight"].T).view(T, c.heads, c.head_dim)
    k = (x @ w[f"{prefix}.k_proj.weight"].T).view(T, c.kv_heads, c.head_dim)
    v = (x @ w[f"{prefix}.v_proj.weight"].T).view(T, c.kv_heads, c.head_dim)
    cos, sin = plain.rotary_tables(torch.arange(T), c.head_dim, c.theta, x.dtype)
    q, k = plain.apply_rotary(q, cos, sin), plain.apply_rotary(k, cos, sin)
    made = (k, v)
    if kv_from is not None:
        k, v = kv_from
    g = c.heads // c.kv_heads
    s = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(g, 1)) * c.head_dim ** -0.5
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    ok = j <= i
    if window:
        ok &= j > i - window
    s = s.masked_fill(~ok[None], float("-inf"))
    out = torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), v.repeat_interleave(g, 1)).reshape(T, -1)
    return out @ w[f"{prefix}.o_proj.weight"].T, made


def plain_toy(c, w, tokens):
    x = w["toy.embed.weight"][torch.as_tensor(tokens)]
    T = x.shape[0]
    kv0 = None
    for pos, (i, kind) in enumerate([(0, "full"), (1, "mean"), (2, "window"), (0, "full"), (3, "shared")]):
        p = f"toy.layers.{i}"
        h = plain.rms_norm(x, w[f"{p}.norm1.weight"], c.eps)
        if kind == "mean":
            mixed = (h.cumsum(0) / torch.arange(1, T + 1)[:, None]) @ w[f"{p}.mix.weight"].T
        else:
            mixed, made = plain_attention(h, w, f"{p}.attn", c, c.window if kind == "window" else None,
                                          kv_from=kv0 if kind == "shared" else None)
            if pos == 0:
                kv0 = made
        x = x + mixed
        x = x + plain.swiglu_mlp(plain.rms_norm(x, w[f"{p}.norm2.weight"], c.eps), w, f"{p}.mlp")
    return plain.rms_norm(x, w["toy.norm.weight"], c.eps) @ w["toy.head.weight"].T


# --------------------------------------------------------------------------- the test

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_steps_like_its_plain_restatement(tmp_path, dtype):
    from safetensors.torch import load_file, save_file
    from slipstream_b200.engine.runner import ModelRunner, StepEntry
    from slipstream_b200.registry import unregister_architecture
    from slipstream_b200.weights.random_init import write_random_model

    define_toy()
    try:
        c = ToyConfig()
        write_random_model(c, tmp_path, seed=5)
        tensors = {k: v.clone() for k, v in load_file(str(tmp_path / "model.safetensors")).items()}  # not views of the file
        for k in tensors:  # far from uniform attention, visible feed-forward
            if "q_proj" in k or "k_proj" in k:
                tensors[k] = tensors[k] * 12
            elif tensors[k].dim() == 2 and "mix" not in k:
                tensors[k] = tensors[k] * 4
        save_file(tensors, str(tmp_path / "model.safetensors"))
        w = {k: (v.bfloat16() if dtype == "bfloat16" and v.dim() == 2 else v).double() for k, v in tensors.items()}

        page = 4
        runner = ModelRunner(str(tmp_path), dtype=dtype, page_size=page, num_pages=40, max_num_seqs=3)
        model = runner.model
        # two cache groups: all keys (three writers: entries 0 and 3; entry 4 shares 0's) and a window
        specs = [(l.spec.window, l.num_entries) for l in model.group_layouts]
        assert sorted(specs, key=str) == sorted([(None, 2), (c.window, 1)], key=str)
        assert not runner.use_cuda_graphs  # the toy mixer did not declare itself safe to capture
        assert [len(s) for s in model.entry_state] == [0, 2, 0, 0, 0]

        reqs = {"a": random_tokens(c.vocab_size, 61, 1), "b": random_tokens(c.vocab_size, 30, 2), "c": random_tokens(c.vocab_size, 47, 3)}
        want = {k: plain_toy(c, w, v).float() for k, v in reqs.items()}
        tol = (3e-5 if dtype == "float32" else 4e-2)

        def check(rows, what):
            for k, ref in want.items():
                err = (torch.cat(rows[k]) - ref).abs().max(dim=1).values
                assert err.max() <= tol * ref.abs().max(), (what, k, int(err.argmax()), err.max().item())

        # whole, each alone
        rows = {}
        for k, toks in reqs.items():
            rows[k] = [runner.step([StepEntry(k, toks, list(range(len(toks))))]).cpu()]
            runner.release(k)
        check(rows, "whole")
        # portions and single tokens, all three live at once; windowed pages are given back on the way
        rows = {k: [] for k in reqs}
        at = {k: 0 for k in reqs}
        sizes = {"a": [7, 1, 1, 13, 2, 1, 30, 1, 5], "b": [2, 2, 1, 1, 1, 20, 3], "c": [40, 1, 1, 1, 1, 1, 1, 1]}
        held_window_pages = []
        for step in range(9):
            entries = []
            for k in reqs:
                if step < len(sizes[k]):
                    take = sizes[k][step]
                    entries.append(StepEntry(k, reqs[k][at[k]: at[k] + take], list(range(take))))
                    at[k] += take
            out = runner.step(entries).cpu()
            i = 0
            for e in entries:
                rows[e.request_id].append(out[i: i + len(e.tokens)])
                i += len(e.tokens)
            runner.cache.check_invariants()
            g = [n for n, l in enumerate(model.group_layouts) if l.spec.window][0]
            held_window_pages.append(max(sum(p >= 0 for p in runner.cache.get(k).tables[g]) for k in reqs))
        assert all(at[k] == len(reqs[k]) for k in reqs)
        check(rows, "portions")
        assert held_window_pages[-1] <= (c.window + page - 1) // page + 1
        for k in reqs:
            runner.release(k)
        assert all(p.num_free == 40 for p in runner.cache.pools)
        # a released slot is zeroed for its next request: replay "a" in the slot "c" used last
        rows = {"a": [runner.step([StepEntry("a2", reqs["a"], list(range(61)))]).cpu()]}
        err = (rows["a"][0] - want["a"]).abs().max()
        assert err <= tol * want["a"].abs().max()
        runner.check()
    finally:
        unregister_architecture("ToyMixForCausalLM")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_cache_group_with_its_own_page_size_and_a_quarter_of_the_pages(tmp_path, dtype):
    """The same toy as a hybrid whose windowed layer keeps its keys in pages of 8 tokens, 10 of them, beside the
    other layers' 40 pages of 4: every group has its own pool, page size and block table.  Whole requests, then
    three live requests in portions and single tokens, against the plain restatement."""
    from slipstream_b200.engine.runner import ModelRunner, StepEntry
    from slipstream_b200.registry import unregister_architecture
    from slipstream_b200.weights.random_init import write_random_model
    from conftest import sharpen

    define_toy()
    try:
        c = ToyConfig(window_page=8)
        write_random_model(c, tmp_path, seed=6)
        sharpen(tmp_path, factor=10.0)
        _, tensors = plain.read_model_folder(tmp_path, torch.float32)
        w = {k: (v.bfloat16() if dtype == "bfloat16" and v.dim() == 2 else v).double() for k, v in tensors.items()}
        runner = ModelRunner(str(tmp_path), dtype=dtype, page_size=4, num_pages=[40, 10], max_num_seqs=3)
        cache = runner.cache
        assert [(l.spec.window, l.page_size, l.num_pages) for l in runner.model.group_layouts] == [(None, 4, 40), (9, 8, 10)]
        assert [t.shape[1] for t in runner.store.kv] == [40, 10] and [t.shape[4] for t in runner.store.kv] == [4, 8]
        reqs = {"a": random_tokens(c.vocab_size, 61, 11), "b": random_tokens(c.vocab_size, 30, 12),
                "c": random_tokens(c.vocab_size, 47, 13)}
        want = {k: plain_toy(c, w, v).float() for k, v in reqs.items()}
        tol = 3e-5 if dtype == "float32" else 4e-2

        def check(rows, what):
            for k, ref in want.items():
                err = (torch.cat(rows[k]) - ref).abs().max(dim=1).values
                assert err.max() <= tol * ref.abs().max(), (what, k, int(err.argmax()), err.max().item())

        rows = {}
        for k, toks in reqs.items():
            rows[k] = [runner.step([StepEntry(k, toks, list(range(len(toks))))]).cpu()]
            runner.release(k)
        check(rows, "whole")
        rows, at = {k: [] for k in reqs}, {k: 0 for k in reqs}
        sizes = {"a": [7, 1, 1, 13, 2, 1, 14, 16, 1, 5], "b": [2, 2, 1, 1, 1, 12, 8, 3], "c": [24, 16, 1, 1, 1, 1, 1, 1, 1]}
        fewest_free = [40, 10]
        for step in range(10):
            entries = []
            for k in reqs:
                if step < len(sizes[k]):
                    take = sizes[k][step]
                    entries.append(StepEntry(k, reqs[k][at[k]: at[k] + take], list(range(take))))
                    at[k] += take
            out = runner.step(entries).cpu()
            i = 0
            for e in entries:
                rows[e.request_id].append(out[i: i + len(e.tokens)])
                i += len(e.tokens)
            cache.check_invariants()
            fewest_free = [min(a, b) for a, b in zip(fewest_free, cache.free_pages())]
        assert all(at[k] == len(reqs[k]) for k in reqs)
        check(rows, "portions")
        assert fewest_free[1] <= 4, "the small pool was never under pressure"
        for k in reqs:
            runner.release(k)
        assert cache.all_pages_free() and cache.free_pages() == [40, 10]
        runner.check()
    finally:
        unregister_architecture("ToyMixForCausalLM")


# =========================================================================== a second toy: other parts again
# A feed-forward with routing (every token goes to the one expert its router picks) and another position
# encoding (a learned table added to the stream; queries and keys are not rotated), again defined here and
# registered without a change to the package.

@dataclass(frozen=True)
class RoutedConfig:
    architecture: ClassVar[str] = "ToyRoutedForCausalLM"
    vocab_size: int = 113
    hidden_size: int = 48
    num_hidden_layers: int = 2
    max_position_embeddings: int = 160
    torch_dtype: str = "float32"
    eos_token_id: int | None = None
    heads: int = 3
    kv_heads: int = 3
    head_dim: int = 16
    experts: int = 4
    inter: int = 40
    eps: float = 1e-6

    @classmethod
    def from_dict(cls, data, generation=None):
        return cls(**{k: v for k, v in data.items() if k in cls.__dataclass_fields__})

    def to_dict(self):
        return dict(asdict(self), architectures=[self.architecture])


def define_routed():
    from slipstream_b200.models.decoder import DecoderLM
    from slipstream_b200.parts import (FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, LMHead, NoPositionEncoding,
                                       PagedAttention, PositionEncoding, PreNormBlock, RMSNorm, TokenEmbedding, WeightSpec)
    from slipstream_b200.registry import register_architecture, unregister_architecture

    FEED_FORWARDS.unregister("top1_experts")
    POSITION_ENCODINGS.unregister("learned_table")

    @FEED_FORWARDS.register("top1_experts")
    class Top1Experts(FeedForward):
        """y = p_e * W2_e relu(W1_e x) for the expert e with the largest router logit; p = softmax(router)."""

        def __init__(self, name, hidden, inter, experts):
            self.name, self.hidden, self.inter, self.experts = name, hidden, inter, experts

        def weight_specs(self):
            n = self.name
            return ([WeightSpec(f"{n}.router.weight", (self.experts, self.hidden), init=("normal", 1.0))] +
                    [WeightSpec(f"{n}.experts.{e}.w1.weight", (self.inter, self.hidden), init=("normal", 0.3)) for e in range(self.experts)] +
                    [WeightSpec(f"{n}.experts.{e}.w2.weight", (self.hidden, self.inter), init=("normal", 0.3)) for e in range(self.experts)])

        def bind(self, weights, runtime):
            super().bind(weights, runtime)
            n = self.name
            self.router = weights[f"{n}.router.weight"]
            self.w1 = torch.stack([weights[f"{n}.experts.{e}.w1.weight"] for e in range(self.experts)])
            self.w2 = torch.stack([weights[f"{n}.experts.{e}.w2.weight"] for e in range(self.experts)])

        def forward(self, x, ctx):
            logits = x.float() @ self.router.float().T          # router logits in float32
            probs = torch.softmax(logits, -1)
            pick = logits.argmax(-1)
            out = torch.zeros_like(x)
            for e in range(self.experts):                        # tokens of one expert together
                rows = (pick == e).nonzero().flatten()
                if rows.numel():
                    h = torch.relu(x[rows] @ self.w1[e].T)
                    out[rows] = ((h @ self.w2[e].T).float() * probs[rows, e, None]).to(x.dtype)
            return out

    @POSITION_ENCODINGS.register("learned_table")
    class LearnedTable(PositionEncoding):
        """One learned vector per position, added to the stream after the embedding."""

        def __init__(self, name, positions, hidden):
            self.name, self.positions, self.hidden = name, positions, hidden

        def weight_specs(self):
            return [WeightSpec(f"{self.name}.weight", (self.positions, self.hidden), init=("normal", 0.5))]

        def bind(self, weights, runtime):
            super().bind(weights, runtime)
            self.table = weights[f"{self.name}.weight"]

        def on_embedding(self, residual, ctx):
            residual += self.table[ctx.positions.long()].float()

    def build(c: RoutedConfig):
        def block(i):
            p = f"routed.layers.{i}"
            attn = PagedAttention(f"{p}.attn", c.hidden_size, c.heads, c.kv_heads, c.head_dim, NoPositionEncoding(), qkv_bias=True)
            return PreNormBlock(attn, Top1Experts(f"{p}.moe", c.hidden_size, c.inter, c.experts),
                                RMSNorm(f"{p}.norm1", c.hidden_size, c.eps), RMSNorm(f"{p}.norm2", c.hidden_size, c.eps))

        return DecoderLM(c, TokenEmbedding("routed.embed", c.vocab_size, c.hidden_size),
                         [block(i) for i in range(c.num_hidden_layers)], RMSNorm("routed.norm", c.hidden_size, c.eps),
                         LMHead("routed.head", c.vocab_size, c.hidden_size, None),
                         position_encoding=LearnedTable("routed.positions", c.max_position_embeddings, c.hidden_size))

    unregister_architecture("ToyRoutedForCausalLM")
    register_architecture("ToyRoutedForCausalLM", RoutedConfig, build)


def plain_routed(c, w, tokens):
    T = len(tokens)
    x = w["routed.embed.weight"][torch.as_tensor(tokens)] + w["routed.positions.weight"][:T]
    picks = []
    for i in range(c.num_hidden_layers):
        p = f"routed.layers.{i}"
        h = plain.rms_norm(x, w[f"{p}.norm1.weight"], c.eps)
        q = (h @ w[f"{p}.attn.q_proj.weight"].T + w[f"{p}.attn.q_proj.bias"]).view(T, c.heads, c.head_dim)
        k = (h @ w[f"{p}.attn.k_proj.weight"].T + w[f"{p}.attn.k_proj.bias"]).view(T, c.kv_heads, c.head_dim)
        v = (h @ w[f"{p}.attn.v_proj.weight"].T + w[f"{p}.attn.v_proj.bias"]).view(T, c.kv_heads, c.head_dim)
        s = torch.einsum("ihd,jhd->hij", q, k) * c.head_dim ** -0.5
        s = s.masked_fill(~(torch.arange(T)[None, :] <= torch.arange(T)[:, None])[None], float("-inf"))
        x = x + torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), v).reshape(T, -1) @ w[f"{p}.attn.o_proj.weight"].T
        h = plain.rms_norm(x, w[f"{p}.norm2.weight"], c.eps)
        logits = h @ w[f"{p}.moe.router.weight"].T
        probs, pick = torch.softmax(logits, -1), logits.argmax(-1)
        picks.append((pick, logits))
        y = torch.zeros_like(x)
        for t in range(T):
            e = int(pick[t])
            y[t] = probs[t, e] * (torch.relu(h[t] @ w[f"{p}.moe.experts.{e}.w1.weight"].T) @ w[f"{p}.moe.experts.{e}.w2.weight"].T)
        x = x + y
    return plain.rms_norm(x, w["routed.norm.weight"], c.eps) @ w["routed.head.weight"].T, picks


def test_toy_routing_and_a_learned_position_table(tmp_path):
    """float32: the router's pick must not flip between the engine and the plain restatement, which a
    reduced-precision path could not promise; every expert is used."""
    from safetensors.torch import load_file
    from slipstream_b200.engine.runner import ModelRunner, StepEntry
    from slipstream_b200.registry import unregister_architecture
    from slipstream_b200.weights.random_init import write_random_model

    define_routed()
    try:
        c = RoutedConfig()
        write_random_model(c, tmp_path, seed=11)
        w = {k: v.clone().double() for k, v in load_file(str(tmp_path / "model.safetensors")).items()}
        runner = ModelRunner(str(tmp_path), dtype="float32", page_size=8, num_pages=24, max_num_seqs=2)
        assert not runner.use_cuda_graphs  # the toy parts did not declare themselves safe to capture
        reqs = {"a": random_tokens(c.vocab_size, 70, 4), "b": random_tokens(c.vocab_size, 33, 5)}
        want = {}
        used = set()
        for k, toks in reqs.items():
            ref, picks = plain_routed(c, w, toks)
            want[k] = ref.float()
            for pick, logits in picks:
                used |= set(pick.tolist())
                top2 = logits.topk(2, -1).values
                assert (top2[:, 0] - top2[:, 1]).min() > 1e-4, "a router tie would make the comparison meaningless"
        assert used == set(range(c.experts))

        def check(rows, what):
            for k, ref in want.items():
                err = (torch.cat(rows[k]) - ref).abs().max()
                assert err <= 3e-5 * ref.abs().max(), (what, k, err.item())

        rows = {}
        for k, toks in reqs.items():
            rows[k] = [runner.step([StepEntry(k, toks, list(range(len(toks))))]).cpu()]
            runner.release(k)
        check(rows, "whole")
        # both live: portions of one beside single tokens of the other
        rows, at = {k: [] for k in reqs}, {k: 0 for k in reqs}
        sizes = {"a": [30, 1, 1, 1, 2, 35], "b": [1, 1, 20, 1, 1, 9]}
        for step in range(6):
            entries = []
            for k in reqs:
                take = sizes[k][step]
                entries.append(StepEntry(k, reqs[k][at[k]: at[k] + take], list(range(take))))
                at[k] += take
            out = runner.step(entries).cpu()
            i = 0
            for e in entries:
                rows[e.request_id].append(out[i: i + len(e.tokens)])
                i += len(e.tokens)
        assert all(at[k] == len(reqs[k]) for k in reqs)
        check(rows, "portions")
        runner.check()
    finally:
        unregister_architecture("ToyRoutedForCausalLM")
