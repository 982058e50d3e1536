"""Who applies which norm when a branch may end in the norm behind it: the host-side logic of
`PreNormBlock.forward_chained`, `IntoNorm`, `settle` and `DecoderLM.forward`, with parts that do arithmetic on CPU
tensors and write down what they were asked (no GPU, no kernels)."""
from types import SimpleNamespace

import torch

from slipstream_b200.models.decoder import DecoderLM
from slipstream_b200.parts.base import Embedding, FeedForward, Head, LayerBinding, Mixer, Norm
from slipstream_b200.parts.block import PreNormBlock

LOG: list[str] = []


class Pending:
    """Stands for ops.PendingNorm: a norm of the stream that has not been computed."""

    def __init__(self, norm, stream):
        self.norm, self.stream = norm, stream

    def materialize(self):
        LOG.append(f"{self.norm.name}.materialize")
        return self.norm.scale * self.stream


class FakeNorm(Norm):
    def __init__(self, name, scale, splits):
        self.name, self.scale, self.splits = name, scale, splits

    def add_norm(self, residual, delta, rows=None):
        LOG.append(f"{self.name}.add_norm" + ("[rows]" if rows is not None else ""))
        if delta is not None and rows is None:
            residual += delta
        x = residual if delta is None or rows is None else residual + delta
        return self.scale * (x if rows is None else x[rows])

    def add_norm_of_linear(self, residual, x, weight, bias):
        if not self.splits:
            return super_add_norm_of_linear(self, residual, x, weight)
        LOG.append(f"{self.name}.split")
        residual += x * weight
        return Pending(self, residual)


def super_add_norm_of_linear(norm, residual, x, weight):
    LOG.append(f"{norm.name}.linear_then_norm")
    return norm.add_norm(residual, x * weight)


def value_of(x):
    return x.norm.scale * x.stream if isinstance(x, Pending) else x


class FakeMixer(Mixer):
    def __init__(self, name, w, into, pending):
        self.name, self.w = name, w
        self.takes_into, self.takes_pending_norm = into, pending

    def forward(self, x, ctx, layer, into=None):
        LOG.append(f"{self.name}({'pending' if isinstance(x, Pending) else 'tensor'})")
        h = value_of(x) + 1.0
        return into.close(h, self.w, None) if into is not None else h * self.w


class FakeFeedForward(FeedForward):
    def __init__(self, name, w, into, pending):
        self.name, self.w = name, w
        self.takes_into, self.takes_pending_norm = into, pending

    def forward(self, x, ctx, into=None):
        LOG.append(f"{self.name}({'pending' if isinstance(x, Pending) else 'tensor'})")
        h = value_of(x) * 2.0
        return into.close(h, self.w, None) if into is not None else h * self.w


class FakeEmbedding(Embedding):
    def forward(self, token_ids):
        return token_ids.float().unsqueeze(1).repeat(1, 4)


class FakeHead(Head):
    vocab_size = 4

    def __init__(self, pending):
        self.takes_pending_norm = pending

    def forward(self, x):
        LOG.append(f"head({'pending' if isinstance(x, Pending) else 'tensor'})")
        return value_of(x) * 10.0


def build(n_blocks, into, pending, splits, head_pending=True):
    blocks = [PreNormBlock(FakeMixer(f"mix{i}", 0.5 + i, into, pending), FakeFeedForward(f"ffn{i}", 0.25, into, pending),
                           FakeNorm(f"n{i}a", 1.5, splits), FakeNorm(f"n{i}b", 0.75, splits)) for i in range(n_blocks)]
    model = DecoderLM(None, FakeEmbedding(), blocks, FakeNorm("final", 2.0, splits), FakeHead(head_pending))
    model.bindings = [LayerBinding(kv=None, group=-1) for _ in blocks]
    return model


def plain(tokens, n_blocks, rows):
    x = tokens.float().unsqueeze(1).repeat(1, 4)
    for i in range(n_blocks):
        x = x + (1.5 * x + 1.0) * (0.5 + i)
        x = x + (0.75 * x * 2.0) * 0.25
    return 2.0 * x[rows] * 10.0


def run(model, tokens, rows, every_row):
    del LOG[:]
    ctx = SimpleNamespace(token_ids=tokens, extras={"every_row_wanted": every_row}, num_logits=len(rows),
                          logit_rows=torch.tensor(rows))
    return model.forward(ctx)


def test_parts_that_take_part_pass_pending_norms_down_the_chain():
    tokens = torch.tensor([1, 2, 3])
    model = build(2, into=True, pending=True, splits=True)
    out = run(model, tokens, [0, 1, 2], every_row=True)
    assert torch.allclose(out, plain(tokens, 2, [0, 1, 2]))
    # only the first norm is computed by itself; every other is split, and nothing is materialised
    assert LOG == ["n0a.add_norm", "mix0(tensor)", "n0b.split", "ffn0(pending)", "n1a.split", "mix1(pending)", "n1b.split",
                   "ffn1(pending)", "final.split", "head(pending)"]


def test_the_final_norm_selects_rows_unless_every_row_is_wanted():
    tokens = torch.tensor([1, 2, 3])
    model = build(2, into=True, pending=True, splits=True)
    out = run(model, tokens, [2], every_row=False)
    assert torch.allclose(out, plain(tokens, 2, [2]))
    assert LOG[-3:] == ["ffn1(pending)", "final.add_norm[rows]", "head(tensor)"]


def test_a_part_that_wants_a_tensor_gets_one():
    tokens = torch.tensor([4, 5])
    model = build(2, into=True, pending=False, splits=True, head_pending=False)
    out = run(model, tokens, [0, 1], every_row=True)
    assert torch.allclose(out, plain(tokens, 2, [0, 1]))
    assert "n0b.materialize" in LOG and "final.materialize" in LOG and "head(tensor)" in LOG
    assert not any("(pending)" in entry for entry in LOG)


def test_parts_that_know_nothing_of_it_run_as_before():
    tokens = torch.tensor([4, 5])
    model = build(2, into=False, pending=False, splits=True)
    out = run(model, tokens, [1], every_row=False)
    assert torch.allclose(out, plain(tokens, 2, [1]))
    assert LOG == ["n0a.add_norm", "mix0(tensor)", "n0b.add_norm", "ffn0(tensor)", "n1a.add_norm", "mix1(tensor)",
                   "n1b.add_norm", "ffn1(tensor)", "final.add_norm[rows]", "head(tensor)"]


def test_a_norm_that_cannot_be_split_runs_behind_the_projection():
    tokens = torch.tensor([7])
    model = build(1, into=True, pending=True, splits=False)
    out = run(model, tokens, [0], every_row=True)
    assert torch.allclose(out, plain(tokens, 1, [0]))
    assert LOG == ["n0a.add_norm", "mix0(tensor)", "n0b.linear_then_norm", "n0b.add_norm", "ffn0(tensor)",
                   "final.linear_then_norm", "final.add_norm", "head(tensor)"]
