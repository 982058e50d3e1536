"""The plain implementation against the reference's own model code (stored outputs made by
tests/golden/make_golden.py), and against itself where parts can be checked alone."""
import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen2 as plain

GOLDEN = Path(__file__).parent / "golden" / "tiny_qwen2_reference.npz"


@pytest.mark.parametrize("case", ["tied", "untied"])
def test_plain_matches_reference_model_code(case):
    data = np.load(GOLDEN)
    config = json.loads(bytes(data[f"{case}/config"]).decode())
    weights = {k.split("/w/", 1)[1]: torch.from_numpy(data[k]) for k in data.files if k.startswith(f"{case}/w/")}
    tokens = data[f"{case}/tokens"].tolist()
    want = torch.from_numpy(data[f"{case}/logits"])
    got = plain.forward_logits(config, weights, tokens)
    assert got.shape == want.shape
    assert (got - want).abs().max().item() < 2e-6
    # float64 arithmetic agrees with the float32 reference to float32 rounding
    got64 = plain.forward_logits(config, {k: v.double() for k, v in weights.items()}, tokens)
    assert (got64.float() - want).abs().max().item() < 1e-5


def test_rms_norm_formula():
    x = torch.randn(5, 24, dtype=torch.float64)
    w = torch.randn(24, dtype=torch.float64)
    got = plain.rms_norm(x, w, 1e-5)
    want = w * x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5)
    assert torch.allclose(got, want, atol=1e-12)


def test_rotary_is_a_rotation_by_position_times_frequency():
    d, theta = 8, 100.0
    pos = torch.tensor([0, 3, 11])
    cos, sin = plain.rotary_tables(pos, d, theta, torch.float64)
    x = torch.randn(3, 2, d, dtype=torch.float64)
    y = plain.apply_rotary(x, cos, sin)
    for t, p in enumerate(pos.tolist()):
        for i in range(d // 2):
            ang = p * float(plain.inverse_frequencies(d, theta)[i])
            a, b = x[t, 0, i].item(), x[t, 0, i + d // 2].item()
            assert math.isclose(y[t, 0, i].item(), a * math.cos(ang) - b * math.sin(ang), abs_tol=1e-6)
            assert math.isclose(y[t, 0, i + d // 2].item(), b * math.cos(ang) + a * math.sin(ang), abs_tol=1e-6)
    assert torch.equal(y[0], x[0])  # position 0 is the identity


def test_attention_is_causal_and_shares_kv_heads():
    torch.manual_seed(0)
    q = torch.randn(6, 4, 8, dtype=torch.float64)
    k = torch.randn(6, 2, 8, dtype=torch.float64)
    v = torch.randn(6, 2, 8, dtype=torch.float64)
    out = plain.causal_attention(q, k, v, 8 ** -0.5).view(6, 4, 8)
    # row 0 sees only key 0
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])
    # changing a later key does not change earlier rows
    k2 = k.clone(); k2[5] += 1.0
    out2 = plain.causal_attention(q, k2, v, 8 ** -0.5).view(6, 4, 8)
    assert torch.equal(out[:5], out2[:5]) and not torch.equal(out[5], out2[5])
    # one row by hand
    h, g = 2, 1
    s = (q[3, h] @ k[:4, g].T) * 8 ** -0.5
    want = torch.softmax(s, -1) @ v[:4, g]
    assert torch.allclose(out[3, h], want)


def test_filtered_logits_chain():
    logits = torch.tensor([2.0, 1.0, 0.5, -1.0, 3.0])
    out = plain.filtered_logits(logits, temperature=0.5, top_k=3)
    assert torch.isinf(out[[2, 3]]).all() and out[4] == 6.0
    out = plain.filtered_logits(logits, temperature=1.0, top_p=0.7)
    probs = torch.softmax(logits.double(), -1)
    # sorted: 3.0 (idx4), 2.0 (idx0), ...: keep while the mass before a token is < top_p
    kept = [4] + ([0] if probs[4] < 0.7 else [])
    assert sorted(torch.nonzero(~torch.isinf(out)).flatten().tolist()) == sorted(kept + ([1] if probs[4] + probs[0] < 0.7 else []))
    out = plain.filtered_logits(logits, temperature=1.0, min_p=0.2)
    assert torch.isinf(out[3]) and not torch.isinf(out[0])
    out = plain.filtered_logits(logits, temperature=1.0, repetition_penalty=2.0, history=[0, 3, 3])
    assert out[0] == 1.0 and out[3] == -2.0 and out[1] == 1.0
    assert plain.greedy_token(torch.tensor([1.0, 5.0, 5.0])) == 1
