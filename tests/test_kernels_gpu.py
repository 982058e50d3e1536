"""Each CUDA kernel alone against a plain float32/float64 PyTorch restatement of the same op, at sizes
other than the engine's test models (widths and vocabularies that are no power of two, head sizes in
steps of 16, odd group sizes, pages of odd size)."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from slipstream_b200 import ops as o
    return o


def tol(dtype, f32=1e-5, bf16=1.6e-2):
    return f32 if dtype == torch.float32 else bf16


def rel_err(got, ref):
    return ((got.double() - ref.double()).abs().max() / ref.double().abs().max().clamp_min(1e-30)).item()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden, vocab", [(72, 101), (3584, 1000)])
def test_embedding(dtype, hidden, vocab):
    table = torch.randn(vocab, hidden, device=DEV).to(dtype)
    ids = torch.randint(0, vocab, (37,), device=DEV, dtype=torch.int32)
    got = ops().embedding(ids, table)
    assert got.dtype == torch.float32 and torch.equal(got, table[ids.long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [48, 1000, 3584, 5120])
def test_add_rmsnorm(dtype, hidden):
    torch.manual_seed(hidden)
    n, eps = 19, 1e-5
    residual = torch.randn(n, hidden, device=DEV) * 3
    delta = torch.randn(n, hidden, device=DEV).to(dtype)
    weight = (1 + 0.1 * torch.randn(hidden, device=DEV)).to(dtype)
    summed = residual.double() + delta.double()
    ref = summed * torch.rsqrt(summed.pow(2).mean(-1, keepdim=True) + eps) * weight.double()
    res = residual.clone()
    got = ops().add_rmsnorm(res, delta, weight, eps, dtype)
    assert rel_err(got, ref) < tol(dtype, 2e-6, 1.2e-2)
    assert torch.allclose(res.double(), summed, atol=1e-6)  # the stream is updated in float32
    # without a delta; and selected rows only, which leaves the stream alone
    got = ops().add_rmsnorm(res, None, weight, eps, dtype)
    assert rel_err(got, ref) < tol(dtype, 2e-6, 1.2e-2)
    rows = torch.tensor([5, 0, 18], device=DEV, dtype=torch.int32)
    res2 = residual.clone()
    got = ops().add_rmsnorm(res2, delta, weight, eps, dtype, rows=rows)
    assert rel_err(got, ref[rows.long()]) < tol(dtype, 2e-6, 1.2e-2) and torch.equal(res2, residual)
    # a float32 weight beside bfloat16 activations
    if dtype == torch.bfloat16:
        got = ops().add_rmsnorm(residual.clone(), delta, weight.float(), eps, dtype)
        assert rel_err(got, ref) < 1.2e-2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q, n_kv, d, rot, page", [(6, 2, 16, 16, 4), (7, 1, 48, 48, 5), (8, 8, 128, 64, 16), (3, 3, 80, 0, 7), (28, 4, 128, 128, 16), (5, 1, 32, 8, 8)])
def test_rope_and_cache(dtype, n_q, n_kv, d, rot, page):
    torch.manual_seed(d)
    n, pages, theta = 23, 9, 50000.0
    qkv = torch.randn(n, (n_q + 2 * n_kv) * d, device=DEV).to(dtype)
    pos = torch.randint(0, 5000, (n,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(pages * page, device=DEV)[:n].to(torch.int32)
    slots[3] = -1  # this token is not written
    kv = torch.zeros(pages, 2, n_kv, page, d, device=DEV, dtype=dtype)
    inv_freq = None
    x = qkv.double().view(n, n_q + 2 * n_kv, d).clone()
    ref = x.clone()
    if rot:
        inv_freq = (1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(DEV)
        # the angle is a float32 product, as in slipstream/models/layers/rope.py:100
        ang = (pos.float()[:, None] * inv_freq[None, :]).double()
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
        x1, x2 = x[:, : n_q + n_kv, : rot // 2], x[:, : n_q + n_kv, rot // 2: rot]
        ref[:, : n_q + n_kv, : rot // 2] = x1 * c - x2 * s
        ref[:, : n_q + n_kv, rot // 2: rot] = x2 * c + x1 * s
    work = qkv.clone()
    ops().rope_and_cache(work, pos, slots, inv_freq, kv, n_q, n_kv, d, rot)
    got = work.view(n, n_q + 2 * n_kv, d)
    assert rel_err(got[:, :n_q], ref[:, :n_q]) < tol(dtype, 3e-6, 8e-3)
    for t in range(n):
        if slots[t] < 0:
            continue
        p, o = int(slots[t]) // page, int(slots[t]) % page
        assert rel_err(kv[p, 0, :, o], ref[t, n_q: n_q + n_kv]) < tol(dtype, 3e-6, 8e-3)
        assert torch.equal(kv[p, 1, :, o], qkv.view(n, -1, d)[t, n_q + n_kv:])
    assert int((kv != 0).any(-1).any(-1).any(-1).sum()) <= n - 1  # no other page touched
    ops().check_errors(torch.device(DEV))


def test_gather_tokens_takes_only_the_rows_that_name_a_source():
    ids = torch.tensor([5, 6, 7, 8, 9, 10], dtype=torch.int32, device=DEV)
    src = torch.tensor([-1, 2, -1, 0, 1, -1], dtype=torch.int32, device=DEV)
    pending = torch.tensor([100, 200, 300], dtype=torch.int32, device=DEV)
    ops().gather_tokens(ids, src, pending)
    assert ids.tolist() == [5, 300, 7, 100, 200, 10]


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    x = (torch.randn(13, 2 * 1234, device=DEV) * 3).to(dtype)
    g, u = x[:, :1234].double(), x[:, 1234:].double()
    assert rel_err(ops().swiglu(x), g * torch.sigmoid(g) * u) < tol(dtype, 2e-6, 8e-3)
    # gate and up alternating in runs of 2 and of 617 columns
    for block in (2, 617):
        v = x.double().view(13, 1234 // block, 2, block)
        g, u = v[:, :, 0].reshape(13, 1234), v[:, :, 1].reshape(13, 1234)
        assert rel_err(ops().swiglu(x, block=block), g * torch.sigmoid(g) * u) < tol(dtype, 2e-6, 8e-3)
    # widths that take the 16-byte path in bfloat16: runs of 64, of 8, and the plain [gate | up]
    x = (torch.randn(70, 2 * 1280, device=DEV) * 3).to(dtype)
    for block in (64, 8, 1280):
        v = x.double().view(70, 1280 // block, 2, block)
        g, u = v[:, :, 0].reshape(70, 1280), v[:, :, 1].reshape(70, 1280)
        assert rel_err(ops().swiglu(x, block=block), g * torch.sigmoid(g) * u) < tol(dtype, 2e-6, 8e-3)


@pytest.mark.parametrize("m, n, k", [(1, 130, 70), (37, 65, 1000), (200, 333, 96)])
def test_float32_matrix_product_is_exact_to_rounding_and_independent_of_the_batch(m, n, k):
    torch.manual_seed(m)
    x, w, b = torch.randn(m, k, device=DEV), torch.randn(n, k, device=DEV), torch.randn(n, device=DEV)
    got = ops().gemm_simt(x, w, b)
    ref = x.double() @ w.double().T + b.double()
    assert rel_err(got, ref) < 2e-6  # TF32 would be 1e-3
    alone = ops().gemm_simt(x[:1].contiguous(), w, b)
    assert torch.equal(alone, got[:1])


def test_bfloat16_linear_gives_float32_logits():
    x, w = torch.randn(5, 200, device=DEV).bfloat16(), torch.randn(1001, 200, device=DEV).bfloat16()
    got = ops().linear(x, w, None, out_dtype=torch.float32)
    assert got.dtype == torch.float32 and rel_err(got, x.double() @ w.double().T) < 1e-5
    got = ops().gemm_simt(x, w, None, out_dtype=torch.float32)
    assert rel_err(got, x.double() @ w.double().T) < 1e-5


# --------------------------------------------------------------------------- attention

def make_attention_case(dtype, lens, q_lens, n_q, n_kv, d, page, seed, sharp=None):
    """Random pages in random order; returns tensors for the kernels and per-request dense K, V."""
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    blocks = [(l + page - 1) // page for l in lens]
    pages = sum(blocks) + 3
    perm = torch.randperm(pages, generator=g).tolist()
    max_blocks = max(blocks)
    table = torch.full((R, max_blocks), -1, dtype=torch.int32)
    kv = torch.randn(pages, 2, n_kv, page, d, generator=g) * 0.5
    k = 0
    for r in range(R):
        for b in range(blocks[r]):
            table[r, b] = perm[k]
            k += 1
    if sharp is not None:  # one far key stands out for the last query of request 0
        key_pos = sharp
        kv[table[0, key_pos // page], 0, :, key_pos % page] *= 0
    N = sum(q_lens)
    q = torch.randn(N, n_q, d, generator=g)
    q_start = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    if sharp is not None:
        row = int(q_start[1]) - 1
        direction = torch.randn(d, generator=g)
        direction /= direction.norm()
        q[row] = direction * 6
        kv[table[0, sharp // page], 0, :, sharp % page] = direction * 6
        kv[table[0, sharp // page], 1, :, sharp % page] = 5.0
    return (q.to(dtype).to(DEV), kv.to(dtype).to(DEV), table.to(DEV), q_start.to(DEV),
            torch.tensor(lens, dtype=torch.int32, device=DEV))


def attention_reference(q, kv, table, q_start, seq_lens, n_kv, page, scale, window):
    N, n_q, d = q.shape
    out = torch.zeros(N, n_q, d, dtype=torch.float64)
    qd, kvd = q.double().cpu(), kv.double().cpu()
    G = n_q // n_kv
    for r in range(seq_lens.numel()):
        a, b, S = int(q_start[r]), int(q_start[r + 1]), int(seq_lens[r])
        T = b - a
        nb = (S + page - 1) // page
        pg = table[r, :nb].long().cpu()
        K = kvd[pg, 0].permute(1, 0, 2, 3).reshape(n_kv, nb * page, d)[:, :S]
        V = kvd[pg, 1].permute(1, 0, 2, 3).reshape(n_kv, nb * page, d)[:, :S]
        for h in range(n_q):
            s = (qd[a:b, h] @ K[h // G].T) * scale
            pos = torch.arange(S - T, S)[:, None]
            key = torch.arange(S)[None, :]
            ok = key <= pos
            if window:
                ok &= key > pos - window
            s = s.masked_fill(~ok, float("-inf"))
            out[a:b, h] = torch.softmax(s, -1) @ V[h // G]
    return out


CASES = [  # lens, q_lens, n_q, n_kv, d, page, window
    ([70, 5, 130], [70, 5, 17], 4, 2, 16, 4, 0),
    ([300, 64, 65, 1], [3, 64, 1, 1], 7, 1, 48, 5, 0),
    ([200, 129], [200, 100], 6, 3, 128, 16, 0),
    ([500, 77, 300], [30, 77, 1], 8, 2, 64, 16, 37),
    ([90], [90], 5, 5, 32, 8, 64),
    ([257, 31], [2, 31], 40, 2, 16, 32, 0),  # a group of 20 heads
]


@pytest.mark.parametrize("case", range(len(CASES)))
@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_tiled_kernels(dtype, case):
    lens, q_lens, n_q, n_kv, d, page, window = CASES[case]
    q, kv, table, q_start, seq_lens = make_attention_case(dtype, lens, q_lens, n_q, n_kv, d, page, seed=case)
    scale = d ** -0.5
    ref = attention_reference(q, kv, table, q_start, seq_lens, n_kv, page, scale, window)
    from slipstream_b200.engine.context import query_tiles_host
    ql = np.asarray(q_lens, dtype=np.int32)
    out = torch.full((q.shape[0], n_q * d), float("nan"), device=DEV, dtype=dtype)
    req, q0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(ql, 16))
    ops().paged_attention_simt(q.view(q.shape[0], -1), n_q * d, out, kv, table, req, q0, q_start, seq_lens,
                               n_q, n_kv, d, scale, window)
    assert rel_err(out.view_as(ref).cpu(), ref) < tol(dtype, 3e-6, 1e-2)
    if dtype == torch.bfloat16:
        out2 = torch.full_like(out, float("nan"))
        req, r0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(ql * (n_q // n_kv), 64))
        ops().paged_attention_prefill(q.view(q.shape[0], -1), n_q * d, out2, kv, table, req, r0, q_start, seq_lens,
                                      n_q, n_kv, d, scale, window)
        assert rel_err(out2.view_as(ref).cpu(), ref) < 1e-2
    ops().check_errors(torch.device(DEV))


@pytest.mark.parametrize("slices", [1, 2, 5, 16, 32, 64])  # one cluster; 2, 4, 8 clusters of 8 (TMA-fed kernel) or single blocks
@pytest.mark.parametrize("n_q, n_kv, d, page, window", [(28, 4, 128, 16, 0), (6, 6, 16, 4, 0), (40, 2, 64, 7, 0),
                                                         (8, 2, 32, 16, 100), (3, 1, 256, 16, 0), (40, 2, 64, 8, 0),
                                                         (9, 3, 128, 64, 150), (4, 4, 64, 32, 33)])
def test_split_decode_attention(slices, n_q, n_kv, d, page, window):
    lens = [1, 63, 64, 65, 700, 129, 2000]
    q, kv, table, q_start, seq_lens = make_attention_case(torch.bfloat16, lens, [1] * len(lens), n_q, n_kv, d, page, seed=d)
    scale = d ** -0.5
    ref = attention_reference(q, kv, table, q_start, seq_lens, n_kv, page, scale, window)
    # tiles moved by cp.async, and by TMA where the sizes allow it, through a ring of two stages and of three
    kernels = [(False, 2)] + ([(True, 2), (True, 3)] if ops().tcgen05_attention_fits(d, n_q, n_kv, page, 0) else [])
    for tma, stages in kernels:
        out = torch.full((q.shape[0], n_q * d), float("nan"), device=DEV, dtype=torch.bfloat16)
        ops().paged_attention_decode(q.view(q.shape[0], -1), n_q * d, out, kv, table, q_start, seq_lens, len(lens),
                                     n_q, n_kv, d, scale, window, n_slices=slices, tma=tma, stages=stages)
        assert rel_err(out.view_as(ref).cpu(), ref) < 1e-2, (tma, stages)
    ops().check_errors(torch.device(DEV))


@pytest.mark.parametrize("slices", [1, 3, 8, 11, 24])
@pytest.mark.parametrize("n_q, n_kv, d, rot, page, window", [(28, 4, 128, 128, 16, 0), (6, 6, 16, 8, 4, 0),
                                                              (40, 2, 64, 64, 7, 0), (8, 2, 32, 0, 16, 100),
                                                              (40, 2, 64, 32, 8, 0), (9, 3, 128, 128, 64, 150)])
def test_decode_attention_that_rotates_and_writes_the_newest_token_itself(slices, n_q, n_kv, d, rot, page, window):
    """The decode kernel given the projection output as it is (rope=...) must leave the same pages and the
    same output, bit for bit, as the rotary kernel followed by the decode kernel."""
    lens = [1, 63, 64, 65, 700, 129, 2000, 16, 17]
    R = len(lens)
    _, kv, table, q_start, seq_lens = make_attention_case(torch.bfloat16, lens, [1] * R, n_q, n_kv, d, page, seed=d + 1)
    g = torch.Generator().manual_seed(5)
    qkv = (torch.randn(R, (n_q + 2 * n_kv) * d, generator=g) * 0.7).bfloat16().to(DEV)
    inv_freq = (1.0 / 10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / max(rot, 1))).to(DEV) if rot else None
    positions = (seq_lens - 1).int()
    pages_of = table.long()[torch.arange(R, device=DEV), (positions // page).long()]
    slots = (pages_of * page + positions % page).int()
    scale = d ** -0.5
    for tma, stages in [(False, 2)] + ([(True, 2), (True, 3)] if ops().tcgen05_attention_fits(d, n_q, n_kv, page, 0) else []):
        # two steps, then one step, with the same way of moving the tiles (cp.async, or TMA with a ring of 2 or 3)
        qkv_a, kv_a = qkv.clone(), kv.clone()
        ops().rope_and_cache(qkv_a, positions, slots, inv_freq, kv_a, n_q, n_kv, d, rot)
        out_a = torch.full((R, n_q * d), float("nan"), device=DEV, dtype=torch.bfloat16)
        ops().paged_attention_decode(qkv_a, qkv_a.shape[1], out_a, kv_a, table, q_start, seq_lens, R, n_q, n_kv, d, scale,
                                     window, n_slices=slices, tma=tma, stages=stages)
        qkv_b, kv_b = qkv.clone(), kv.clone()
        out_b = torch.full_like(out_a, float("nan"))
        ops().paged_attention_decode(qkv_b, qkv_b.shape[1], out_b, kv_b, table, q_start, seq_lens, R, n_q, n_kv, d,
                                     scale, window, n_slices=slices, rope=(inv_freq, rot), tma=tma, stages=stages)
        assert torch.equal(kv_a, kv_b), "the pages differ"
        assert not torch.equal(kv_b, kv) and torch.equal(qkv_b, qkv)
        assert torch.equal(out_a, out_b), (tma, stages)
    ops().check_errors(torch.device(DEV))


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_among_hundreds_is_found(dtype):
    """One key 700 tokens back matches the last query far better than all others: its value must
    dominate the output, through every kernel."""
    n_q, n_kv, d, page = 4, 2, 64, 16
    for q_len in (1, 40):
        q, kv, table, q_start, seq_lens = make_attention_case(dtype, [900, 50], [q_len, 3], n_q, n_kv, d, page, seed=1, sharp=197)
        ref = attention_reference(q, kv, table, q_start, seq_lens, n_kv, page, 1.0, 0)
        row = q_len - 1
        assert ref[row].min() > 4.9  # the oracle itself sees the far key
        from slipstream_b200.engine.context import query_tiles_host
        ql = np.asarray([q_len, 3], dtype=np.int32)
        out = torch.zeros((q.shape[0], n_q * d), device=DEV, dtype=dtype)
        req, q0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(ql, 16))
        ops().paged_attention_simt(q.view(q.shape[0], -1), n_q * d, out, kv, table, req, q0, q_start, seq_lens, n_q, n_kv, d, 1.0, 0)
        assert out[row].float().min() > 4.9 and rel_err(out.view_as(ref).cpu(), ref) < tol(dtype, 3e-6, 1e-2)
        if dtype == torch.bfloat16:
            out.zero_()
            req, r0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(ql * 2, 64))
            ops().paged_attention_prefill(q.view(q.shape[0], -1), n_q * d, out, kv, table, req, r0, q_start, seq_lens, n_q, n_kv, d, 1.0, 0)
            assert out[row].float().min() > 4.9 and rel_err(out.view_as(ref).cpu(), ref) < 1e-2


# --------------------------------------------------------------------------- sampling

def test_argmax_lowest_index_wins_ties():
    logits = torch.randn(9, 152064, device=DEV)
    logits[2, 777] = logits[2, 70000] = 50.0
    logits[5] = 0.0
    got = ops().argmax(logits).cpu()
    want = logits.argmax(-1).cpu()
    assert got[2] == 777 and got[5] == 0
    assert all(int(got[i]) == int(want[i]) for i in (0, 1, 3, 4, 6, 7, 8))


# --------------------------------------------------------------------------- tcgen05 matrix product

@pytest.mark.parametrize("tokens, features, k", [(1, 128, 64), (8, 3584, 3584), (8, 200, 136), (13, 4608, 3584), (33, 1000, 512),
                                                 (64, 263, 80), (8, 3584, 18944), (65, 256, 64), (300, 520, 200), (2048, 4608, 3584),
                                                 (129, 100, 72)])
def test_tcgen05_matrix_product(tokens, features, k):
    torch.manual_seed(tokens + features)
    x = torch.randn(tokens, k, device=DEV).bfloat16()
    w = (torch.randn(features, k, device=DEV) * 0.05).bfloat16()
    b = torch.randn(features, device=DEV).bfloat16()
    ref = x.double() @ w.double().T
    got = ops().gemm_tcgen05(x, w, None, torch.float32)
    assert rel_err(got, ref) < 2e-5, "float32 output of bfloat16 inputs is exact up to the order of additions"
    got = ops().gemm_tcgen05(x, w, b)
    assert got.dtype == torch.bfloat16 and rel_err(got, ref + b.double()) < 6e-3
    got = ops().gemm_tcgen05(x, w, b.float(), torch.float32)
    assert rel_err(got, ref + b.double()) < 2e-5
    ops().check_errors(torch.device(DEV))


@pytest.mark.parametrize("tokens, features, k", [(2048, 4608, 3584), (300, 200, 136), (129, 1024, 64), (1000, 520, 2048)])
def test_tcgen05_persistent_product_for_many_tokens(tokens, features, k):
    torch.manual_seed(tokens)
    x = torch.randn(tokens, k, device=DEV).bfloat16()
    w = (torch.randn(features, k, device=DEV) * 0.05).bfloat16()
    b = torch.randn(features, device=DEV).bfloat16()
    ref = x.double() @ w.double().T
    got = ops().gemm_tcgen05_many(x, w, None, torch.float32)
    assert rel_err(got, ref) < 2e-5, "float32 output of bfloat16 inputs is exact up to the order of additions"
    assert rel_err(ops().gemm_tcgen05_many(x, w, b), ref + b.double()) < 6e-3
    assert rel_err(ops().gemm_tcgen05_many(x, w, b.float(), torch.float32), ref + b.double()) < 2e-5
    ops().check_errors(torch.device(DEV))


@pytest.mark.parametrize("tokens, features, k", [(2048, 3584, 3584), (600, 1000, 264)])
def test_tcgen05_two_sm_product_at_every_tile_width(tokens, features, k):
    """The pairs of SMs compute tiles of 256 rows and any multiple of 16 columns; the launcher picks the width
    whose tiles fill whole rounds of the pairs (208 for 2,048 x 3,584 outputs), and every width gives the same."""
    torch.manual_seed(features)
    x = torch.randn(tokens, k, device=DEV).bfloat16()
    w = (torch.randn(features, k, device=DEV) * 0.05).bfloat16()
    b = torch.randn(features, device=DEV).bfloat16()
    ref = x.double() @ w.double().T + b.double()
    for cols in (0, 16, 48, 64, 112, 208, 240, 256):
        got = ops().gemm_tcgen05_many(x, w, b, torch.float32, tile_cols=cols)
        assert rel_err(got, ref) < 2e-5, cols
    for cols in (8, 24, 272):
        with pytest.raises(ops().KernelError):
            ops().gemm_tcgen05_many(x, w, b, torch.float32, tile_cols=cols)
    ops().check_errors(torch.device(DEV))


@pytest.mark.parametrize("tokens, inter, k, bias", [(2048, 18944, 3584, False), (70, 192, 136, True), (513, 640, 200, True)])
def test_tcgen05_persistent_product_with_swiglu(tokens, inter, k, bias):
    torch.manual_seed(inter)
    x = torch.randn(tokens, k, device=DEV).bfloat16()
    gate, up = ((torch.randn(inter, k, device=DEV) * 0.05).bfloat16() for _ in range(2))
    bg, bu = ((torch.randn(inter, device=DEV) * 0.5).bfloat16() for _ in range(2))
    mix = lambda a, b: torch.stack([a.reshape(inter // 64, 64, *a.shape[1:]), b.reshape(inter // 64, 64, *b.shape[1:])], 1).reshape(2 * inter, *a.shape[1:]).contiguous()
    g = x.double() @ gate.double().T + (bg.double() if bias else 0)
    u = x.double() @ up.double().T + (bu.double() if bias else 0)
    got = ops().gemm_tcgen05_many(x, mix(gate, up), mix(bg, bu) if bias else None, swiglu=True)
    assert got.shape == (tokens, inter) and rel_err(got, g * torch.sigmoid(g) * u) < 8e-3
    ops().check_errors(torch.device(DEV))


def test_tcgen05_split_k_is_deterministic_and_leaves_its_counters_clean():
    x = torch.randn(8, 18944, device=DEV).bfloat16()
    w = (torch.randn(3584, 18944, device=DEV) * 0.02).bfloat16()
    assert ops().gemm_plan(8, 3584, 18944)[2] > 1
    a = ops().gemm_tcgen05(x, w, None, torch.float32)
    for _ in range(3):
        assert torch.equal(ops().gemm_tcgen05(x, w, None, torch.float32), a)
    for slices in (1, 2, 7, 12):  # 2..8: added through a cluster; more: through scratch memory
        got = ops().gemm_tcgen05(x, w, None, torch.float32, plan=(True, 16, slices))
        assert rel_err(got, a) < 1e-4  # 18,944 float32 additions in another order
    ops().check_errors(torch.device(DEV))


@pytest.mark.parametrize("tokens, inter, k, bias", [(1, 64, 64, False), (8, 18944, 3584, False), (33, 192, 136, True), (64, 640, 200, True)])
def test_tcgen05_fused_swiglu(tokens, inter, k, bias):
    """Weight rows alternate 64 gate and 64 up features; the epilogue gives silu(gate) * up."""
    torch.manual_seed(inter)
    x = torch.randn(tokens, k, device=DEV).bfloat16()
    gate, up = ((torch.randn(inter, k, device=DEV) * 0.05).bfloat16() for _ in range(2))
    bg, bu = ((torch.randn(inter, device=DEV) * 0.5).bfloat16() for _ in range(2))
    mix = lambda a, b: torch.stack([a.reshape(inter // 64, 64, *a.shape[1:]), b.reshape(inter // 64, 64, *b.shape[1:])], 1).reshape(2 * inter, *a.shape[1:]).contiguous()
    g = x.double() @ gate.double().T + (bg.double() if bias else 0)
    u = x.double() @ up.double().T + (bu.double() if bias else 0)
    ref = g * torch.sigmoid(g) * u
    for plan in (None, (True, 16 if tokens <= 16 else 64, 1), (True, 64, 3)):
        got = ops().gemm_tcgen05(x, mix(gate, up), mix(bg, bu) if bias else None, swiglu=True, plan=plan)
        assert got.shape == (tokens, inter) and rel_err(got, ref) < 8e-3, plan
    got = ops().gate_up_swiglu(x, mix(gate, up), mix(bg, bu) if bias else None, 64)
    assert rel_err(got, ref) < 8e-3
    ops().check_errors(torch.device(DEV))


@pytest.mark.parametrize("tokens, features, k, bias, w_f32", [(8, 3584, 3584, False, False), (1, 3584, 18944, False, False),
                                                             (16, 896, 4864, True, True), (5, 256, 136, True, False),
                                                             (3, 1024, 512, False, True), (11, 5120, 13824, False, False),
                                                             (2, 3584, 3584, False, False)])
def test_projection_into_the_stream_and_the_norm_finished_by_the_next_product(tokens, features, k, bias, w_f32):
    """`linear_add_rmsnorm` with few bfloat16 tokens: the projection adds its output to the float32 stream in its
    epilogue and leaves round(norm weight * stream) and the sums of squares; the norm comes back pending, and the
    next product runs on that matrix and scales every token's output at the end.  Against float64 arithmetic with
    the same roundings (the branch output to bfloat16 before the add, weight * stream to bfloat16), against the
    exact norm, and against the kernels it replaces (the same stream bit for bit)."""
    torch.manual_seed(features + tokens)
    assert ops().adds_to_stream(tokens, features, k)
    x = torch.randn(tokens, k, device=DEV).bfloat16()
    w = (torch.randn(features, k, device=DEV) * 0.05).bfloat16()
    b = torch.randn(features, device=DEV).bfloat16() if bias else None
    nw = 1 + 0.1 * torch.randn(features, device=DEV)
    nw = nw if w_f32 else nw.bfloat16()
    stream0 = torch.randn(tokens, features, device=DEV) * 3
    stream0[0] *= 30  # rows of different size: each needs its own scale
    eps = 1e-5
    delta = (x.double() @ w.double().T + (b.double() if bias else 0)).bfloat16().double()
    stream_ref = (stream0.double() + delta).float()
    launches = ops().launch_count()
    stream = stream0.clone()
    got = ops().linear_add_rmsnorm(x, w, b, stream, nw, eps, torch.bfloat16)
    assert ops().launch_count() == launches + 1 and isinstance(got, ops().PendingNorm) and got.shape == stream.shape
    # the branch output may round the other way where the float32 sum lies at a tie: a step of its bfloat16
    assert rel_err(stream, stream_ref) < 3e-3 and (stream - stream_ref).abs().max() <= 2 ** -6 * delta.abs().max()
    assert torch.allclose(got.squares.double().sum(1), stream.double().pow(2).sum(1), rtol=1e-5)
    assert torch.equal(got.scaled, (nw.float() * stream).bfloat16())
    rstd = torch.rsqrt(stream.double().pow(2).mean(-1, keepdim=True) + eps)
    exact = nw.double() * stream.double() * rstd               # the norm without any rounding
    ops().set_norm_fusion(False)
    try:
        stream2 = stream0.clone()
        two = ops().linear_add_rmsnorm(x, w, b, stream2, nw, eps, torch.bfloat16)
        assert ops().launch_count() == launches + 3 and isinstance(two, torch.Tensor)
    finally:
        ops().set_norm_fusion(True)
    assert torch.equal(stream, stream2)
    assert rel_err(two, exact) < 1e-2
    # the products behind the norm: a projection with bias, and gate/up with SwiGLU, each from the pending norm
    # (37,888 and 19,072 weight rows: a tile per SM and more, every block walks all K steps alone and stores its tile
    # itself; the others: K slices in a cluster)
    for features2, swiglu in ((328, False), (4608, False), (19072, False), (1024, True), (37888, True)):
        assert ops().takes_pending_norm(got, features2)
        if features2 > 5000 and tokens not in (1, 2, 8):
            continue
        w2 = (torch.randn(features2, features, device=DEV) * 0.05).bfloat16()
        b2 = torch.randn(features2, device=DEV).bfloat16()
        launches = ops().launch_count()
        same_roundings = (got.scaled.double() @ w2.double().T) * rstd + b2.double()
        unrounded = exact @ w2.double().T + b2.double()
        if swiglu:
            inside, after = ops().gate_up_swiglu(got, w2, b2, 64), ops().gate_up_swiglu(two, w2, b2, 64)

            def act(y):
                g, u = (y.view(tokens, -1, 2, 64)[:, :, i].reshape(tokens, -1) for i in (0, 1))
                return g * torch.sigmoid(g) * u
            same_roundings, unrounded = act(same_roundings), act(unrounded)
        else:
            inside, after = ops().linear(got, w2, b2), ops().linear(two, w2, b2)
        assert ops().launch_count() == launches + 2, "one launch each: no norm kernel"
        assert rel_err(inside, same_roundings) < 6e-3, (features2, swiglu)
        # one rounding of the activations instead of two: no further from the exact result than the norm kernel's way
        assert rel_err(inside, unrounded) <= max(rel_err(after, unrounded) * 1.2, 6e-3), (features2, swiglu)
        assert torch.equal(inside, ops().gate_up_swiglu(got, w2, b2, 64) if swiglu else ops().linear(got, w2, b2))
    # float32 logits behind a final norm: every block stores its tile itself
    head = (torch.randn(19200, features, device=DEV) * 0.05).bfloat16()
    logits = ops().linear(got, head, None, out_dtype=torch.float32)
    assert logits.dtype == torch.float32 and rel_err(logits, (got.scaled.double() @ head.double().T) * rstd) < 1e-4
    # a product that does not stream its weights, or a part that wants a tensor, gets the norm kernel's result
    assert rel_err(got.materialize(), exact) < 1e-2
    wide = (torch.randn(72, features, device=DEV) * 0.05).float()
    as_f32 = ops().PendingNorm(got.stream, got.scaled, got.squares, nw.float(), eps, torch.float32)
    assert rel_err(ops().linear(as_f32, wide), (nw.double() * stream.double() * rstd) @ wide.double().T) < 1e-4
    ops().check_errors(torch.device(DEV))


@pytest.mark.parametrize("tokens, features, k, bias, w_f32", [(2048, 3584, 3584, False, False), (2300, 3600, 2048, True, True),
                                                             (2048, 3584, 18944, False, False)])
def test_long_prompt_portions_take_the_same_way_through_the_two_sm_kernel(tokens, features, k, bias, w_f32):
    """`linear_add_rmsnorm` from 2,048 tokens: the persistent two-SM kernel adds its tiles to the stream (a row per
    thread of its epilogue), and the products behind the norm scale their rows.  Same checks as for decode steps."""
    torch.manual_seed(features + tokens)
    assert not ops().adds_to_stream(tokens, features, k), "off unless asked for (it did not pay when measured)"
    ops().set_norm_fusion(True, long_portions=True)
    try:
        check_long_portion(tokens, features, k, bias, w_f32)
    finally:
        ops().set_norm_fusion(True)


def check_long_portion(tokens, features, k, bias, w_f32):
    assert ops().adds_to_stream(tokens, features, k)
    x = torch.randn(tokens, k, device=DEV).bfloat16()
    w = (torch.randn(features, k, device=DEV) * 0.05).bfloat16()
    b = torch.randn(features, device=DEV).bfloat16() if bias else None
    nw = 1 + 0.1 * torch.randn(features, device=DEV)
    nw = nw if w_f32 else nw.bfloat16()
    stream0 = torch.randn(tokens, features, device=DEV) * 3
    stream0[::7] *= 30
    eps = 1e-6
    delta = (x.double() @ w.double().T + (b.double() if bias else 0)).bfloat16().double()
    stream_ref = (stream0.double() + delta).float()
    launches = ops().launch_count()
    stream = stream0.clone()
    got = ops().linear_add_rmsnorm(x, w, b, stream, nw, eps, torch.bfloat16)
    assert ops().launch_count() == launches + 1 and isinstance(got, ops().PendingNorm)
    assert rel_err(stream, stream_ref) < 3e-3 and (stream - stream_ref).abs().max() <= 2 ** -6 * delta.abs().max()
    assert torch.allclose(got.squares.double().sum(1), stream.double().pow(2).sum(1), rtol=1e-5)
    assert torch.equal(got.scaled, (nw.float() * stream).bfloat16())
    rstd = torch.rsqrt(stream.double().pow(2).mean(-1, keepdim=True) + eps)
    exact = nw.double() * stream.double() * rstd
    ops().set_norm_fusion(False)
    try:
        stream2 = stream0.clone()
        two = ops().linear_add_rmsnorm(x, w, b, stream2, nw, eps, torch.bfloat16)
        assert isinstance(two, torch.Tensor)
    finally:
        ops().set_norm_fusion(True, long_portions=True)
    assert torch.equal(stream, stream2)
    for features2, swiglu in ((4608, False), (37888, True)):
        if swiglu and k > 4000:
            continue
        assert ops().takes_pending_norm(got, features2, swiglu=swiglu)
        w2 = (torch.randn(features2, features, device=DEV) * 0.05).bfloat16()
        b2 = torch.randn(features2, device=DEV).bfloat16()
        same_roundings = (got.scaled.double() @ w2.double().T) * rstd + b2.double()
        unrounded = exact @ w2.double().T + b2.double()
        launches = ops().launch_count()
        if swiglu:
            inside, after = ops().gate_up_swiglu(got, w2, b2, 64), ops().gate_up_swiglu(two, w2, b2, 64)

            def act(y):
                g, u = (y.view(tokens, -1, 2, 64)[:, :, i].reshape(tokens, -1) for i in (0, 1))
                return g * torch.sigmoid(g) * u
            same_roundings, unrounded = act(same_roundings), act(unrounded)
        else:
            inside, after = ops().linear(got, w2, b2), ops().linear(two, w2, b2)
        assert ops().launch_count() == launches + 2, "one launch each: no norm kernel"
        assert rel_err(inside, same_roundings) < 6e-3, (features2, swiglu)
        assert rel_err(inside, unrounded) <= max(rel_err(after, unrounded) * 1.2, 6e-3), (features2, swiglu)
        del w2, same_roundings, unrounded
    ops().check_errors(torch.device(DEV))


def test_the_add_and_norm_stay_two_launches_where_the_product_is_not_a_cluster():
    """float32, many tokens, a width that is no multiple of 128: `linear` then `add_rmsnorm`, same result."""
    for dtype, tokens, features, k in ((torch.float32, 4, 128, 64), (torch.bfloat16, 40, 256, 128), (torch.bfloat16, 4, 200, 64)):
        torch.manual_seed(tokens)
        assert dtype == torch.float32 or not ops().adds_to_stream(tokens, features, k)
        x = torch.randn(tokens, k, device=DEV).to(dtype)
        w = (torch.randn(features, k, device=DEV) * 0.1).to(dtype)
        nw = (1 + 0.1 * torch.randn(features, device=DEV)).to(dtype)
        stream = torch.randn(tokens, features, device=DEV)
        want_stream = stream.clone()
        want = ops().add_rmsnorm(want_stream, ops().linear(x, w), nw, 1e-6, dtype)
        got = ops().linear_add_rmsnorm(x, w, None, stream, nw, 1e-6, dtype)
        assert torch.equal(got, want) and torch.equal(stream, want_stream)


TC5_CASES = [  # lens, q_lens, n_q, n_kv, d, page
    ([200, 129], [200, 100], 6, 3, 128, 16),
    ([300, 64, 65, 1, 130], [3, 64, 1, 1, 130], 28, 4, 128, 16),   # groups of 7: 18 tokens per tile
    ([500, 77], [400, 77], 4, 4, 64, 8),                           # one head per group: 128 tokens per tile
    ([257, 31, 700], [2, 31, 300], 40, 2, 64, 32),                 # groups of 20
    ([1000], [1000], 8, 1, 128, 64),
]


@pytest.mark.parametrize("case", range(len(TC5_CASES)))
def test_tcgen05_prefill_attention(case):
    lens, q_lens, n_q, n_kv, d, page = TC5_CASES[case]
    q, kv, table, q_start, seq_lens = make_attention_case(torch.bfloat16, lens, q_lens, n_q, n_kv, d, page, seed=50 + case)
    scale = d ** -0.5
    ref = attention_reference(q, kv, table, q_start, seq_lens, n_kv, page, scale, 0)
    from slipstream_b200.engine.context import query_tiles_host
    tok = 128 // (n_q // n_kv)
    req, t0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(np.asarray(q_lens, dtype=np.int32), tok))
    for parts in (1, 2, 4, 8):  # blocks of a cluster that share the keys of a query tile (some get none of them)
        out = torch.full((q.shape[0], n_q * d), float("nan"), device=DEV, dtype=torch.bfloat16)
        ops().paged_attention_prefill_tcgen05(q.view(q.shape[0], -1), n_q * d, out, kv, table, req, t0, q_start, seq_lens,
                                              n_q, n_kv, d, scale, parts)
        assert rel_err(out.view_as(ref).cpu(), ref) < 1e-2, parts
    ops().check_errors(torch.device(DEV))


def test_tcgen05_prefill_attention_with_growing_maxima():
    """Keys grow with their position, so every row's running maximum moves by far more than the
    threshold of the lazy rescaling, in different tiles for different rows of a warp."""
    n_q, n_kv, d, page, n = 28, 4, 128, 16, 700
    q, kv, table, q_start, seq_lens = make_attention_case(torch.bfloat16, [n], [n], n_q, n_kv, d, page, seed=77)
    kvf = kv.float()
    for p in range(n):
        kvf[table[0, p // page].long(), 0, :, p % page] *= 1.0 + 0.02 * p * ((p * 7919) % 5 == 0)
    kv = kvf.bfloat16()
    scale = 1.0
    ref = attention_reference(q, kv, table, q_start, seq_lens, n_kv, page, scale, 0)
    from slipstream_b200.engine.context import query_tiles_host
    req, t0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(np.asarray([n], dtype=np.int32), 128 // 7))
    for parts in (1, 4):
        out = torch.full((n, n_q * d), float("nan"), device=DEV, dtype=torch.bfloat16)
        ops().paged_attention_prefill_tcgen05(q.view(n, -1), n_q * d, out, kv, table, req, t0, q_start, seq_lens, n_q, n_kv, d, scale, parts)
        assert rel_err(out.view_as(ref).cpu(), ref) < 1e-2, parts
    ops().check_errors(torch.device(DEV))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sharp", [15, 16, 63, 64, 127, 128, 191, 899])
def test_a_standout_key_at_a_page_or_tile_edge(dtype, sharp):
    """The one key that matters sits on the last slot of a page, the first slot of the next, the edge of a
    64-key tile, or is the newest key: every kernel must find it there."""
    n_q, n_kv, d, page = 4, 2, 64, 16
    from slipstream_b200.engine.context import query_tiles_host
    for q_len in (1, 5):
        q, kv, table, q_start, seq_lens = make_attention_case(dtype, [900, 50], [q_len, 3], n_q, n_kv, d, page, seed=sharp, sharp=sharp)
        ref = attention_reference(q, kv, table, q_start, seq_lens, n_kv, page, 1.0, 0)
        row = q_len - 1
        assert ref[row].min() > 4.9
        ql = np.asarray([q_len, 3], dtype=np.int32)
        outs = {}
        out = torch.zeros((q.shape[0], n_q * d), device=DEV, dtype=dtype)
        req, q0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(ql, 16))
        ops().paged_attention_simt(q.view(q.shape[0], -1), n_q * d, out, kv, table, req, q0, q_start, seq_lens, n_q, n_kv, d, 1.0, 0)
        outs["simt"] = out
        if dtype == torch.bfloat16:
            out = torch.zeros_like(out)
            req, r0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(ql * 2, 64))
            ops().paged_attention_prefill(q.view(q.shape[0], -1), n_q * d, out, kv, table, req, r0, q_start, seq_lens, n_q, n_kv, d, 1.0, 0)
            outs["mma"] = out
            out = torch.zeros_like(out)
            req, t0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(ql, 64))
            ops().paged_attention_prefill_tcgen05(q.view(q.shape[0], -1), n_q * d, out, kv, table, req, t0, q_start, seq_lens, n_q, n_kv, d, 1.0)
            outs["tcgen05"] = out
            out = torch.zeros_like(out)
            ops().paged_attention_prefill_tcgen05(q.view(q.shape[0], -1), n_q * d, out, kv, table, req, t0, q_start, seq_lens, n_q, n_kv, d, 1.0, 8)
            outs["tcgen05, keys in 8 parts"] = out
        for name, o in outs.items():
            assert o[row].float().min() > 4.9, (name, q_len)
            assert rel_err(o.view_as(ref).cpu(), ref) < tol(dtype, 3e-6, 1e-2), (name, q_len)
    if dtype == torch.bfloat16:  # and through the split decode kernel
        q, kv, table, q_start, seq_lens = make_attention_case(dtype, [900, 50], [1, 1], n_q, n_kv, d, page, seed=sharp, sharp=sharp)
        ref = attention_reference(q, kv, table, q_start, seq_lens, n_kv, page, 1.0, 0)
        for slices in (1, 4):
            out = torch.zeros((2, n_q * d), device=DEV, dtype=dtype)
            ops().paged_attention_decode(q.view(2, -1), n_q * d, out, kv, table, q_start, seq_lens, 2, n_q, n_kv, d, 1.0, 0, n_slices=slices)
            assert out[0].float().min() > 4.9 and rel_err(out.view_as(ref).cpu(), ref) < 1e-2


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_edge_of_a_window(dtype):
    """With a window of W keys, the key W back is invisible and the key W - 1 back is visible: put the
    standout key on either side of the edge."""
    n_q, n_kv, d, page, window, n = 2, 1, 32, 8, 40, 300
    from slipstream_b200.engine.context import query_tiles_host
    for back, seen in ((window - 1, True), (window, False)):
        sharp = n - 1 - back
        q, kv, table, q_start, seq_lens = make_attention_case(dtype, [n, 20], [1, 2], n_q, n_kv, d, page, seed=3, sharp=sharp)
        ref = attention_reference(q, kv, table, q_start, seq_lens, n_kv, page, 1.0, window)
        assert (ref[0].min() > 4.9) == seen
        ql = np.asarray([1, 2], dtype=np.int32)
        out = torch.zeros((3, n_q * d), device=DEV, dtype=dtype)
        req, q0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(ql, 16))
        ops().paged_attention_simt(q.view(3, -1), n_q * d, out, kv, table, req, q0, q_start, seq_lens, n_q, n_kv, d, 1.0, window)
        assert (out[0].float().min() > 4.9) == seen and rel_err(out.view_as(ref).cpu(), ref) < tol(dtype, 3e-6, 1e-2)
        if dtype == torch.bfloat16:
            out.zero_()
            req, r0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(ql * 2, 64))
            ops().paged_attention_prefill(q.view(3, -1), n_q * d, out, kv, table, req, r0, q_start, seq_lens, n_q, n_kv, d, 1.0, window)
            assert (out[0].float().min() > 4.9) == seen and rel_err(out.view_as(ref).cpu(), ref) < 1e-2


@pytest.mark.parametrize("n_q, n_kv, d, page", [(28, 4, 128, 16), (6, 2, 64, 32), (4, 2, 32, 8)])
def test_what_a_pages_last_owner_left_behind_reaches_nobody(n_q, n_kv, d, page):
    """Pages are not cleared when they change hands: behind a request's newest token its last page still holds the
    keys and values of whoever had it before, here infinities and NaN.  Their scores are masked, and their values
    must not get into the result either (0 x inf): every attention kernel gives what it gives with clean pages."""
    from slipstream_b200.engine.context import query_tiles_host
    lens, q_lens = [70, 5, 130, 33, 1], [70, 5, 17, 1, 1]
    q, kv, table, q_start, seq_lens = make_attention_case(torch.bfloat16, lens, q_lens, n_q, n_kv, d, page, seed=3)
    scale = d ** -0.5
    ref = attention_reference(q, kv, table, q_start, seq_lens, n_kv, page, scale, 0)
    dirty = kv.clone()
    for r, n in enumerate(lens):
        if n % page:
            last = int(table[r, (n - 1) // page])
            dirty[last, :, :, n % page:] = float("inf")
            dirty[last, 1, :, n % page:, ::2] = float("nan")
    qf = q.view(q.shape[0], -1)
    ql = np.asarray(q_lens, dtype=np.int32)

    def check(out, what):
        assert torch.isfinite(out).all(), what
        assert rel_err(out.view_as(ref).cpu(), ref) < 1e-2, what

    out = torch.full((q.shape[0], n_q * d), float("nan"), device=DEV, dtype=torch.bfloat16)
    req, q0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(ql, 16))
    ops().paged_attention_simt(qf, n_q * d, out, dirty, table, req, q0, q_start, seq_lens, n_q, n_kv, d, scale, 0)
    check(out, "simt")
    out.fill_(float("nan"))
    req, r0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(ql * (n_q // n_kv), 64))
    ops().paged_attention_prefill(qf, n_q * d, out, dirty, table, req, r0, q_start, seq_lens, n_q, n_kv, d, scale, 0)
    check(out, "mma.sync prefill")
    if ops().tcgen05_attention_fits(d, n_q, n_kv, page, 0):
        req, t0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(ql, 128 // (n_q // n_kv)))
        for parts in (1, 2):
            out.fill_(float("nan"))
            ops().paged_attention_prefill_tcgen05(qf, n_q * d, out, dirty, table, req, t0, q_start, seq_lens, n_q, n_kv, d,
                                                  scale, parts)
            check(out, f"tcgen05 prefill, {parts} parts")
    # decode: every request brings its last token only
    last_rows = (q_start[1:] - 1).long()
    qd = qf[last_rows].contiguous()
    refd = ref.view(q.shape[0], -1)[last_rows.cpu()]
    starts = torch.arange(len(lens) + 1, dtype=torch.int32, device=DEV)
    for tma in [False] + ([True] if ops().tcgen05_attention_fits(d, n_q, n_kv, page, 0) else []):
        for slices in (1, 2, 8):
            outd = torch.full((len(lens), n_q * d), float("nan"), device=DEV, dtype=torch.bfloat16)
            ops().paged_attention_decode(qd, n_q * d, outd, dirty, table, starts, seq_lens, len(lens), n_q, n_kv, d, scale, 0,
                                         n_slices=slices, tma=tma)
            assert torch.isfinite(outd).all(), (tma, slices)
            assert rel_err(outd.cpu(), refd) < 1e-2, (tma, slices)
    ops().check_errors(torch.device(DEV))
