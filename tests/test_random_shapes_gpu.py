"""Many shapes and schedules drawn at random, each judged like the fixed cases of the other test files: the
attention kernels and the matrix products against float64 arithmetic, the sampling kernel against the plain
chain with the same noise, and the engine under tight page pools and small budgets against the same engine
with room.  The draws are seeded: a failure names its trial, which reproduces it."""
import random

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from conftest import random_tokens
from test_generate_gpu import gumbel_noise, make_engine, run_sample
from test_kernels_gpu import attention_reference, make_attention_case, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
EDGES = [1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 191, 192, 193, 255, 256, 257]


def ops():
    from slipstream_b200 import ops as o
    return o


def test_attention_kernels_at_random_sizes_with_stale_rows_behind_every_request():
    """Head sizes in steps of 16, groups of 1 to 16 heads, pages of 4 to 64 tokens (sizes that do not divide a
    tile among them), windows, requests that end on and beside the edges of pages and tiles, prompt portions
    and single tokens, keys in 1 to 8 parts and 1 to 64 slices; the rows of a request's last page behind its end
    hold Inf or NaN."""
    from slipstream_b200.engine.context import query_tiles_host
    for trial in range(250):
        rng = random.Random(trial)
        d = rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128, 128, 128, 160, 192, 256])
        n_kv, g = rng.choice([1, 2, 3, 4]), rng.choice([1, 2, 3, 4, 5, 7, 8, 16])
        n_q = n_kv * g
        page = rng.choice([4, 5, 7, 8, 16, 16, 32, 64])
        window = rng.choice([0, 0, 0, rng.randint(1, 300)])
        R = rng.randint(1, 5)
        lens = [rng.choice(EDGES + [rng.randint(1, 1200)]) for _ in range(R)]
        decode = rng.random() < 0.4
        q_lens = [1] * R if decode else [min(n, rng.choice([1, 2, n, max(1, n // 2), rng.randint(1, n)])) for n in lens]
        q, kv, table, q_start, seq_lens = make_attention_case(torch.bfloat16, lens, q_lens, n_q, n_kv, d, page, seed=trial)
        for r, n in enumerate(lens):
            if n % page:
                kv[int(table[r, (n - 1) // page]), :, :, n % page:] = float("inf") if trial % 2 else float("nan")
        scale = d ** -0.5
        ref = attention_reference(q, kv, table, q_start, seq_lens, n_kv, page, scale, window)
        ql = np.asarray(q_lens, dtype=np.int32)
        what = f"trial {trial}: d={d} kv heads={n_kv} group={g} page={page} window={window} lens={lens} q_lens={q_lens}"
        flat = q.view(q.shape[0], -1)
        fresh = lambda: torch.full((q.shape[0], n_q * d), float("nan"), device=DEV, dtype=torch.bfloat16)

        out = fresh()
        req, r0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(ql * g, 64))
        ops().paged_attention_prefill(flat, n_q * d, out, kv, table, req, r0, q_start, seq_lens, n_q, n_kv, d, scale, window)
        assert rel_err(out.view_as(ref).cpu(), ref) < 1e-2, what
        if ops().tcgen05_attention_fits(d, n_q, n_kv, page, window):
            req, t0 = (torch.from_numpy(a).to(DEV) for a in query_tiles_host(ql, 128 // g))
            for parts in (1, rng.choice([2, 4, 8])):
                out = fresh()
                ops().paged_attention_prefill_tcgen05(flat, n_q * d, out, kv, table, req, t0, q_start, seq_lens, n_q, n_kv,
                                                      d, scale, parts)
                assert rel_err(out.view_as(ref).cpu(), ref) < 1e-2, (what, parts)
        if decode:
            fits = ops().tcgen05_attention_fits(d, n_q, n_kv, page, 0)
            for tma, stages in [(False, 2)] + ([(True, 2), (True, 3)] if fits else []):
                slices = rng.choice([1, 2, 3, 5, 8, 16, 24, 64])
                out = fresh()
                ops().paged_attention_decode(flat, n_q * d, out, kv, table, q_start, seq_lens, R, n_q, n_kv, d, scale,
                                             window, n_slices=slices, tma=tma, stages=stages)
                assert rel_err(out.view_as(ref).cpu(), ref) < 1e-2, (what, tma, stages, slices)
    ops().check_errors(torch.device(DEV))


def test_matrix_products_at_random_sizes():
    """1 to 700 tokens, widths from 16 to 4,608 that are no multiple of a tile, K any multiple of 8: the streaming
    kernel with its K slices, the one-SM and two-SM kernels at several tile widths, the fused SwiGLU, and whatever
    `linear` picks."""
    for trial in range(200):
        rng = random.Random(trial)
        torch.manual_seed(trial)
        small = rng.random() < 0.6
        tokens = rng.choice([1, 2, 7, 8, 15, 16, 17, 31, 32, 33, 63, 64] if small else [65, 127, 128, 129, 255, 256, 257, 300, 511, 700])
        features = rng.choice([16, 24, 100, 127, 128, 129, 200, 256, 264, 1000, 1152, 3584, 4608])
        k = 8 * rng.randint(1, 300) if rng.random() < 0.7 else rng.choice([64, 128, 896, 3584, 4864])
        x = torch.randn(tokens, k, device=DEV).bfloat16()
        w = (torch.randn(features, k, device=DEV) * 0.05).bfloat16()
        b = torch.randn(features, device=DEV).bfloat16() if rng.random() < 0.5 else None
        ref = x.double() @ w.double().T + (b.double() if b is not None else 0)
        what = f"trial {trial}: {tokens} x {features} x {k}, bias {b is not None}"
        if small:
            assert rel_err(ops().gemm_tcgen05(x, w, b, torch.float32), ref) < 3e-5, what
            assert rel_err(ops().gemm_tcgen05(x, w, b), ref) < 8e-3, what
            slices, bn = rng.choice([1, 2, 3, 5, 8, 11]), 16 if tokens <= 16 else (32 if tokens <= 32 else 64)
            if slices <= (k + 63) // 64:
                assert rel_err(ops().gemm_tcgen05(x, w, b, torch.float32, plan=(True, bn, slices)), ref) < 1e-4, (what, slices)
        else:
            assert rel_err(ops().gemm_tcgen05_many(x, w, b, torch.float32), ref) < 3e-5, what
            cols = rng.choice([16, 48, 64, 112, 208, 256])
            assert rel_err(ops().gemm_tcgen05_many(x, w, b, torch.float32, tile_cols=cols), ref) < 3e-5, (what, cols)
            assert rel_err(ops().gemm_tcgen05(x, w, b, torch.float32, plan=(False, 128, 1)), ref) < 3e-5, what
        assert rel_err(ops().linear(x, w, b), ref) < 8e-3, what
        if features % 128 == 0 and (small or features % 256 == 0):
            gate, up = (ref.view(tokens, -1, 2, 64)[:, :, i].reshape(tokens, -1) for i in (0, 1))
            assert rel_err(ops().gate_up_swiglu(x, w, b, 64), gate * torch.sigmoid(gate) * up) < 1.2e-2, what
    ops().check_errors(torch.device(DEV))


def test_sampling_kernel_at_random_settings():
    """Vocabularies from 6 to 151,936, every filter on and off, histories for the penalty, 64-bit seeds and
    draw counters: the kernel's token is one the plain chain keeps and the arg-max of its filtered logits plus
    the same noise.  Temperature 0 or top_k 1 is the arg-max of the raw logits, as in
    slipstream/core/sampling_params.py:46-48."""
    for trial in range(200):
        rng = random.Random(trial)
        torch.manual_seed(trial)
        vocab = rng.choice([6, 33, 100, 255, 1000, 5000, 32001, 151936])
        m = rng.randint(1, 9)
        logits = (torch.randn(m, vocab) * rng.choice([0.5, 2.5, 6.0])).to(DEV)
        rows, histories = [], []
        seen = torch.zeros(m, (vocab + 31) // 32, dtype=torch.int32, device=DEV)
        for i in range(m):
            rows.append(dict(temperature=rng.choice([0.0, 0.3, 0.7, 1.0, 1.5]),
                             seed=rng.choice([0, 5, 2 ** 40 + 3, rng.randint(0, 2 ** 62)]), draw=rng.choice([0, 1, 77, 2 ** 33]),
                             top_k=rng.choice([-1, -1, 1, 2, 40, vocab, vocab + 5]), top_p=rng.choice([1.0, 1.0, 0.95, 0.5, 0.01]),
                             min_p=rng.choice([0.0, 0.0, 0.05, 0.5]), repetition_penalty=rng.choice([1.0, 1.0, 1.3, 0.8])))
            histories.append([rng.randrange(vocab) for _ in range(rng.randint(0, 12))])
            if histories[-1]:
                ops().mark_seen(seen[i], torch.tensor(histories[-1], dtype=torch.int32, device=DEV), vocab)
        got = run_sample(logits, rows, seen=seen, slots=torch.arange(m, dtype=torch.int32, device=DEV))
        for i, r in enumerate(rows):
            row = logits[i].cpu()
            if r["temperature"] == 0.0 or r["top_k"] == 1:
                assert got[i] == int(row.argmax()), (trial, i, r)
                continue
            kept = plain.filtered_logits(row, temperature=r["temperature"], top_k=r["top_k"] if r["top_k"] <= vocab else -1,
                                         top_p=r["top_p"], min_p=r["min_p"], repetition_penalty=r["repetition_penalty"],
                                         history=histories[i]).numpy()
            score = kept + gumbel_noise(r["seed"], r["draw"], vocab)
            assert np.isfinite(kept[got[i]]) and score[got[i]] >= score.max() - 1e-3, (trial, i, r, got[i])


def test_engine_under_random_schedules_gives_the_tokens_of_the_engine_with_room(model_folders):
    """2 to 10 requests with prompts of 1 to 75 tokens and 1 to 40 new tokens, greedy or sampled with seeds,
    filters and penalty; pools of pages from barely enough for the longest request to three times that, at most
    2 to 16 requests and 3 to 256 tokens a step, prompt portions of 2 to 256 tokens.  In float32 every token
    equals that of an engine with 512 pages that runs whole prompts; in bfloat16 (rounding may move a token) the
    lengths do; every page comes back."""
    from slipstream_b200 import SamplingParams
    from slipstream_b200.engine.llm_engine import Request
    roomy, preemptions = {}, 0
    for trial in range(60):
        rng = random.Random(trial)
        name = rng.choice(sorted(model_folders))
        folder, config, page = model_folders[name]
        dtype = rng.choice(["float32", "float32", "bfloat16"])
        reqs = []
        for i in range(rng.randint(2, 10)):
            sample = rng.random() < 0.4
            params = SamplingParams(max_tokens=rng.randint(1, 40), temperature=rng.choice([0.7, 1.0]) if sample else 0.0,
                                    ignore_eos=True, top_k=rng.choice([-1, 5, 50]) if sample else -1,
                                    top_p=rng.choice([1.0, 0.9]) if sample else 1.0,
                                    repetition_penalty=rng.choice([1.0, 1.2]) if sample else 1.0,
                                    seed=trial * 100 + i if sample else None)
            longest_prompt = min(config.max_position_embeddings, 120) - 45
            reqs.append((f"r{i}", random_tokens(config.vocab_size, rng.randint(1, longest_prompt), trial * 31 + i), params))
        need = (max(len(p) + prm.max_tokens for _, p, prm in reqs) + page - 1) // page
        pages = rng.randint(need + 1, max(need + 2, 3 * need))
        sched = dict(max_num_seqs=rng.choice([2, 4, 16]), max_num_batched_tokens=rng.choice([3, 8, 32, 256]),
                     prefill_chunk_size=rng.choice([2, 7, 16, 64, 256]))
        batch = lambda: [Request(rid, None, p, prm, float(i)) for i, (rid, p, prm) in enumerate(reqs)]
        if (name, dtype) not in roomy:
            roomy[(name, dtype)] = make_engine(folder, page, dtype=dtype, pages=512)
        want = roomy[(name, dtype)].generate_batch(batch())
        tight = make_engine(folder, page, dtype=dtype, pages=pages, **sched)
        got = tight.generate_batch(batch())
        what = f"trial {trial}: {name} {dtype} {len(reqs)} requests, {pages} pages ({need} for the longest), {sched}"
        tight.runner.check()
        tight.runner.cache.check_invariants()
        assert tight.runner.cache.min_free_pages() == pages, what
        assert [len(g) for g in got] == [prm.max_tokens for _, _, prm in reqs], what
        if dtype == "float32":
            assert got == want, what
        preemptions += tight.scheduler.preemptions
    assert preemptions > 20, "the pools were meant to run out"
