"""The decode-attention entry point that allocates nothing (csrc/no_alloc.h), called through its exported
C symbol and compared with the ordinary entry point, whose scratch memory the caller allocates.

Some hosts of this library cannot hand it an allocator: all device memory was carved up at start-up, or the
code runs inside another runtime's pool, or a latency bound forbids a call that may stall the device.  For
them the library keeps 8 MiB of scratch in a built-in array.  The test makes two calls in a row with
different inputs (the array keeps the first call's contents, which must not leak into the second), and
checks that a call too large for the array is refused.

This file sorts last on purpose: a run that stops at the first failure has then run every other test.
"""
import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOO_LARGE = -1001


def _library(head_dim):
    from slipstream_b200 import ops

    lib = ctypes.CDLL(ops.attention_library(head_dim)._name)  # the same .so, through plain ctypes
    fn = lib.ss_attn_decode_noalloc
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int64, c_float, c_int, c_int, c_void_p, c_void_p]
    lib.ss_attn_decode_noalloc_floats.restype = c_int64
    lib.ss_attn_decode_noalloc_floats.argtypes = [c_int, c_int, c_int]
    lib.ss_attn_decode_noalloc_message.restype = ctypes.c_char_p
    lib.ss_attn_decode_noalloc_message.argtypes = [c_int]
    return lib


def _case(seed, lens, n_q, n_kv, d, page):
    g = torch.Generator().manual_seed(seed)
    blocks = [(l + page - 1) // page for l in lens]
    pages = sum(blocks) + 2
    order = torch.randperm(pages, generator=g).tolist()
    table = torch.full((len(lens), max(blocks)), -1, dtype=torch.int32)
    k = 0
    for r, nb in enumerate(blocks):
        for b in range(nb):
            table[r, b] = order[k]
            k += 1
    kv = (torch.randn(pages, 2, n_kv, page, d, generator=g) * 0.7).bfloat16().to(DEV)
    q = torch.randn(len(lens), n_q * d, generator=g).bfloat16().to(DEV)
    q_start = torch.arange(len(lens) + 1, dtype=torch.int32, device=DEV)
    return q, kv, table.to(DEV), q_start, torch.tensor(lens, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("n_q, n_kv, d, page, slices", [(28, 4, 128, 16, 6), (6, 2, 64, 4, 3)])
def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row(n_q, n_kv, d, page, slices):
    from slipstream_b200 import ops

    lib = _library(d)
    err = ops.error_word(torch.device(DEV))
    for call, lens in enumerate(([900, 64, 1, 333, 130], [17, 700, 65, 2, 1024])):
        q, kv, table, q_start, seq_lens = _case(10 * d + call, lens, n_q, n_kv, d, page)
        want = torch.zeros(len(lens), n_q * d, dtype=torch.bfloat16, device=DEV)
        ops.paged_attention_decode(q, n_q * d, want, kv, table, q_start, seq_lens, len(lens), n_q, n_kv, d,
                                   d ** -0.5, 0, n_slices=slices)
        got = torch.full_like(want, float("nan"))
        before = torch.cuda.memory_allocated()
        rc = lib.ss_attn_decode_noalloc(q.data_ptr(), n_q * d, got.data_ptr(), n_q * d, kv.data_ptr(),
                                        table.data_ptr(), table.shape[1], len(lens), q_start.data_ptr(),
                                        seq_lens.data_ptr(), n_q, n_kv, page, kv.shape[0], d ** -0.5, 0, slices,
                                        err.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0, lib.ss_attn_decode_noalloc_message(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        # same kernels, same order of additions: the same bits; the tests' bfloat16 bound is 1e-2 of the largest value
        scale = want.float().abs().max().item()
        assert (got.float() - want.float()).abs().max().item() <= 1e-2 * scale
        assert torch.equal(got, want)
    ops.check_errors(torch.device(DEV))


def test_a_call_beyond_the_built_in_scratch_is_refused():
    lib = _library(128)
    need = lib.ss_attn_decode_noalloc_floats(512, 28, 32)
    assert need > 2 * 1024 * 1024
    rc = lib.ss_attn_decode_noalloc(None, 0, None, 0, None, None, 1, 512, None, None, 28, 4, 16, 1, 1.0, 0, 32, None, None)
    assert rc == TOO_LARGE
    assert b"8 MiB" in lib.ss_attn_decode_noalloc_message(rc)
    assert lib.ss_attn_decode_noalloc(None, 0, None, 0, None, None, 1, 4, None, None, 7, 2, 16, 1, 1.0, 0, 1, None, None) == -1002
