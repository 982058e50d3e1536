"""The decode-attention entry point that allocates nothing (csrc/no_alloc.h), called through its exported
C symbol.

Some hosts of this library cannot hand it an allocator: all device memory was carved up at start-up, or the
code runs inside another runtime's pool, or a latency bound forbids a call that may stall the device.  For
them the library keeps 8 MiB of scratch in a built-in array.  The test makes two calls in a row with
different inputs and no synchronisation between them (the array keeps the first call's contents, which must
not leak into the second), compares both with double-precision attention on the CPU and, where the ordinary
entry point takes the same route through scratch memory, with that bit for bit; watches the driver's count of
free device memory around the calls; and checks that calls too large for the array are refused.

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


def float64_attention(q, kv, table, seq_lens, n_q, n_kv, d, page):
    """Softmax attention of one query token per request over its pages, in double precision on the CPU: the
    yardstick that shares nothing with the kernels."""
    out = torch.zeros(len(seq_lens), n_q, d, dtype=torch.float64)
    qd, kvd, group = q.double().cpu().view(-1, n_q, d), kv.double().cpu(), n_q // n_kv
    for r, length in enumerate(seq_lens.tolist()):
        blocks = (length + page - 1) // page
        pages = table[r, :blocks].long().cpu()
        keys = kvd[pages, 0].permute(1, 0, 2, 3).reshape(n_kv, blocks * page, d)[:, :length]
        values = kvd[pages, 1].permute(1, 0, 2, 3).reshape(n_kv, blocks * page, d)[:, :length]
        for h in range(n_q):
            scores = (keys[h // group] @ qd[r, h]) * d ** -0.5
            out[r, h] = torch.softmax(scores, 0) @ values[h // group]
    return out.view(len(seq_lens), n_q * d)


def free_device_bytes():
    return torch.cuda.mem_get_info()[0]  # the driver's own count: it sees a raw cudaMalloc, torch's counters do not


# slices up to 8: the ordinary entry point combines them inside a thread-block cluster, this one in its scratch
# array, so the two agree to rounding only; above 8 both take the scratch route and must agree bit for bit
@pytest.mark.parametrize("n_q, n_kv, d, page, slices", [(28, 4, 128, 16, 6), (6, 2, 64, 4, 3), (28, 4, 128, 16, 12),
                                                         (6, 2, 64, 4, 9), (5, 1, 16, 4, 17)])
def test_no_alloc_entry_point_twice_in_a_row(n_q, n_kv, d, page, slices):
    from slipstream_b200 import ops

    lib = _library(d)
    device = torch.device(DEV)
    err = ops.error_word(device)
    cases = [_case(10 * d + call, lens, n_q, n_kv, d, page)
             for call, lens in enumerate(([900, 64, 1, 333, 130], [17, 700, 65, 2, 1024]))]
    outs = [torch.full((5, n_q * d), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in cases]
    stream = torch.cuda.current_stream().cuda_stream

    def call(case, out):
        q, kv, table, q_start, seq_lens = case
        return lib.ss_attn_decode_noalloc(q.data_ptr(), n_q * d, out.data_ptr(), n_q * d, kv.data_ptr(),
                                          table.data_ptr(), table.shape[1], 5, q_start.data_ptr(),
                                          seq_lens.data_ptr(), n_q, n_kv, page, kv.shape[0], d ** -0.5, 0, slices,
                                          err.data_ptr(), stream)

    # the first call on a device looks the array up; it comes first, outside what is measured below
    assert call(cases[0], outs[0]) == 0
    torch.cuda.synchronize()
    outs[0].fill_(float("nan"))
    torch.cuda.synchronize()
    before = free_device_bytes()
    # two calls back to back in one stream, nothing between them: the second starts from what the first left in
    # the array, and must not read it before its own slices have written theirs
    codes = [call(case, out) for case, out in zip(cases, outs)]
    during = free_device_bytes()
    torch.cuda.synchronize()
    assert codes == [0, 0], [lib.ss_attn_decode_noalloc_message(c).decode() for c in codes]
    assert during == before == free_device_bytes(), "device memory was allocated by the calls"
    for (q, kv, table, q_start, seq_lens), got in zip(cases, outs):
        ref = float64_attention(q, kv, table, seq_lens, n_q, n_kv, d, page)
        assert (got.double().cpu() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item()
        if slices > 8:  # the ordinary entry point down the same route: the same additions in the same order
            want = torch.zeros_like(got)
            ops.paged_attention_decode(q, n_q * d, want, kv, table, q_start, seq_lens, 5, n_q, n_kv, d, d ** -0.5, 0,
                                       n_slices=slices, tma=False)
            assert torch.equal(got, want)
    ops.check_errors(device)


def test_a_call_beyond_the_built_in_scratch_is_refused():
    lib = _library(128)
    need = lib.ss_attn_decode_noalloc_floats(512, 28, 32)
    assert need > 2 * 1024 * 1024
    rc = lib.ss_attn_decode_noalloc(None, 0, None, 0, None, None, 1, 512, None, None, 28, 4, 16, 1, 1.0, 0, 32, None, None)
    assert rc == TOO_LARGE
    assert b"8 MiB" in lib.ss_attn_decode_noalloc_message(rc)
    assert lib.ss_attn_decode_noalloc(None, 0, None, 0, None, None, 1, 4, None, None, 7, 2, 16, 1, 1.0, 0, 1, None, None) == -1002
    # more slices than the kernel's merge has room for: refused on the host, nothing launched
    rc = lib.ss_attn_decode_noalloc(None, 0, None, 0, None, None, 1, 1, None, None, 1, 1, 16, 1, 1.0, 0, 65, None, None)
    assert rc == -1002 and b"64" in lib.ss_attn_decode_noalloc_message(rc)


def test_the_ordinary_entry_points_refuse_too_many_slices():
    from slipstream_b200 import ops

    q = torch.zeros(1, 128, dtype=torch.bfloat16, device=DEV)
    kv = torch.zeros(4, 2, 1, 16, 128, dtype=torch.bfloat16, device=DEV)
    table = torch.zeros(1, 4, dtype=torch.int32, device=DEV)
    q_start = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    lens = torch.tensor([40], dtype=torch.int32, device=DEV)
    for tma in (False, True):
        with pytest.raises(ops.KernelError, match="CUDA error"):
            ops.paged_attention_decode(q, 128, torch.empty_like(q), kv, table, q_start, lens, 1, 1, 1, 128, 1.0, 0,
                                       n_slices=65, tma=tma)
