"""The host-side rules that pick a kernel's shape (no GPU needed): slices of the decode attention, key parts of
the prefill attention, tile and K slices of the streaming matrix product, and which product a projection runs."""
import numpy as np

from slipstream_b200.ops import functions as F

SMS = 148  # the rules take the device's number of multiprocessors; here a B200's, without a device


def test_decode_slices_fill_one_wave_and_go_wide_only_for_few_long_requests():
    for n_requests in (1, 2, 3, 8, 24, 64, 300):
        for ctx in (1, 64, 1000, 8192, 32768):
            s = F.decode_slices(n_requests, 4, 7, ctx, sms=SMS)
            assert s in (1, 2, 4, 8) and s <= max(1, (ctx + 63) // 64)
            assert s == 1 or n_requests * 4 * s <= 2 * SMS
            w = F.decode_slices(n_requests, 4, 7, ctx, wide=True, sms=SMS)
            assert w == s or (w % 8 == 0 and w > 8 and n_requests * 4 * w <= 2 * SMS and ctx >= 64 * 8 * w)
    assert F.decode_slices(1, 4, 7, 32768, wide=True, sms=SMS) == 64 and F.decode_slices(8, 4, 7, 32768, wide=True, sms=SMS) == 8
    assert F.is_long_context(8192) and not F.is_long_context(8191)


def test_prefill_key_parts_only_while_all_blocks_run_at_once():
    assert F.prefill_key_parts([2048], [2048], 18, 4, sms=SMS) == 1          # 456 blocks
    assert F.prefill_key_parts([64], [4096], 18, 4, sms=SMS) == 8            # 16 blocks of 64 key tiles
    assert F.prefill_key_parts([512], [4096], 18, 4, sms=SMS) == 2           # 116 blocks
    assert F.prefill_key_parts([64], [600], 18, 4, sms=SMS) == 1             # too few key tiles to share
    assert F.prefill_key_parts([1] * 8 + [256], [4096] * 9, 18, 4, sms=SMS) == 2
    assert F.prefill_key_parts([], [], 18, 4, sms=SMS) == 1
    rng = np.random.default_rng(0)
    for _ in range(200):
        n = int(rng.integers(1, 6))
        seq = rng.integers(1, 20000, n)
        q = np.minimum(seq, rng.integers(1, 3000, n))
        parts = F.prefill_key_parts(q, seq, 18, 4, sms=SMS)
        blocks = int(((q + 17) // 18).sum()) * 4
        assert parts in (1, 2, 4, 8)
        assert parts == 1 or (blocks * parts <= 2 * SMS and (int(seq.max()) - 1) // 64 + 1 >= 8 * parts)


def test_streaming_product_plan_and_routing():
    for tokens in (1, 8, 16, 17, 33, 64):
        for features, k in ((4608, 3584), (3584, 3584), (37888, 3584), (3584, 18944), (152064, 3584), (96, 64)):
            swapped, bn, slices = F.gemm_plan(tokens, features, k, SMS)
            assert swapped and bn >= tokens and bn in (16, 32, 64) and 1 <= slices <= 8
            assert slices <= (k + 63) // 64
    # few tokens: every projection streams its weights through our kernel; 17 to 64: the large ones
    assert all(F.streams_weights(8, f, k, SMS) for f, k in ((4608, 3584), (3584, 3584), (37888, 3584), (3584, 18944)))
    assert F.streams_weights(64, 37888, 3584, SMS) and F.streams_weights(64, 3584, 18944, SMS) and not F.streams_weights(64, 3584, 3584, SMS)
    assert not F.streams_weights(65, 37888, 3584, SMS) and not F.streams_weights(8, 3584, 3580, SMS)
    assert F.many_tokens_swiglu_fits(2048, 37888, SMS) and not F.many_tokens_swiglu_fits(512, 37888, SMS)
    # prompt portions: the two-SM kernel from 2,048 tokens at the 7B and 14B layer sizes, the library elsewhere
    for features, k in ((4608, 3584), (3584, 3584), (3584, 18944), (7168, 5120), (5120, 13824)):
        assert F.many_tokens_fits(2048, features, k, SMS) and not F.many_tokens_fits(2047, features, k, SMS)
    for features, k in ((1152, 896), (896, 4864), (2048, 1536), (3584, 3580)):
        assert not F.many_tokens_fits(4096, features, k, SMS)


def test_where_a_projection_adds_itself_to_the_stream():
    """The last projection of a branch takes over the add and prepares the norm behind it in decode steps of up to
    16 tokens, where its K slices are a cluster and the width is a multiple of 128; for long prompt portions only
    when asked for."""
    for features, k in ((3584, 3584), (3584, 18944), (896, 4864), (5120, 13824), (128, 256)):
        for tokens in (1, 8, 16):
            assert F.adds_to_stream(tokens, features, k, SMS), (tokens, features, k)
        assert not F.adds_to_stream(17, features, k, SMS) and not F.adds_to_stream(64, features, k, SMS)
    assert not F.adds_to_stream(8, 3600, 3584, SMS)       # a width that is no multiple of 128
    assert not F.adds_to_stream(8, 3584, 3580, SMS)       # K that the tensor-core product does not take
    assert not F.adds_to_stream(8, 128, 64, SMS)          # one K step: nothing to cut into slices
    assert not F.adds_to_stream(2048, 3584, 3584, SMS)    # the two-SM kernel could; it did not pay
    try:
        F.set_norm_fusion(True, long_portions=True)
        assert F.adds_to_stream(2048, 3584, 3584, SMS) and not F.adds_to_stream(2047, 3584, 3584, SMS)
        F.set_norm_fusion(False)
        assert not F.adds_to_stream(8, 3584, 3584, SMS) and not F.adds_to_stream(2048, 3584, 3584, SMS)
    finally:
        F.set_norm_fusion(True)
    assert F.adds_to_stream(8, 3584, 3584, SMS)
