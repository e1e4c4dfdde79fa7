"""Pins the CPU oracle against the closed-form known-answer cases the reference's own tests hold.

Each case reproduces the inputs of one reference test and its expected values:
  * StoreKvCacheWritesSlotsAndSkipsPadding            tests/test_tensor.cpp:411-450
  * AttentionPrefillMatchesReference                  tests/test_layers.cpp:82-116
  * AttentionDecodeReadsKvCache                       tests/test_layers.cpp:118-153
  * AttentionPrefillWithPrefixCacheReadsPagedKvCache  tests/test_layers.cpp:155-191
"""
import math

import numpy as np

import oracle


def test_store_kvcache_writes_slots_and_skips_padding():
    key = np.arange(1, 13, dtype=np.float32).reshape(3, 1, 4)
    value = -key
    k_cache = np.zeros((2, 3, 1, 4), dtype=np.float32)
    v_cache = np.zeros((2, 3, 1, 4), dtype=np.float32)
    slots = np.array([2, -1, 5], dtype=np.int32)
    oracle.store_kvcache(key, value, k_cache, v_cache, slots)
    exp_k = np.zeros(24, dtype=np.float32)
    exp_v = np.zeros(24, dtype=np.float32)
    exp_k[8:12] = key.reshape(-1)[0:4]
    exp_v[8:12] = value.reshape(-1)[0:4]
    exp_k[20:24] = key.reshape(-1)[8:12]
    exp_v[20:24] = value.reshape(-1)[8:12]
    assert np.array_equal(k_cache.reshape(-1), exp_k)
    assert np.array_equal(v_cache.reshape(-1), exp_v)


def test_store_kvcache_ignores_slots_beyond_cache_and_int64():
    key = np.arange(8, dtype=np.float32).reshape(2, 4)
    value = key + 100
    k_cache = np.zeros((3, 4), dtype=np.float32)
    v_cache = np.zeros((3, 4), dtype=np.float32)
    oracle.store_kvcache(key, value, k_cache, v_cache, np.array([3, 1], dtype=np.int64))
    assert np.array_equal(k_cache[1], key[1]) and not k_cache[0].any() and not k_cache[2].any()
    assert np.array_equal(v_cache[1], value[1])


def test_prefill_dense_matches_reference_closed_form():
    q = np.array([1, 0, 0, 1, 1, 1], dtype=np.float32).reshape(3, 1, 2)
    k = q.copy()
    v = np.array([1, 2, 3, 4, 5, 6], dtype=np.float32).reshape(3, 1, 2)
    s = 1.0 / math.sqrt(2.0)
    out = oracle.prefill_attention_dense(q, k, v, [0, 3], [0, 3], 1, 2, s)
    b0, b1 = math.exp(0.0 * s - 1.0 * s), 1.0
    c0 = c1 = math.exp(1.0 * s - 2.0 * s)
    c2 = 1.0
    expected = [1.0, 2.0,
                (b0 * 1 + b1 * 3) / (b0 + b1), (b0 * 2 + b1 * 4) / (b0 + b1),
                (c0 * 1 + c1 * 3 + c2 * 5) / (c0 + c1 + c2),
                (c0 * 2 + c1 * 4 + c2 * 6) / (c0 + c1 + c2)]
    np.testing.assert_allclose(out.reshape(-1), expected, atol=1e-5, rtol=0)
    # null cu_seqlens: the whole batch is one sequence (src/kernels/attention.cu:37-43)
    out2 = oracle.prefill_attention_dense(q, k, v, None, None, 1, 2, s)
    np.testing.assert_allclose(out2.reshape(-1), expected, atol=1e-5, rtol=0)


def _paged_fixture():
    k_cache = np.array([1, 0, 0, 1, 0, 0, 0, 0], dtype=np.float32).reshape(2, 2, 1, 2)
    v_cache = np.array([1, 2, 3, 4, 0, 0, 0, 0], dtype=np.float32).reshape(2, 2, 1, 2)
    key = np.array([1, 1], dtype=np.float32).reshape(1, 1, 2)
    value = np.array([5, 6], dtype=np.float32).reshape(1, 1, 2)
    oracle.store_kvcache(key, value, k_cache, v_cache, np.array([2], dtype=np.int32))
    s = 1.0 / math.sqrt(2.0)
    p0 = p1 = math.exp(1.0 * s - 2.0 * s)
    p2 = 1.0
    expected = [(p0 * 1 + p1 * 3 + p2 * 5) / (p0 + p1 + p2),
                (p0 * 2 + p1 * 4 + p2 * 6) / (p0 + p1 + p2)]
    return k_cache, v_cache, s, expected


def test_decode_reads_kv_cache_through_block_table():
    k_cache, v_cache, s, expected = _paged_fixture()
    q = np.array([1, 1], dtype=np.float32).reshape(1, 1, 2)
    out = oracle.decode_attention_paged(q, k_cache, v_cache, [3], [[0, 1]], 1, 2, 2, s)
    np.testing.assert_allclose(out.reshape(-1), expected, atol=1e-5, rtol=0)


def test_decode_zero_context_gives_zero_rows():
    k_cache, v_cache, s, _ = _paged_fixture()
    q = np.ones((2, 1, 2), dtype=np.float32)
    out = oracle.decode_attention_paged(q, k_cache, v_cache, [0, 3], [[0, 0], [0, 1]], 1, 2, 2, s)
    assert not out[0].any() and out[1].any()


def test_prefill_paged_prefix_uses_bottom_right_causal_alignment():
    k_cache, v_cache, s, expected = _paged_fixture()
    q = np.array([1, 1], dtype=np.float32).reshape(1, 1, 2)
    out = oracle.prefill_attention_paged(q, k_cache, v_cache, [0, 1], [0, 3], [[0, 1]], 1, 2, 2, s)
    np.testing.assert_allclose(out.reshape(-1), expected, atol=1e-5, rtol=0)


def test_rounding_helpers_are_round_to_nearest_even():
    lib = oracle.lib()
    assert lib.oracle_round_bf16(1.0) == 1.0
    assert lib.oracle_round_bf16(1.00390625) == 1.0            # tie -> even
    assert lib.oracle_round_bf16(1.01171875) == 1.015625       # tie -> even (up)
    assert lib.oracle_round_fp16(1.00048828125) == 1.0         # tie -> even
    assert lib.oracle_round_fp16(65519.0) == 65504.0
    x = np.random.default_rng(0).standard_normal(1000).astype(np.float32)
    ref = np.array([lib.oracle_round_bf16(float(t)) for t in x], dtype=np.float32)
    assert np.array_equal(oracle.round_bf16(x), ref)
