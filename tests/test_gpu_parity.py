"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Tolerances: store_kvcache (and every copied byte) bit-exact; bf16 / fp16 attention within max-abs
2e-2 and mean-abs 2e-3 of the fp32 oracle on the same rounded inputs; fp32 attention within 2e-5.
"""
import math

import numpy as np
import pytest

import oracle
from util import assert_attention_close, nvk, to_dev, to_np, workloads

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _dt(name):
    return {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[name]


def round_f16(x):
    return x.astype(np.float16).astype(np.float32)


# ---------------------------------------------------------------------------------------- store

def test_store_kvcache_known_answer_fp32():
    """tests/test_tensor.cpp:411-450 of the reference, through the C ABI."""
    key = np.arange(1, 13, dtype=np.float32).reshape(3, 1, 4)
    value = -key
    k_cache = torch.zeros(2, 3, 1, 4, device="cuda")
    v_cache = torch.zeros(2, 3, 1, 4, device="cuda")
    nvk().store_kvcache(to_dev(key), to_dev(value), k_cache, v_cache, to_dev(np.array([2, -1, 5], np.int32)))
    exp_k = np.zeros(24, np.float32)
    exp_k[8:12] = key.reshape(-1)[0:4]
    exp_k[20:24] = key.reshape(-1)[8:12]
    assert np.array_equal(to_np(k_cache).reshape(-1), exp_k)
    assert np.array_equal(to_np(v_cache).reshape(-1), -exp_k)


@pytest.mark.parametrize("dtype,row_elems,slot_dtype", [
    ("bf16", 8 * 128, np.int32), ("bf16", 1 * 128, np.int64), ("f16", 2 * 64, np.int32),
    ("f32", 8 * 128, np.int32), ("f32", 3, np.int32), ("bf16", 5, np.int64), ("bf16", 36, np.int32),
])
def test_store_kvcache_bit_exact_with_padding_and_oob(dtype, row_elems, slot_dtype):
    rng = np.random.default_rng(3)
    n, cache_rows = 300, 1024
    key = rng.standard_normal((n, row_elems)).astype(np.float32)
    value = rng.standard_normal((n, row_elems)).astype(np.float32)
    slots = rng.permutation(cache_rows)[:n].astype(slot_dtype)
    slots[::7] = -1                      # padding rows
    slots[5] = cache_rows                # beyond the cache: ignored (src/kernels/kvcache.cu:34)
    slots[11] = cache_rows + 12345
    tk, tv = to_dev(key, _dt(dtype)), to_dev(value, _dt(dtype))
    k_cache = torch.randn(cache_rows, row_elems, device="cuda").to(_dt(dtype))
    v_cache = torch.randn(cache_rows, row_elems, device="cuda").to(_dt(dtype))
    kc_ref = k_cache.cpu().view(torch.uint8).numpy().copy()
    vc_ref = v_cache.cpu().view(torch.uint8).numpy().copy()
    oracle.store_kvcache(tk.cpu().view(torch.uint8).numpy(), tv.cpu().view(torch.uint8).numpy(), kc_ref, vc_ref, slots)
    nvk().store_kvcache(tk, tv, k_cache, v_cache, to_dev(slots))
    assert np.array_equal(k_cache.cpu().view(torch.uint8).numpy(), kc_ref)
    assert np.array_equal(v_cache.cpu().view(torch.uint8).numpy(), vc_ref)


@pytest.mark.parametrize("dtype,row_elems,slot_dtype,n", [
    ("bf16", 8 * 128, np.int32, 5000), ("f16", 2 * 128, np.int64, 4099), ("bf16", 8 * 128, np.int32, 9001),
])
def test_store_kvcache_large_copies_bit_exact(dtype, row_elems, slot_dtype, n):
    """Sizes at which whole rows go through the bulk-copy engine: padding and out-of-range slots in runs and alone,
    at the start and at the end, every row and every untouched cache row compared byte for byte."""
    rng = np.random.default_rng(31)
    cache_rows = n + 777
    key = rng.standard_normal((n, row_elems)).astype(np.float32)
    value = rng.standard_normal((n, row_elems)).astype(np.float32)
    slots = rng.permutation(cache_rows)[:n].astype(slot_dtype)
    slots[::5] = -1
    slots[0:9] = -1                      # a run of skipped rows at the start
    slots[100:140] = cache_rows + 3      # a run beyond the cache
    slots[-3:] = -1                      # and at the end
    tk, tv = to_dev(key, _dt(dtype)), to_dev(value, _dt(dtype))
    k_cache = torch.randn(cache_rows, row_elems, device="cuda").to(_dt(dtype))
    v_cache = torch.randn(cache_rows, row_elems, device="cuda").to(_dt(dtype))
    kc_ref = k_cache.cpu().view(torch.uint8).numpy().copy()
    vc_ref = v_cache.cpu().view(torch.uint8).numpy().copy()
    oracle.store_kvcache(tk.cpu().view(torch.uint8).numpy(), tv.cpu().view(torch.uint8).numpy(), kc_ref, vc_ref, slots)
    nvk().store_kvcache(tk, tv, k_cache, v_cache, to_dev(slots))
    assert np.array_equal(k_cache.cpu().view(torch.uint8).numpy(), kc_ref)
    assert np.array_equal(v_cache.cpu().view(torch.uint8).numpy(), vc_ref)


def test_store_kvcache_misaligned_views_and_duplicate_slots():
    rng = np.random.default_rng(5)
    n, row, cache_rows = 64, 24, 128
    buf_k = torch.zeros(n * row + 1, dtype=torch.bfloat16, device="cuda")
    key = buf_k[1:].view(n, row)             # 2-byte aligned only
    key.copy_(to_dev(rng.standard_normal((n, row)).astype(np.float32), torch.bfloat16))
    value = to_dev(rng.standard_normal((n, row)).astype(np.float32), torch.bfloat16)
    slots = rng.permutation(cache_rows)[:n].astype(np.int32)
    slots[1] = slots[0]                      # same slot twice with the same payload is idempotent
    key[1] = key[0]
    value[1] = value[0]
    k_cache = torch.zeros(cache_rows, row, dtype=torch.bfloat16, device="cuda")
    v_cache = torch.zeros(cache_rows, row, dtype=torch.bfloat16, device="cuda")
    nvk().store_kvcache(key, value, k_cache, v_cache, to_dev(slots))
    kc_ref = np.zeros((cache_rows, row), np.float32)
    vc_ref = np.zeros((cache_rows, row), np.float32)
    oracle.store_kvcache(to_np(key), to_np(value), kc_ref, vc_ref, slots)
    assert np.array_equal(to_np(k_cache), kc_ref) and np.array_equal(to_np(v_cache), vc_ref)


def test_store_kvcache_rejects_bad_arguments():
    k = torch.zeros(2, 4, device="cuda")
    with pytest.raises(ValueError):
        nvk().store_kvcache(k, k, k, k, torch.zeros(0, dtype=torch.int32, device="cuda"))
    with pytest.raises(ValueError):
        nvk().store_kvcache(k, k, k, k, torch.zeros(2, dtype=torch.float32, device="cuda"))
    with pytest.raises(ValueError):
        nvk().store_kvcache(k.cpu(), k, k, k, torch.zeros(2, dtype=torch.int32, device="cuda"))


# --------------------------------------------------------------------------------------- decode

def _run_decode(w, dtype, num_kv_heads, head_dim, block_size, use_workspace=True, do_store=True):
    td = _dt(dtype)
    q = to_dev(w["q"], td)
    k_cache, v_cache = to_dev(w["k_cache"], td), to_dev(w["v_cache"], td)
    ctx, bt = to_dev(w["context_lens"]), to_dev(w["block_tables"])
    kc_ref, vc_ref = w["k_cache"].copy(), w["v_cache"].copy()
    if do_store:
        nvk().store_kvcache(to_dev(w["k_new"], td), to_dev(w["v_new"], td), k_cache, v_cache, to_dev(w["slot_mapping"]))
        oracle.store_kvcache(w["k_new"], w["v_new"], kc_ref, vc_ref, w["slot_mapping"])
    out = torch.full_like(q, float("nan"))
    ws = None
    if use_workspace:
        nbytes = nvk().decode_attention_workspace_bytes(q.shape[0], q.shape[1], num_kv_heads, head_dim, bt.shape[1], block_size)
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    nvk().launch_decode_attention_paged(q, k_cache, v_cache, ctx, bt, num_kv_heads, head_dim, block_size, w["scale"], out, ws)
    torch.cuda.synchronize()
    ref = oracle.decode_attention_paged(w["q"], kc_ref, vc_ref, w["context_lens"], w["block_tables"],
                                        num_kv_heads, head_dim, block_size, w["scale"])
    return to_np(out), ref


def test_decode_known_answer_fp32_block_size_2():
    """tests/test_layers.cpp:118-153 of the reference: store slot 2, then attend over 3 keys."""
    k_cache = to_dev(np.array([1, 0, 0, 1, 0, 0, 0, 0], np.float32).reshape(2, 2, 1, 2))
    v_cache = to_dev(np.array([1, 2, 3, 4, 0, 0, 0, 0], np.float32).reshape(2, 2, 1, 2))
    nvk().store_kvcache(to_dev(np.array([[[1, 1]]], np.float32)), to_dev(np.array([[[5, 6]]], np.float32)),
                        k_cache, v_cache, to_dev(np.array([2], np.int32)))
    q = to_dev(np.array([[[1, 1]]], np.float32))
    out = torch.empty_like(q)
    s = 1.0 / math.sqrt(2.0)
    nvk().launch_decode_attention_paged(q, k_cache, v_cache, to_dev(np.array([3], np.int32)),
                                        to_dev(np.array([[0, 1]], np.int32)), 1, 2, 2, s, out)
    p0 = math.exp(1.0 * s - 2.0 * s)
    expected = [(p0 * 1 + p0 * 3 + 5) / (2 * p0 + 1), (p0 * 2 + p0 * 4 + 6) / (2 * p0 + 1)]
    np.testing.assert_allclose(to_np(out).reshape(-1), expected, atol=1e-5, rtol=0)


def test_decode_cpu_reference_config_fp32():
    """Qwen3-0.6B shape of the CPU-runnable configuration: 16/8 heads, D 128, fp32, batch 8, contexts in
    [64, 1024], 64-block pool, values N(0,1)*0.5, q pre-scaled by 1/sqrt(128), kernel scale 1."""
    wl = workloads()
    w = wl.make_decode_workload(8, 16, 8, 128, 256, 64, 1024, seed=1234, value_scale=0.5, prescale_q=True,
                                rounded=False)
    assert w["k_cache"].shape[0] <= 64 and w["scale"] == 1.0
    got, ref = _run_decode(w, "f32", 8, 128, 256)
    assert_attention_close(got, ref, half=False)


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("num_heads,num_kv_heads", [(32, 8), (16, 8), (8, 8), (8, 1), (14, 2)])
def test_decode_tensor_core_path_matches_oracle(dtype, num_heads, num_kv_heads):
    wl = workloads()
    w = wl.make_decode_workload(9, num_heads, num_kv_heads, 128, 256, 1, 2300, seed=100 + num_heads,
                                pad_blocks_to=12)
    if dtype == "f16":
        for k in ("q", "k_new", "v_new", "k_cache", "v_cache"):
            w[k] = round_f16(w[k])
    got, ref = _run_decode(w, dtype, num_kv_heads, 128, 256)
    assert_attention_close(got, ref)


def test_decode_context_edge_lengths_and_zero_rows():
    """Contexts around tile / block / chunk boundaries; context 0 rows must come out as zeros."""
    wl = workloads()
    lens = [0, 1, 15, 16, 17, 255, 256, 257, 511, 512, 513, 1023, 1024, 1025, 2047, 2048, 2049, 3000]
    w = wl.make_decode_workload(len(lens), 32, 8, 128, 256, 0, 0, seed=9, context_lens=lens, extra_pool_blocks=3)
    for use_ws in (True, False):
        got, ref = _run_decode(w, "bf16", 8, 128, 256, use_workspace=use_ws)
        assert not np.isnan(got).any()
        assert not got[0].any()
        assert_attention_close(got, ref)


def test_decode_graph_padded_table_and_small_batch_split():
    """Block-table rows padded far beyond the live blocks (CUDA-graph layout, model_runner.cpp:147) and a
    batch small enough that the split policy picks short chunks."""
    wl = workloads()
    w = wl.make_decode_workload(2, 32, 8, 128, 256, 3000, 4096, seed=21, pad_blocks_to=64)
    got, ref = _run_decode(w, "bf16", 8, 128, 256)
    assert_attention_close(got, ref)


def test_decode_stale_cache_contents_beyond_context_are_ignored():
    """Slots past context_len may hold anything (even NaN): they must not reach the output."""
    wl = workloads()
    w = wl.make_decode_workload(4, 32, 8, 128, 256, 10, 700, seed=33)
    kc, vc = w["k_cache"], w["v_cache"]
    for b, n in enumerate(w["context_lens"]):
        blk = w["block_tables"][b, (n - 1) // 256]
        kc[blk, (n - 1) % 256 + 1:] = np.nan
        vc[blk, (n - 1) % 256 + 1:] = np.nan
    got, ref = _run_decode(w, "bf16", 8, 128, 256)
    assert not np.isnan(got).any()
    assert_attention_close(got, ref)


@pytest.mark.parametrize("dtype,head_dim,block_size,num_heads,num_kv_heads", [
    ("f32", 64, 16, 4, 2), ("bf16", 64, 16, 4, 4), ("f32", 2, 2, 1, 1), ("f16", 96, 8, 6, 3), ("f32", 128, 32, 2, 1),
])
def test_decode_general_path_shapes(dtype, head_dim, block_size, num_heads, num_kv_heads):
    wl = workloads()
    w = wl.make_decode_workload(5, num_heads, num_kv_heads, head_dim, block_size, 0, 200, seed=head_dim,
                                rounded=(dtype == "bf16"))
    if dtype == "f16":
        for k in ("q", "k_new", "v_new", "k_cache", "v_cache"):
            w[k] = round_f16(w[k])
    got, ref = _run_decode(w, dtype, num_kv_heads, head_dim, block_size)
    assert_attention_close(got, ref, half=(dtype != "f32"))


# -------------------------------------------------------------------------------------- prefill

def test_prefill_dense_known_answer_fp32():
    """tests/test_layers.cpp:82-116 of the reference."""
    q = np.array([1, 0, 0, 1, 1, 1], np.float32).reshape(3, 1, 2)
    v = np.array([1, 2, 3, 4, 5, 6], np.float32).reshape(3, 1, 2)
    s = 1.0 / math.sqrt(2.0)
    out = torch.empty(3, 1, 2, device="cuda")
    cu = to_dev(np.array([0, 3], np.int32))
    nvk().launch_prefill_attention_dense(to_dev(q), cu, to_dev(q), to_dev(v), cu, 1, 2, s, out)
    b0 = math.exp(-s)
    c0 = math.exp(-s)
    expected = [1, 2, (b0 + 3) / (b0 + 1), (2 * b0 + 4) / (b0 + 1),
                (c0 + 3 * c0 + 5) / (2 * c0 + 1), (2 * c0 + 4 * c0 + 6) / (2 * c0 + 1)]
    np.testing.assert_allclose(to_np(out).reshape(-1), expected, atol=1e-5, rtol=0)
    out2 = torch.empty_like(out)
    nvk().launch_prefill_attention_dense(to_dev(q), None, to_dev(q), to_dev(v), None, 1, 2, s, out2)
    np.testing.assert_allclose(to_np(out2).reshape(-1), expected, atol=1e-5, rtol=0)


def test_prefill_paged_prefix_known_answer_fp32():
    """tests/test_layers.cpp:155-191 of the reference: cu_q {0,1}, cu_k {0,3}: bottom-right alignment."""
    k_cache = to_dev(np.array([1, 0, 0, 1, 1, 1, 0, 0], np.float32).reshape(2, 2, 1, 2))
    v_cache = to_dev(np.array([1, 2, 3, 4, 5, 6, 0, 0], np.float32).reshape(2, 2, 1, 2))
    q = to_dev(np.array([[[1, 1]]], np.float32))
    out = torch.empty_like(q)
    s = 1.0 / math.sqrt(2.0)
    nvk().launch_prefill_attention_paged(q, to_dev(np.array([0, 1], np.int32)), k_cache, v_cache,
                                         to_dev(np.array([0, 3], np.int32)), to_dev(np.array([[0, 1]], np.int32)),
                                         1, 2, 2, s, out)
    p0 = math.exp(1.0 * s - 2.0 * s)
    expected = [(p0 * 1 + p0 * 3 + 5) / (2 * p0 + 1), (p0 * 2 + p0 * 4 + 6) / (2 * p0 + 1)]
    np.testing.assert_allclose(to_np(out).reshape(-1), expected, atol=1e-5, rtol=0)
    with pytest.raises(ValueError):
        nvk().launch_prefill_attention_paged(q, None, k_cache, v_cache, None, to_dev(np.array([[0, 1]], np.int32)),
                                             1, 2, 2, s, out)


def _run_prefill(p, dtype, num_kv_heads, head_dim, block_size, paged, store_first=False):
    td = _dt(dtype)
    q = to_dev(p["q"], td)
    out = torch.full_like(q, float("nan"))
    cu_q, cu_k = to_dev(p["cu_q"]), to_dev(p["cu_k"])
    if paged:
        kc, vc = to_dev(p["k_cache"], td), to_dev(p["v_cache"], td)
        if store_first:   # clear the new tokens' slots, then let store_kvcache put them back
            flat_k = kc.view(-1, num_kv_heads, head_dim)
            flat_v = vc.view(-1, num_kv_heads, head_dim)
            idx = to_dev(p["slot_mapping"]).long()
            flat_k[idx] = 0
            flat_v[idx] = 0
            nvk().store_kvcache(to_dev(p["k_new"], td), to_dev(p["v_new"], td), kc, vc, to_dev(p["slot_mapping"]))
        nvk().launch_prefill_attention_paged(q, cu_q, kc, vc, cu_k, to_dev(p["block_tables"]), num_kv_heads,
                                             head_dim, block_size, p["scale"], out)
        ref = oracle.prefill_attention_paged(p["q"], p["k_cache"], p["v_cache"], p["cu_q"], p["cu_k"],
                                             p["block_tables"], num_kv_heads, head_dim, block_size, p["scale"])
    else:
        nvk().launch_prefill_attention_dense(q, cu_q, to_dev(p["k"], td), to_dev(p["v"], td), cu_k, num_kv_heads,
                                             head_dim, p["scale"], out)
        ref = oracle.prefill_attention_dense(p["q"], p["k"], p["v"], p["cu_q"], p["cu_k"], num_kv_heads,
                                             head_dim, p["scale"])
    torch.cuda.synchronize()
    return to_np(out), ref


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_prefill_dense_tensor_core_path(dtype):
    wl = workloads()
    p = wl.make_prefill_workload([1, 63, 64, 65, 200, 129], [0] * 6, 8, 2, 128, 256, seed=2, paged=False)
    if dtype == "f16":
        for k in ("q", "k", "v"):
            p[k] = round_f16(p[k])
    got, ref = _run_prefill(p, dtype, 2, 128, 256, paged=False)
    assert not np.isnan(got).any()
    assert_attention_close(got, ref)


def test_prefill_paged_with_prefix_hits_and_store():
    """Half of the sequences carry a whole-block prefix; new tokens are written by store_kvcache first."""
    wl = workloads()
    p = wl.make_prefill_workload([300, 77, 256, 130, 5], [256, 0, 512, 0, 768], 8, 2, 128, 256, seed=4)
    got, ref = _run_prefill(p, "bf16", 2, 128, 256, paged=True, store_first=True)
    assert not np.isnan(got).any()
    assert_attention_close(got, ref)


def test_prefill_paged_chunk_starting_mid_block_and_single_query_token():
    """Chunked prefill starts a chunk at any offset (model_runner.cpp:508-512); a fully cached prompt
    recomputes one token (tests/test_model_runner.cpp:182-239)."""
    wl = workloads()
    p = wl.make_prefill_workload([100, 1, 64], [37, 255, 1000], 4, 4, 128, 256, seed=6)
    got, ref = _run_prefill(p, "bf16", 4, 128, 256, paged=True)
    assert_attention_close(got, ref)


def test_prefill_gqa_group_of_four_matches_oracle():
    wl = workloads()
    p = wl.make_prefill_workload([190, 320], [0, 256], 32, 8, 128, 256, seed=8)
    got, ref = _run_prefill(p, "bf16", 8, 128, 256, paged=True)
    assert_attention_close(got, ref)


@pytest.mark.parametrize("dtype,head_dim,block_size,paged", [("f32", 64, 16, True), ("f32", 32, 4, False), ("bf16", 64, 16, True)])
def test_prefill_general_path_shapes(dtype, head_dim, block_size, paged):
    wl = workloads()
    p = wl.make_prefill_workload([5, 33, 1], [16 if paged else 0, 0, 48 if paged else 7], 4, 2, head_dim, block_size,
                                 seed=head_dim, rounded=(dtype == "bf16"), paged=paged)
    got, ref = _run_prefill(p, dtype, 2, head_dim, block_size, paged=paged)
    assert_attention_close(got, ref, half=(dtype != "f32"))


def test_prefill_rows_without_visible_keys_are_zero():
    """k_len < q_len: the first rows see no key at all (allowed_k <= 0, attention.cu:153-158)."""
    rng = np.random.default_rng(0)
    q = workloads().round_bf16(rng.standard_normal((5, 2, 128)).astype(np.float32))
    k = workloads().round_bf16(rng.standard_normal((3, 2, 128)).astype(np.float32))
    v = workloads().round_bf16(rng.standard_normal((3, 2, 128)).astype(np.float32))
    cu_q, cu_k = np.array([0, 5], np.int32), np.array([0, 3], np.int32)
    out = torch.full((5, 2, 128), float("nan"), device="cuda", dtype=torch.bfloat16)
    nvk().launch_prefill_attention_dense(to_dev(q, torch.bfloat16), to_dev(cu_q), to_dev(k, torch.bfloat16),
                                         to_dev(v, torch.bfloat16), to_dev(cu_k), 2, 128, 0.1, out)
    ref = oracle.prefill_attention_dense(q, k, v, cu_q, cu_k, 2, 128, 0.1)
    got = to_np(out)
    assert not got[:2].any() and not ref[:2].any()
    assert_attention_close(got, ref)


# ------------------------------------------------------------------------------- fused prologue

# (q heads, kv heads, head_dim, rows): 1 to 8 sixteen-byte pieces per lane, lane groups without a head (5 / 56 heads),
# more rows than the persistent grid has blocks (each block then pipelines several rows)
@pytest.mark.parametrize("num_q_heads,num_kv_heads,head_dim,rows", [
    (32, 8, 128, 37), (4, 1, 128, 37), (4, 2, 64, 37), (3, 1, 128, 9), (40, 8, 64, 50), (8, 2, 256, 37), (32, 8, 256, 20),
    (64, 16, 128, 37), (96, 16, 128, 21), (32, 8, 128, 700), (64, 8, 128, 401)])
def test_fused_split_norm_rope_store_matches_oracle(num_q_heads, num_kv_heads, head_dim, rows):
    wl = workloads()
    cache_rows, max_pos = max(512, rows + 64), 300
    w = wl.make_prologue_workload(rows, num_q_heads, num_kv_heads, head_dim, cache_rows, max_pos, seed=12)
    w["slot_mapping"][3] = -1                      # padded row: nothing written
    w["positions"][5] = max_pos + 7                # out of table: left un-rotated (split_qkv.cu:123)
    table = oracle.build_cos_sin_cache(max_pos, head_dim, w["rope_base"])
    kc_ref = np.zeros((cache_rows, num_kv_heads, head_dim), np.float32)
    vc_ref = np.zeros((cache_rows, num_kv_heads, head_dim), np.float32)
    q_ref = oracle.fused_split_norm_rope_store(w["qkv"], w["positions"], w["q_norm_weight"], w["k_norm_weight"],
                                               w["eps"], table, w["slot_mapping"], kc_ref, vc_ref, num_q_heads,
                                               num_kv_heads, head_dim)
    bf = torch.bfloat16
    kc = torch.zeros(cache_rows, num_kv_heads, head_dim, dtype=bf, device="cuda")
    vc = torch.zeros_like(kc)
    q_out = torch.empty(rows, num_q_heads, head_dim, dtype=bf, device="cuda")
    nvk().fused_split_norm_rope_store(to_dev(w["qkv"], bf), to_dev(w["positions"]), to_dev(w["q_norm_weight"], bf),
                                      to_dev(w["k_norm_weight"], bf), w["eps"], to_dev(table), to_dev(w["slot_mapping"]),
                                      kc, vc, num_q_heads, num_kv_heads, head_dim, q_out)
    torch.cuda.synchronize()
    # V rows are copies: bit-exact.  q / K pass through fp32 RMSNorm + RoPE and one bf16 rounding: the
    # GPU's rsqrt and fma contraction may move a value by one bf16 ulp (2^-8 relative).
    assert np.array_equal(to_np(vc), vc_ref)
    for got, ref in ((to_np(q_out), q_ref), (to_np(kc), kc_ref)):
        tol = np.maximum(np.abs(ref), 1e-3) * 2.0 ** -7
        assert (np.abs(got - ref) <= tol).all()
        assert (got == ref).mean() > 0.98


# ------------------------------------------------------- the kernels the library picks by shape

@pytest.mark.parametrize("num_heads,num_kv_heads", [(3, 3), (6, 2), (5, 1)])
def test_prefill_odd_gqa_groups_take_the_single_tile_tensor_core_kernel(num_heads, num_kv_heads):
    """Query-head groups of odd size (1, 3, 5) cannot be split into head pairs: the one-block-per-(tile, head)
    tcgen05 kernel serves them, paged with prefixes and dense."""
    wl = workloads()
    p = wl.make_prefill_workload([140, 1, 260, 129], [256, 512, 0, 0], num_heads, num_kv_heads, 128, 256, seed=31)
    got, ref = _run_prefill(p, "bf16", num_kv_heads, 128, 256, paged=True, store_first=True)
    assert not np.isnan(got).any()
    assert_attention_close(got, ref)
    d = wl.make_prefill_workload([70, 200, 1], [0, 0, 0], num_heads, num_kv_heads, 128, 256, seed=32, paged=False)
    got, ref = _run_prefill(d, "f16" if num_heads == 5 else "bf16", num_kv_heads, 128, 256, paged=False)
    assert_attention_close(got, ref)


@pytest.mark.parametrize("block_size", [64, 192])
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_prefill_small_cache_blocks_take_the_mma_sync_kernel(block_size, dtype):
    """A 128-key TMA tile must not straddle a cache block, so caches whose block size is a multiple of 64 but not of
    128 go to the mma.sync kernel (64-key tiles): prefix hits, a chunk that starts mid-block, a one-token sequence."""
    wl = workloads()
    p = wl.make_prefill_workload([150, 1, 64, 333], [block_size, 3 * block_size, 37, 0], 8, 2, 128, block_size, seed=33)
    if dtype == "f16":
        for k in ("q", "k_cache", "v_cache", "k_new", "v_new"):
            p[k] = round_f16(p[k])
    got, ref = _run_prefill(p, dtype, 2, 128, block_size, paged=True, store_first=True)
    assert not np.isnan(got).any()
    assert_attention_close(got, ref)


# -------------------------------------------------------------------------------- int64 index tensors

def test_int64_index_tensors_give_the_same_bits_as_int32():
    """The reference's kernels take int32 or int64 for each of cu_seqlens_q, cu_seqlens_k, context_lens and
    block_tables on its own (src/kernels/attention.cu:644-660, :708-735); so does the C ABI.  Mixed widths, every
    kernel family: tensor-core decode (split and unsplit), the general decode path, int8 decode, tcgen05 prefill
    (head pairs and single tile), the mma.sync prefill and the general prefill path."""
    wl = workloads()
    bf = torch.bfloat16
    L = torch.int64
    # decode: tensor-core path with and without workspace, general path (fp32)
    for dtype, hq, hkv, d, bs in (("bf16", 8, 2, 128, 256), ("f32", 4, 2, 64, 16)):
        w = wl.make_decode_workload(6, hq, hkv, d, bs, 1, 900, seed=41, rounded=(dtype == "bf16"))
        td = _dt(dtype)
        q, kc, vc = to_dev(w["q"], td), to_dev(w["k_cache"], td), to_dev(w["v_cache"], td)
        ctx, bt = to_dev(w["context_lens"]), to_dev(w["block_tables"])
        ws_bytes = nvk().decode_attention_workspace_bytes(6, hq, hkv, d, bt.shape[1], bs)
        for ws in (None, torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")):
            outs = []
            for c, t in ((ctx, bt), (ctx.to(L), bt), (ctx, bt.to(L)), (ctx.to(L), bt.to(L))):
                out = torch.full_like(q, float("nan"))
                nvk().launch_decode_attention_paged(q, kc, vc, c, t, hkv, d, bs, w["scale"], out, ws)
                outs.append(out)
            torch.cuda.synchronize()
            assert all(torch.equal(outs[0], o) for o in outs[1:])
    # prefill: head pairs (8/2), single tile (3/3), mma.sync (block 64), general path (head_dim 64)
    for hq, hkv, d, bs in ((8, 2, 128, 256), (3, 3, 128, 256), (8, 2, 128, 64), (4, 2, 64, 16)):
        p = wl.make_prefill_workload([130, 1, 70], [bs, 2 * bs, 0], hq, hkv, d, bs, seed=42)
        q, kc, vc = to_dev(p["q"], bf), to_dev(p["k_cache"], bf), to_dev(p["v_cache"], bf)
        cq, ck, bt = to_dev(p["cu_q"]), to_dev(p["cu_k"]), to_dev(p["block_tables"])
        outs = []
        for a, b, t in ((cq, ck, bt), (cq.to(L), ck, bt), (cq, ck.to(L), bt.to(L)), (cq.to(L), ck.to(L), bt.to(L))):
            out = torch.full_like(q, float("nan"))
            nvk().launch_prefill_attention_paged(q, a, kc, vc, b, t, hkv, d, bs, p["scale"], out)
            outs.append(out)
        torch.cuda.synchronize()
        assert not torch.isnan(outs[0].float()).any()
        assert all(torch.equal(outs[0], o) for o in outs[1:])
    with pytest.raises(ValueError):
        nvk().launch_decode_attention_paged(q, kc, vc, ctx.to(torch.int16), bt, 2, 64, 16, 1.0, torch.empty_like(q))


def test_decode_context_longer_than_the_block_table_is_clamped():
    """context_lens[b] beyond max_blocks * block_size cannot be addressed by the table row: the kernels clamp it
    (no read past the row, no read of another row's partial results) and the output equals the clamped result."""
    wl = workloads()
    bf = torch.bfloat16
    w = wl.make_decode_workload(4, 8, 2, 128, 256, 700, 1000, seed=43)
    cap = w["block_tables"].shape[1] * 256
    q, kc, vc, bt = to_dev(w["q"], bf), to_dev(w["k_cache"], bf), to_dev(w["v_cache"], bf), to_dev(w["block_tables"])
    clamped = w["context_lens"].copy()
    clamped[1] = cap
    wild = clamped.copy()
    wild[1] = cap + 5000
    ws = torch.empty(max(16, nvk().decode_attention_workspace_bytes(4, 8, 2, 128, bt.shape[1], 256)), dtype=torch.uint8, device="cuda")
    for workspace in (None, ws):
        a, b = torch.full_like(q, float("nan")), torch.full_like(q, float("nan"))
        nvk().launch_decode_attention_paged(q, kc, vc, to_dev(clamped), bt, 2, 128, 256, w["scale"], a, workspace)
        nvk().launch_decode_attention_paged(q, kc, vc, to_dev(wild), bt, 2, 128, 256, w["scale"], b, workspace)
        torch.cuda.synchronize()
        assert torch.isfinite(b.float()).all()
        assert torch.equal(a, b)


def test_prefill_status_is_zero_after_normal_launches():
    """Every tensor-core prefill launch above completed inside its bounded waits: the per-device error word is clear,
    and reading it clears it (plumbing check; a time-out itself is never provoked on a GPU)."""
    assert nvk().prefill_status() == 0
    assert nvk().prefill_status() == 0


# -------------------------------------------- the two forms of the prologue used by the unfused route

@pytest.mark.parametrize("num_q_heads,num_kv_heads,head_dim", [(32, 8, 128), (4, 1, 128), (6, 2, 64)])
def test_prologue_identity_slots_and_no_norm(num_q_heads, num_kv_heads, head_dim):
    """slot_mapping = None writes k / v of row r to row r of plain [rows, Hkv, D] tensors -- bit-identical to the fused
    form with slots 0 .. rows-1; norm weights = None skips the RMSNorm -- bit-identical to the oracle with unit weights
    and the head's own rms multiplied back ... which is not expressible, so it is checked against a torch fp32 RoPE."""
    wl = workloads()
    rows, max_pos = 45, 200
    w = wl.make_prologue_workload(rows, num_q_heads, num_kv_heads, head_dim, rows, max_pos, seed=14)
    table = to_dev(oracle.build_cos_sin_cache(max_pos, head_dim, w["rope_base"]))
    bf = torch.bfloat16
    qkv, pos = to_dev(w["qkv"], bf), to_dev(w["positions"])
    qw, kw = to_dev(w["q_norm_weight"], bf), to_dev(w["k_norm_weight"], bf)
    outs = []
    for slots in (to_dev(np.arange(rows, dtype=np.int32)), None):
        k = torch.zeros(rows, num_kv_heads, head_dim, dtype=bf, device="cuda")
        v = torch.zeros_like(k)
        q = torch.empty(rows, num_q_heads, head_dim, dtype=bf, device="cuda")
        nvk().fused_split_norm_rope_store(qkv, pos, qw, kw, w["eps"], table, slots, k, v, num_q_heads, num_kv_heads, head_dim, q)
        outs.append((q, k, v))
    torch.cuda.synchronize()
    for x, y in zip(*outs):
        assert torch.equal(x, y)
    # no norm: plain neox RoPE of the bf16 inputs, computed in fp32 and rounded once
    k = torch.zeros(rows, num_kv_heads, head_dim, dtype=bf, device="cuda")
    v = torch.zeros_like(k)
    q = torch.empty(rows, num_q_heads, head_dim, dtype=bf, device="cuda")
    nvk().fused_split_norm_rope_store(qkv, pos, None, None, w["eps"], table, None, k, v, num_q_heads, num_kv_heads, head_dim, q)
    torch.cuda.synchronize()
    x = qkv.float().view(rows, num_q_heads + 2 * num_kv_heads, head_dim)
    cs = table[pos.long()]                                     # [rows, D] = [cos | sin]
    cos, sin = cs[:, None, :head_dim // 2], cs[:, None, head_dim // 2:]
    lo, hi = x[..., :head_dim // 2], x[..., head_dim // 2:]
    rot = torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], dim=-1)
    want_q, want_k = rot[:, :num_q_heads], rot[:, num_q_heads:num_q_heads + num_kv_heads]
    for got, want in ((q, want_q), (k, want_k)):
        err = (got.float() - want).abs()
        assert (err <= want.abs().clamp_min(1e-3) * 2.0 ** -7).all()
    assert torch.equal(v, qkv.view(rows, -1, head_dim)[:, num_q_heads + num_kv_heads:])
