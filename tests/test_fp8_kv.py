"""fp8 (e4m3) paged KV cache: nvk_store_kvcache_fp8 / nvk_decode_attention_paged_fp8.

The reference has no fp8 cache (its int8 cache is src/kernels/kvcache.cu:222-369 and src/kernels/attention.cu:746-927; an fp8
one is named as the step after it), so there is no reference output to compare with.  The format is pinned three ways:
the oracle's e4m3 encoder against hand-checked codes and against torch's float8_e4m3fn conversion (CPU), the library's
store bit for bit against the oracle (GPU), and the decode against the oracle's fp32 result on the same quantised cache
and against the 16-bit cache's decode (GPU)."""
import numpy as np
import pytest

import oracle
from util import assert_attention_close, nvk, to_dev, to_np, workloads


def _store(key, val, rows, slots):
    hkv, d = key.shape[1], key.shape[2]
    kc = np.full((rows, hkv, d), 0x55, np.uint8); vc = kc.copy()
    ks = np.full((rows, hkv), -2.0, np.float32); vs = ks.copy()
    oracle.store_kvcache_fp8(key, val, kc, vc, ks, vs, slots)
    return kc, vc, ks, vs


def test_oracle_e4m3_codes_by_hand():
    key = np.zeros((2, 1, 8), np.float32)
    # absmax 448: inverse scale 1, so the elements are encoded as they are
    key[0, 0] = [448.0, -448.0, 1.0, 0.0, 0.015625, 0.001953125, 17.0, 300.0]
    key[1, 0] = 0.0
    kc, _, ks, _ = _store(key, key.copy(), 4, np.array([1, 3], np.int32))
    # 448 = 1.75 * 2^8 -> 0x7e; 1 = 2^0 -> exponent 7, mantissa 0 -> 0x38; 2^-6 = smallest normal 0x08; 2^-9 = smallest
    # subnormal 0x01; 17 = 1.0625 * 2^4 halfway between 16 (0x58) and 18 (0x59) -> ties to even 0x58;
    # 300 = 1.171875 * 2^8 between 288 (0x79) and 320 (0x7a) -> nearer 288
    assert kc[1, 0].tolist() == [0x7e, 0xfe, 0x38, 0x00, 0x08, 0x01, 0x58, 0x79]
    assert ks[1, 0] == 1.0
    assert kc[3, 0].tolist() == [0] * 8 and ks[3, 0] == 0.0          # all-zero vector: scale floor rounds to 0 in fp16
    assert (kc[0] == 0x55).all() and (kc[2] == 0x55).all() and ks[0, 0] == -2.0     # untouched rows


def test_oracle_e4m3_encoder_agrees_with_torch():
    import torch
    rng = np.random.default_rng(41)
    x = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (0.01, 1.0, 30.0, 200.0)])
    key = x.reshape(-1, 1, 64).copy()
    key[:, 0, 0] = 448.0 * np.sign(key[:, 0, 1] + 1e-9)              # absmax 448 in every vector: elements encoded as they are
    np.clip(key, -448.0, 448.0, out=key)
    rows = key.shape[0]
    kc, _, _, _ = _store(key, key.copy(), rows, np.arange(rows, dtype=np.int32))
    ref = torch.from_numpy(key).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(kc, ref)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype_name,head_dim", [("bfloat16", 128), ("float16", 128), ("bfloat16", 64), ("float16", 256)])
def test_store_fp8_is_bit_identical_to_the_oracle(dtype_name, head_dim):
    import torch
    dtype = getattr(torch, dtype_name)
    rng = np.random.default_rng(12)
    tokens, hkv, rows = 70, 4, 160
    key = torch.from_numpy(rng.standard_normal((tokens, hkv, head_dim)).astype(np.float32) * 1.7).to("cuda", dtype)
    val = torch.from_numpy(rng.standard_normal((tokens, hkv, head_dim)).astype(np.float32) * 0.3).to("cuda", dtype)
    key[5] = 0                                                  # an all-zero head vector
    val[6, 0, :] = 1e-4                                         # a constant vector: every element at the top of the range
    slots = rng.permutation(rows)[:tokens].astype(np.int32)
    slots[::9] = -1
    slots[4] = rows + 3
    kc = torch.full((rows, hkv, head_dim), 0x55, dtype=torch.uint8, device="cuda"); vc = kc.clone()
    ks = torch.full((rows, hkv), -2.0, dtype=torch.float16, device="cuda"); vs = ks.clone()
    nvk().store_kvcache_fp8(key, val, kc, vc, ks, vs, to_dev(slots))
    torch.cuda.synchronize()
    rkc, rvc, rks, rvs = _store(to_np(key), to_np(val), rows, slots)
    assert np.array_equal(kc.cpu().numpy(), rkc) and np.array_equal(vc.cpu().numpy(), rvc)
    assert np.array_equal(ks.cpu().numpy().view(np.uint16), rks.astype(np.float16).view(np.uint16))
    assert np.array_equal(vs.cpu().numpy().view(np.uint16), rvs.astype(np.float16).view(np.uint16))


def _quantised_cache(w, hkv, d, block_size):
    rows = w["k_cache"].shape[0] * block_size
    return _store(w["k_cache"].reshape(rows, hkv, d), w["v_cache"].reshape(rows, hkv, d), rows, np.arange(rows, dtype=np.int32))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype_name,num_heads,num_kv_heads,use_ws,index_dtype", [
    ("bfloat16", 32, 8, True, np.int32), ("float16", 16, 8, True, np.int64), ("bfloat16", 8, 8, False, np.int32),
    ("bfloat16", 4, 1, True, np.int32)])
def test_decode_fp8_matches_oracle(dtype_name, num_heads, num_kv_heads, use_ws, index_dtype):
    import torch
    dtype = getattr(torch, dtype_name)
    bs, d = 256, 128
    w = workloads().make_decode_workload(batch=6, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=d, block_size=bs,
                                         ctx_lo=1, ctx_hi=1500, seed=24)
    w["context_lens"][1] = 0                                      # zero row
    w["context_lens"][2] = 257                                    # one token into a second block
    kc, vc, ks, vs = _quantised_cache(w, num_kv_heads, d, bs)
    q = to_dev(w["q"], dtype)
    ref = oracle.decode_attention_paged_fp8(to_np(q), kc, vc, ks, vs, w["context_lens"], w["block_tables"], num_kv_heads, d, bs, w["scale"])
    out = torch.full_like(q, float("nan"))
    lib = nvk()
    ws = None
    if use_ws:
        need = lib.decode_attention_workspace_bytes(q.shape[0], num_heads, num_kv_heads, d, w["block_tables"].shape[1], bs)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    lib.launch_decode_attention_paged_fp8(q, to_dev(kc), to_dev(vc), to_dev(ks, torch.float16), to_dev(vs, torch.float16),
                                          to_dev(w["context_lens"].astype(index_dtype)), to_dev(w["block_tables"].astype(index_dtype)),
                                          num_kv_heads, d, bs, w["scale"], out, ws)
    torch.cuda.synchronize()
    got = to_np(out)
    assert not np.isnan(got).any()
    assert (got[1] == 0).all()
    assert_attention_close(got, ref)


@pytest.mark.gpu
def test_fp8_round_trip_stays_close_to_the_16_bit_cache_and_rejects_other_shapes():
    """store -> decode through the e4m3 cache agrees with the bf16 cache's decode to the accuracy of three mantissa bits
    averaged by the softmax; shapes outside the tensor-core path are refused, not routed elsewhere."""
    import torch
    bs, d, hq, hkv = 256, 128, 32, 8
    w = workloads().make_decode_workload(batch=8, num_heads=hq, num_kv_heads=hkv, head_dim=d, block_size=bs, ctx_lo=300, ctx_hi=2000, seed=25)
    lib = nvk()
    bf = torch.bfloat16
    q, kc16, vc16 = to_dev(w["q"], bf), to_dev(w["k_cache"], bf), to_dev(w["v_cache"], bf)
    rows = kc16.shape[0] * bs
    kc8 = torch.zeros((rows, hkv, d), dtype=torch.uint8, device="cuda"); vc8 = torch.zeros_like(kc8)
    ks = torch.zeros((rows, hkv), dtype=torch.float16, device="cuda"); vs = torch.zeros_like(ks)
    lib.store_kvcache_fp8(kc16.view(rows, hkv, d), vc16.view(rows, hkv, d), kc8, vc8, ks, vs,
                          torch.arange(rows, dtype=torch.int32, device="cuda"))
    ctx, bt = to_dev(w["context_lens"]), to_dev(w["block_tables"])
    need = lib.decode_attention_workspace_bytes(8, hq, hkv, d, bt.shape[1], bs)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    o16 = torch.empty_like(q); o8 = torch.empty_like(q)
    lib.launch_decode_attention_paged(q, kc16, vc16, ctx, bt, hkv, d, bs, w["scale"], o16, ws)
    lib.launch_decode_attention_paged_fp8(q, kc8, vc8, ks, vs, ctx, bt, hkv, d, bs, w["scale"], o8, ws)
    torch.cuda.synchronize()
    err = np.abs(to_np(o8) - to_np(o16))
    assert err.max() <= 4e-2 and err.mean() <= 4e-3
    with pytest.raises((ValueError, RuntimeError)):
        lib.launch_decode_attention_paged_fp8(q.float(), kc8, vc8, ks, vs, ctx, bt, hkv, d, bs, w["scale"], o8.float(), ws)
