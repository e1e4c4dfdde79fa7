"""int8 paged KV cache (store_kvcache_int8 / launch_decode_attention_paged_int8 of the reference,
src/kernels/kvcache.cu:222-369 and src/kernels/attention.cu:746-927).

CPU: the oracle's quantisation rule on hand-checked values.  GPU: the library's store must be bit-identical to the
oracle (int8 bytes and fp16 scales), its decode within the attention tolerance of the oracle's fp32 result on the same
quantised cache."""
import numpy as np
import pytest

import oracle
from util import F32_TOL, assert_attention_close, nvk, to_dev, to_np, workloads


def test_oracle_quantisation_rule_by_hand():
    key = np.zeros((3, 1, 4), np.float32)
    key[0, 0] = [1.0, -2.0, 0.5, 0.0]          # absmax 2: scale 2/127, q = rint(x * 63.5)
    key[1, 0] = [0.0, 0.0, 0.0, 0.0]           # all zero: scale floor 1e-10 (rounds to 0 in fp16), q = 0
    key[2, 0] = [3.0, 3.0, -3.0, 1.5]
    val = key[::-1].copy()
    kc = np.full((4, 1, 4), 99, np.int8); vc = np.full((4, 1, 4), 99, np.int8)
    ks = np.full((4, 1), -1, np.float32); vs = np.full((4, 1), -1, np.float32)
    oracle.store_kvcache_int8(key, val, kc, vc, ks, vs, np.array([2, 0, -1], np.int32))
    assert kc[2, 0].tolist() == [64, -127, 32, 0]            # 63.5 -> 64 (ties to even), 31.75 -> 32
    assert np.float16(ks[2, 0]) == np.float16(2.0 / 127.0) and ks[2, 0] == float(np.float16(2.0 / 127.0))
    assert kc[0, 0].tolist() == [0, 0, 0, 0] and ks[0, 0] == 0.0
    assert vc[2, 0].tolist() == [127, 127, -127, 64] and vc[0, 0].tolist() == [0, 0, 0, 0]
    assert (kc[1] == 99).all() and (kc[3] == 99).all() and ks[1, 0] == -1 and ks[3, 0] == -1   # untouched rows


def _quantised_cache(w, hkv, d, block_size):
    """Oracle-quantised copy of a bf16 decode workload's cache."""
    blocks = w["k_cache"].shape[0]
    rows = blocks * block_size
    kc = np.zeros((rows, hkv, d), np.int8); vc = np.zeros_like(kc)
    ks = np.zeros((rows, hkv), np.float32); vs = np.zeros_like(ks)
    slots = np.arange(rows, dtype=np.int32)
    oracle.store_kvcache_int8(w["k_cache"].reshape(rows, hkv, d), w["v_cache"].reshape(rows, hkv, d), kc, vc, ks, vs, slots)
    return kc, vc, ks, vs


@pytest.mark.gpu
@pytest.mark.parametrize("dtype_name,head_dim", [("bfloat16", 128), ("float16", 128), ("float32", 64), ("bfloat16", 256)])
def test_store_int8_is_bit_identical_to_the_oracle(dtype_name, head_dim):
    import torch
    dtype = getattr(torch, dtype_name)
    rng = np.random.default_rng(11)
    tokens, hkv, rows = 70, 4, 160
    key = torch.from_numpy(rng.standard_normal((tokens, hkv, head_dim)).astype(np.float32) * 1.7).to("cuda", dtype)
    val = torch.from_numpy(rng.standard_normal((tokens, hkv, head_dim)).astype(np.float32) * 0.3).to("cuda", dtype)
    key[5] = 0                                                  # an all-zero head vector
    slots = rng.permutation(rows)[:tokens].astype(np.int32)
    slots[::9] = -1
    slots[4] = rows + 3
    kc = torch.full((rows, hkv, head_dim), 77, dtype=torch.int8, device="cuda"); vc = kc.clone()
    ks = torch.full((rows, hkv), -2.0, dtype=torch.float16, device="cuda"); vs = ks.clone()
    nvk().store_kvcache_int8(key, val, kc, vc, ks, vs, to_dev(slots))
    torch.cuda.synchronize()
    rkc = np.full((rows, hkv, head_dim), 77, np.int8); rvc = rkc.copy()
    rks = np.full((rows, hkv), -2.0, np.float32); rvs = rks.copy()
    oracle.store_kvcache_int8(to_np(key), to_np(val), rkc, rvc, rks, rvs, slots)
    assert np.array_equal(kc.cpu().numpy(), rkc) and np.array_equal(vc.cpu().numpy(), rvc)
    assert np.array_equal(ks.cpu().numpy().view(np.uint16), rks.astype(np.float16).view(np.uint16))
    assert np.array_equal(vs.cpu().numpy().view(np.uint16), rvs.astype(np.float16).view(np.uint16))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype_name,num_heads,num_kv_heads,use_ws", [("bfloat16", 32, 8, True), ("float16", 16, 8, True),
                                                                      ("bfloat16", 8, 8, False), ("bfloat16", 4, 1, True)])
def test_decode_int8_tensor_core_path_matches_oracle(dtype_name, num_heads, num_kv_heads, use_ws):
    import torch
    dtype = getattr(torch, dtype_name)
    bs, d = 256, 128
    w = workloads().make_decode_workload(batch=6, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=d, block_size=bs,
                                         ctx_lo=1, ctx_hi=1500, seed=21)
    w["context_lens"][1] = 0                                      # zero row
    w["context_lens"][2] = 257                                    # one token into a second block
    kc, vc, ks, vs = _quantised_cache(w, num_kv_heads, d, bs)
    q = to_dev(w["q"], dtype)
    qf = to_np(q)
    ref = oracle.decode_attention_paged_int8(qf, kc, vc, ks, vs, w["context_lens"], w["block_tables"], num_kv_heads, d, bs, w["scale"])
    out = torch.full_like(q, float("nan"))
    lib = nvk()
    ws = None
    if use_ws:
        need = lib.decode_attention_workspace_bytes(q.shape[0], num_heads, num_kv_heads, d, w["block_tables"].shape[1], bs)
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    lib.launch_decode_attention_paged_int8(q, to_dev(kc), to_dev(vc), to_dev(ks, torch.float16), to_dev(vs, torch.float16),
                                           to_dev(w["context_lens"]), to_dev(w["block_tables"]), num_kv_heads, d, bs, w["scale"], out, ws)
    torch.cuda.synchronize()
    got = to_np(out)
    assert not np.isnan(got).any()
    assert (got[1] == 0).all()
    assert_attention_close(got, ref)


@pytest.mark.gpu
def test_decode_int8_general_path_fp32_and_small_head_dim():
    import torch
    bs, d, hq, hkv = 16, 64, 6, 2
    w = workloads().make_decode_workload(batch=5, num_heads=hq, num_kv_heads=hkv, head_dim=d, block_size=bs, ctx_lo=0, ctx_hi=90,
                                         seed=22, rounded=False)
    kc, vc, ks, vs = _quantised_cache(w, hkv, d, bs)
    ref = oracle.decode_attention_paged_int8(w["q"], kc, vc, ks, vs, w["context_lens"], w["block_tables"], hkv, d, bs, w["scale"])
    q = to_dev(w["q"])
    out = torch.full_like(q, float("nan"))
    nvk().launch_decode_attention_paged_int8(q, to_dev(kc), to_dev(vc), to_dev(ks, torch.float16), to_dev(vs, torch.float16),
                                             to_dev(w["context_lens"]), to_dev(w["block_tables"]), hkv, d, bs, w["scale"], out)
    torch.cuda.synchronize()
    assert np.abs(to_np(out) - ref).max() <= F32_TOL


@pytest.mark.gpu
def test_int8_round_trip_stays_close_to_the_16_bit_cache():
    """Size-independent property: store -> decode through the int8 cache agrees with the bf16 cache's decode to
    quantisation accuracy (one part in 127 of each head vector's range, averaged by the softmax)."""
    import torch
    bs, d, hq, hkv = 256, 128, 32, 8
    w = workloads().make_decode_workload(batch=8, num_heads=hq, num_kv_heads=hkv, head_dim=d, block_size=bs, ctx_lo=300, ctx_hi=2000, seed=23)
    lib = nvk()
    bf = torch.bfloat16
    q, kc16, vc16 = to_dev(w["q"], bf), to_dev(w["k_cache"], bf), to_dev(w["v_cache"], bf)
    rows = kc16.shape[0] * bs
    kc8 = torch.zeros((rows, hkv, d), dtype=torch.int8, device="cuda"); vc8 = torch.zeros_like(kc8)
    ks = torch.zeros((rows, hkv), dtype=torch.float16, device="cuda"); vs = torch.zeros_like(ks)
    lib.store_kvcache_int8(kc16.view(rows, hkv, d), vc16.view(rows, hkv, d), kc8, vc8, ks, vs,
                           torch.arange(rows, dtype=torch.int32, device="cuda"))
    ctx, bt = to_dev(w["context_lens"]), to_dev(w["block_tables"])
    need = lib.decode_attention_workspace_bytes(8, hq, hkv, d, bt.shape[1], bs)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    o16 = torch.empty_like(q); o8 = torch.empty_like(q)
    lib.launch_decode_attention_paged(q, kc16, vc16, ctx, bt, hkv, d, bs, w["scale"], o16, ws)
    lib.launch_decode_attention_paged_int8(q, kc8, vc8, ks, vs, ctx, bt, hkv, d, bs, w["scale"], o8, ws)
    torch.cuda.synchronize()
    err = np.abs(to_np(o8) - to_np(o16))
    assert err.max() <= 2e-2 and err.mean() <= 2e-3
