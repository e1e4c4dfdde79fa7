"""Golden fixtures produced by the reference's own CUDA kernels (tests/golden/make_golden.py).

CPU part: pins the CPU oracle against the reference itself -- fp32 cases within 2e-5 (the oracle repeats the
reference's arithmetic order; only expf / rsqrtf differ between host and device), copied bytes bit-exact, bf16
cases within the rounding of the reference's bf16 output.  GPU part: this library's kernels against the same
fixtures through the C ABI.
"""
import os
import sys

import numpy as np
import pytest

import oracle
from util import ROOT, assert_attention_close, nvk, to_dev, to_np

sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
import make_golden as golden  # noqa: E402


def _case(name):
    inputs = golden.make_inputs(name)
    fixture = golden.load_fixture(name)
    assert golden.input_checksum(inputs) == str(fixture["checksum"]), "seeded inputs no longer match the fixture"
    return golden.CASES[name][2], inputs, fixture


def _bf16_ulp_close(got, ref, ulps=1.0):
    tol = np.maximum(np.abs(ref), 1e-3) * (2.0 ** -8) * ulps * 2
    return (np.abs(got - ref) <= tol).all()


# ------------------------------------------------------------------------------------------ CPU: oracle

def test_oracle_decode_fp32_matches_reference_kernel():
    kw, w, fx = _case("decode_f32_qwen06_shape")
    kc, vc = w["k_cache"].copy(), w["v_cache"].copy()
    oracle.store_kvcache(w["k_new"], w["v_new"], kc, vc, w["slot_mapping"])
    out = oracle.decode_attention_paged(w["q"], kc, vc, w["context_lens"], w["block_tables"], kw["num_kv_heads"],
                                        kw["head_dim"], kw["block_size"], w["scale"])
    assert np.abs(out - fx["out"]).max() <= 2e-5


def test_oracle_decode_bf16_inputs_match_reference_kernel():
    kw, w, fx = _case("decode_bf16_gqa4")
    kc, vc = w["k_cache"].copy(), w["v_cache"].copy()
    oracle.store_kvcache(w["k_new"], w["v_new"], kc, vc, w["slot_mapping"])
    out = oracle.decode_attention_paged(w["q"], kc, vc, w["context_lens"], w["block_tables"], kw["num_kv_heads"],
                                        kw["head_dim"], kw["block_size"], w["scale"])
    # the reference accumulates in fp32 and rounds once to bf16: the fp32 oracle is within half a bf16 ulp
    assert _bf16_ulp_close(oracle.round_bf16(out), fx["out"])
    assert (oracle.round_bf16(out) == fx["out"]).mean() > 0.97


def test_oracle_prefill_dense_fp32_matches_reference_kernel():
    kw, w, fx = _case("prefill_dense_f32")
    out = oracle.prefill_attention_dense(w["q"], w["k"], w["v"], w["cu_q"], w["cu_k"], kw["num_kv_heads"], kw["head_dim"],
                                         w["scale"])
    assert np.abs(out - fx["out"]).max() <= 2e-5


def test_oracle_prefill_paged_bf16_matches_reference_kernel():
    kw, w, fx = _case("prefill_paged_bf16_prefix")
    out = oracle.prefill_attention_paged(w["q"], w["k_cache"], w["v_cache"], w["cu_q"], w["cu_k"], w["block_tables"],
                                         kw["num_kv_heads"], kw["head_dim"], kw["block_size"], w["scale"])
    assert _bf16_ulp_close(oracle.round_bf16(out), fx["out"])


def test_oracle_store_is_bit_exact_with_reference_kernel():
    _, w, fx = _case("store_bf16")
    kc, vc = w["k_cache"].copy(), w["v_cache"].copy()
    oracle.store_kvcache(w["key"], w["value"], kc, vc, w["slot_mapping"])
    assert np.array_equal(kc, fx["k_cache"]) and np.array_equal(vc, fx["v_cache"])


def test_oracle_fused_prologue_matches_reference_kernel():
    kw, w, fx = _case("prologue_bf16")
    table = golden.cos_sin_table(kw["max_positions"], kw["head_dim"], w["rope_base"])
    kc = np.zeros((kw["cache_rows"], kw["num_kv_heads"], kw["head_dim"]), np.float32)
    vc = np.zeros_like(kc)
    q = oracle.fused_split_norm_rope_store(w["qkv"], w["positions"], w["q_norm_weight"], w["k_norm_weight"], w["eps"], table,
                                           w["slot_mapping"], kc, vc, kw["num_q_heads"], kw["num_kv_heads"], kw["head_dim"])
    assert np.array_equal(vc, fx["v_cache"])                       # V rows are copies
    for got, ref in ((q, fx["q_out"]), (kc, fx["k_cache"])):        # rsqrtf / fma contraction: at most one bf16 ulp
        assert _bf16_ulp_close(got, ref)
        assert (got == ref).mean() > 0.97


# ------------------------------------------------------------------------------------------ GPU: this library

@pytest.mark.gpu
@pytest.mark.parametrize("name", ["decode_f32_qwen06_shape", "decode_bf16_gqa4"])
def test_gpu_decode_matches_reference_fixture(name):
    import torch
    kw, w, fx = _case(name)
    td = torch.float32 if golden.CASES[name][1] == "f32" else torch.bfloat16
    q, kc, vc = to_dev(w["q"], td), to_dev(w["k_cache"], td), to_dev(w["v_cache"], td)
    nvk().store_kvcache(to_dev(w["k_new"], td), to_dev(w["v_new"], td), kc, vc, to_dev(w["slot_mapping"]))
    out = torch.empty_like(q)
    nvk().launch_decode_attention_paged_static(q, kc, vc, to_dev(w["context_lens"]), to_dev(w["block_tables"]),
                                               kw["num_kv_heads"], kw["head_dim"], kw["block_size"], w["scale"], out)
    assert_attention_close(to_np(out), fx["out"], half=(td != torch.float32))


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["prefill_dense_f32", "prefill_paged_bf16_prefix"])
def test_gpu_prefill_matches_reference_fixture(name):
    import torch
    kw, w, fx = _case(name)
    td = torch.float32 if golden.CASES[name][1] == "f32" else torch.bfloat16
    q = to_dev(w["q"], td)
    out = torch.empty_like(q)
    if kw.get("paged", True):
        nvk().launch_prefill_attention_paged(q, to_dev(w["cu_q"]), to_dev(w["k_cache"], td), to_dev(w["v_cache"], td),
                                             to_dev(w["cu_k"]), to_dev(w["block_tables"]), kw["num_kv_heads"], kw["head_dim"],
                                             kw["block_size"], w["scale"], out)
    else:
        nvk().launch_prefill_attention_dense(q, to_dev(w["cu_q"]), to_dev(w["k"], td), to_dev(w["v"], td), to_dev(w["cu_k"]),
                                             kw["num_kv_heads"], kw["head_dim"], w["scale"], out)
    assert_attention_close(to_np(out), fx["out"], half=(td != torch.float32))


@pytest.mark.gpu
def test_gpu_store_and_prologue_match_reference_fixtures():
    import torch
    bf = torch.bfloat16
    _, w, fx = _case("store_bf16")
    kc, vc = to_dev(w["k_cache"], bf), to_dev(w["v_cache"], bf)
    nvk().store_kvcache(to_dev(w["key"], bf), to_dev(w["value"], bf), kc, vc, to_dev(w["slot_mapping"]))
    assert np.array_equal(to_np(kc), fx["k_cache"]) and np.array_equal(to_np(vc), fx["v_cache"])

    kw, w, fx = _case("prologue_bf16")
    table = golden.cos_sin_table(kw["max_positions"], kw["head_dim"], w["rope_base"])
    kc = torch.zeros(kw["cache_rows"], kw["num_kv_heads"], kw["head_dim"], dtype=bf, device="cuda")
    vc = torch.zeros_like(kc)
    q_out = torch.empty(kw["rows"], kw["num_q_heads"], kw["head_dim"], dtype=bf, device="cuda")
    nvk().fused_split_norm_rope_store(to_dev(w["qkv"], bf), to_dev(w["positions"]), to_dev(w["q_norm_weight"], bf),
                                      to_dev(w["k_norm_weight"], bf), w["eps"], to_dev(table), to_dev(w["slot_mapping"]), kc, vc,
                                      kw["num_q_heads"], kw["num_kv_heads"], kw["head_dim"], q_out)
    assert np.array_equal(to_np(vc), fx["v_cache"])
    for got, ref in ((to_np(q_out), fx["q_out"]), (to_np(kc), fx["k_cache"])):
        assert _bf16_ulp_close(got, ref)
        assert (got == ref).mean() > 0.97


# ------------------------------------------------------------------------------------------ int8 KV cache

def _int8_case():
    kw, w, fx = _case("int8_kv_bf16")
    rows = w["k_cache"].shape[0] * kw["block_size"]
    shape = (rows, kw["num_kv_heads"], kw["head_dim"])
    return kw, w, fx, rows, shape


def test_oracle_int8_store_is_bit_exact_with_reference_kernel():
    kw, w, fx, rows, shape = _int8_case()
    kc = np.zeros(shape, np.int8); vc = np.zeros(shape, np.int8)
    ks = np.zeros(shape[:2], np.float32); vs = np.zeros(shape[:2], np.float32)
    oracle.store_kvcache_int8(w["k_cache"].reshape(shape), w["v_cache"].reshape(shape), kc, vc, ks, vs,
                              np.arange(rows, dtype=np.int32))
    assert np.array_equal(kc, fx["k_cache"]) and np.array_equal(vc, fx["v_cache"])
    assert np.array_equal(ks, fx["k_scale"]) and np.array_equal(vs, fx["v_scale"])


def test_oracle_int8_decode_matches_reference_kernel():
    kw, w, fx, rows, shape = _int8_case()
    out = oracle.decode_attention_paged_int8(w["q"], fx["k_cache"], fx["v_cache"], fx["k_scale"], fx["v_scale"], w["context_lens"],
                                             w["block_tables"], kw["num_kv_heads"], kw["head_dim"], kw["block_size"], w["scale"])
    assert _bf16_ulp_close(oracle.round_bf16(out), fx["out"])


@pytest.mark.gpu
def test_library_int8_store_and_decode_match_reference_kernels():
    import torch
    kw, w, fx, rows, shape = _int8_case()
    bf = torch.bfloat16
    lib = nvk()
    kc = torch.zeros(shape, dtype=torch.int8, device="cuda"); vc = torch.zeros_like(kc)
    ks = torch.zeros(shape[:2], dtype=torch.float16, device="cuda"); vs = torch.zeros_like(ks)
    lib.store_kvcache_int8(to_dev(w["k_cache"].reshape(shape), bf), to_dev(w["v_cache"].reshape(shape), bf), kc, vc, ks, vs,
                           torch.arange(rows, dtype=torch.int32, device="cuda"))
    q = to_dev(w["q"], bf)
    out = torch.empty_like(q)
    lib.launch_decode_attention_paged_int8(q, kc, vc, ks, vs, to_dev(w["context_lens"]), to_dev(w["block_tables"]), kw["num_kv_heads"],
                                           kw["head_dim"], kw["block_size"], w["scale"], out)
    torch.cuda.synchronize()
    assert np.array_equal(kc.cpu().numpy(), fx["k_cache"]) and np.array_equal(vc.cpu().numpy(), fx["v_cache"])
    assert np.array_equal(ks.float().cpu().numpy(), fx["k_scale"]) and np.array_equal(vs.float().cpu().numpy(), fx["v_scale"])
    assert_attention_close(to_np(out), fx["out"])
