"""Runs the C++ operator layer's own test programs (nano-vllm-cpp_b200/host/tests/*.cpp).

``test_host_cpu`` needs no GPU: tensor views, the step context, the metadata builders against the arrays the
reference's tests expect, the KV-cache plan.  ``test_host_gpu`` repeats the reference's known-answer cases through
the ``Attention`` layer and the operator wrappers on a B200.
"""
import os
import subprocess

import pytest

from util import ROOT, entry

BUILD_DIR = os.path.join(ROOT, "nano-vllm-cpp_b200", "build")


def _run(name):
    entry.build()
    exe = os.path.join(BUILD_DIR, name)
    assert os.path.exists(exe), f"{exe} was not built"
    return subprocess.run([exe], capture_output=True, text=True, timeout=300)


def test_host_logic_without_a_gpu():
    res = _run("test_host_cpu")
    assert res.returncode == 0, res.stdout + res.stderr
    assert "0 failed" in res.stdout


@pytest.mark.gpu
def test_operator_layer_known_answers_on_gpu():
    res = _run("test_host_gpu")
    assert res.returncode == 0, res.stdout + res.stderr
    assert "0 failed" in res.stdout


# --------------------------------------------------------------------------------------------------------------
# Model shapes through the C++ layer: bf16, 32 / 8 heads, head_dim 128, 256-token blocks.  The driver program
# (host/tests/host_layer_driver.cpp) runs TransformerAttention::forward for a prefill step with prefix hits and for a
# decode step (eagerly, from a captured CUDA graph with an arena allocator, and through the unfused route); this
# side makes the inputs, and checks what came out against the CPU oracle.
# --------------------------------------------------------------------------------------------------------------
def _bf16_bits(x):
    import numpy as np
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    assert not (u & 0xFFFF).any(), "inputs must already be bf16-representable"
    return (u >> 16).astype(np.uint16)


def _from_bf16_bits(path, shape):
    import numpy as np
    u = np.fromfile(path, dtype=np.uint16).astype(np.uint32) << 16
    return u.view(np.float32).reshape(shape)


@pytest.mark.gpu
@pytest.mark.parametrize("index_int64", [0, 1])
def test_model_shapes_through_the_cpp_layer_eager_graph_and_both_routes(tmp_path, index_int64):
    import numpy as np

    import oracle
    from benchmarks import workloads as wl
    from util import assert_attention_close

    hq, hkv, d, bs, max_pos = 32, 8, 128, 256, 2048
    rng = np.random.default_rng(77)
    q_lens, prefix = [300, 70, 257], [256, 0, 512]                       # two of three sequences hit a cached prefix
    k_lens = [p + n for p, n in zip(prefix, q_lens)]
    seqs, total_q = len(q_lens), sum(q_lens)
    # decode: the three prefilled sequences grow by one token, plus one sequence that only lives in the cache
    extra_ctx = 1500
    need = [(k + 1 + bs - 1) // bs for k in k_lens] + [(extra_ctx + bs - 1) // bs]
    max_blocks = max(need) + 1
    num_blocks = sum(need) + 3
    perm = rng.permutation(num_blocks).astype(np.int32)
    tables = np.zeros((seqs + 1, max_blocks), np.int32)
    at = 0
    for i, n in enumerate(need):
        tables[i, :n] = perm[at:at + n]
        at += n
    rows_of = lambda s, pos: tables[s, pos // bs].astype(np.int64) * bs + pos % bs  # noqa: E731
    k_cache = wl.round_bf16(rng.standard_normal((num_blocks, bs, hkv, d)).astype(np.float32))
    v_cache = wl.round_bf16(rng.standard_normal((num_blocks, bs, hkv, d)).astype(np.float32))
    width = (hq + 2 * hkv) * d
    qkv_p = wl.round_bf16(rng.standard_normal((total_q, width)).astype(np.float32))
    qkv_d = wl.round_bf16(rng.standard_normal((seqs + 1, width)).astype(np.float32))
    qw = wl.round_bf16((1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32))
    kw = wl.round_bf16((1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32))
    cu_q = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    cu_k = np.concatenate([[0], np.cumsum(k_lens)]).astype(np.int32)
    pos_p = np.concatenate([np.arange(p, p + n) for p, n in zip(prefix, q_lens)]).astype(np.int32)
    slots_p = np.concatenate([rows_of(s, np.arange(p, p + n)) for s, (p, n) in enumerate(zip(prefix, q_lens))]).astype(np.int32)
    ctx = np.array([k + 1 for k in k_lens] + [extra_ctx], np.int32)
    pos_d = (ctx - 1).astype(np.int32)
    slots_d = np.array([rows_of(s, np.int64(c - 1)) for s, c in enumerate(ctx)]).astype(np.int32)
    idx = np.int64 if index_int64 else np.int32

    case = dict(num_heads=hq, num_kv_heads=hkv, head_dim=d, block_size=bs, num_blocks=num_blocks, num_seqs=seqs,
                total_q=total_q, max_blocks=max_blocks, decode_batch=seqs + 1, max_position=max_pos, bf16=1,
                index_int64=index_int64, max_seqlen_q=max(q_lens), max_seqlen_k=max(k_lens))
    (tmp_path / "case.txt").write_text("".join(f"{k} {v}\n" for k, v in case.items()))
    for name, arr in (("q_norm_weight", _bf16_bits(qw)), ("k_norm_weight", _bf16_bits(kw)), ("k_cache", _bf16_bits(k_cache)),
                      ("v_cache", _bf16_bits(v_cache)), ("prefill_qkv", _bf16_bits(qkv_p)), ("decode_qkv", _bf16_bits(qkv_d)),
                      ("prefill_positions", pos_p), ("decode_positions", pos_d), ("prefill_slot_mapping", slots_p),
                      ("decode_slot_mapping", slots_d), ("cu_seqlens_q", cu_q.astype(idx)), ("cu_seqlens_k", cu_k.astype(idx)),
                      ("prefill_block_tables", tables[:seqs].astype(idx)), ("decode_block_tables", tables.astype(idx)),
                      ("context_lens", ctx.astype(idx))):
        np.ascontiguousarray(arr).tofile(tmp_path / f"{name}.bin")

    entry.build()
    exe = os.path.join(BUILD_DIR, "host_layer_driver")
    res = subprocess.run([exe, str(tmp_path)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr

    # ---- the same two steps on the CPU oracle -----------------------------------------------------------------------
    table = np.fromfile(tmp_path / "cos_sin_cache.bin", dtype=np.float32).reshape(max_pos, d)
    np.testing.assert_allclose(table, oracle.build_cos_sin_cache(max_pos, d, 1.0e6), rtol=0, atol=2e-4)   # libm differences times position
    scale = 1.0 / np.sqrt(d)
    kc = k_cache.reshape(-1, hkv, d).copy()
    vc = v_cache.reshape(-1, hkv, d).copy()
    q_p = oracle.fused_split_norm_rope_store(qkv_p, pos_p, qw, kw, 1e-6, table, slots_p, kc, vc, hq, hkv, d)
    kc, q_p = wl.round_bf16(kc), wl.round_bf16(q_p)               # the cache and q are stored as bf16
    out_p = oracle.prefill_attention_paged(q_p, kc.reshape(k_cache.shape), vc.reshape(v_cache.shape), cu_q, cu_k,
                                           tables[:seqs], hkv, d, bs, scale)
    shape_c = (num_blocks * bs, hkv, d)
    got_kc = _from_bf16_bits(tmp_path / "k_cache_prefill.bin", shape_c)
    assert np.array_equal(_from_bf16_bits(tmp_path / "v_cache_prefill.bin", shape_c), vc)        # V rows are copies
    tol = np.maximum(np.abs(kc), 1e-3) * 2.0 ** -7                                              # K: one bf16 ulp
    assert (np.abs(got_kc - kc) <= tol).all() and (got_kc == kc).mean() > 0.98
    assert_attention_close(_from_bf16_bits(tmp_path / "out_prefill.bin", (total_q, hq, d)), out_p)

    kc2, vc2 = got_kc.copy(), vc.copy()                          # continue from the cache the GPU actually wrote
    q_d = wl.round_bf16(oracle.fused_split_norm_rope_store(qkv_d, pos_d, qw, kw, 1e-6, table, slots_d, kc2, vc2, hq, hkv, d))
    kc2 = wl.round_bf16(kc2)
    out_d = oracle.decode_attention_paged(q_d, kc2.reshape(k_cache.shape), vc2.reshape(v_cache.shape), ctx, tables, hkv, d, bs, scale)
    got_d = _from_bf16_bits(tmp_path / "out_decode.bin", (seqs + 1, hq, d))
    assert_attention_close(got_d, out_d)
    got_kc2 = _from_bf16_bits(tmp_path / "k_cache_decode.bin", shape_c)
    assert (np.abs(got_kc2 - kc2) <= np.maximum(np.abs(kc2), 1e-3) * 2.0 ** -7).all()
    assert np.array_equal(_from_bf16_bits(tmp_path / "v_cache_decode.bin", shape_c), vc2)

    # ---- graph replay and the unfused route give the eager fused route's bits ------------------------------------------
    raw = lambda name: np.fromfile(tmp_path / f"{name}.bin", dtype=np.uint16)  # noqa: E731
    assert np.array_equal(raw("out_decode_graph"), raw("out_decode"))
    assert np.array_equal(raw("k_cache_decode_graph"), raw("k_cache_decode"))
    assert np.array_equal(raw("k_cache_decode_unfused"), raw("k_cache_decode"))
    assert np.array_equal(raw("out_decode_unfused"), raw("out_decode"))
