"""TEST INFRASTRUCTURE ONLY: numpy front-end of the CPU restatement (``nvk_oracle.c``).

Only the tests, the smoke run and the benchmark's CPU-baseline / reference legs import this
package.  It restates, in fp32 on the host, the reference kernels

* ``store_kvcache_kernel``                (src/kernels/kvcache.cu:19-47)
* ``decode_paged_attention_kernel``       (src/kernels/attention.cu:313-405)
* ``prefill_dense_attention_kernel``      (src/kernels/attention.cu:114-202)
* ``prefill_paged_attention_kernel``      (src/kernels/attention.cu:205-302)
* ``fused_split_norm_rope_store_kernel``  (src/kernels/split_qkv.cu:62-154)

Parity pin: known-answer cases of the reference's tests (tests/test_tensor.cpp:411-450,
tests/test_layers.cpp:82-191) plus fixtures under ``tests/golden/`` produced by the
reference's own CUDA kernels.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libnvk_oracle.so")
_lib = None

ROUND_NONE, ROUND_BF16, ROUND_FP16 = 0, 1, 2

_c_f32p = ctypes.POINTER(ctypes.c_float)
_c_i32p = ctypes.POINTER(ctypes.c_int32)


def build(force: bool = False) -> str:
    """Compile the C restatement (and, where the reference checkout exists, ``oracle/_ref``)."""
    src = os.path.join(_HERE, "nvk_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)
             or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src))
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, os.path.join(_HERE, "libnvk_oracle.so")],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


def build_reference() -> str | None:
    """Compile the reference's own kernels behind ``ref_shim.cpp`` (needs the reference checkout)."""
    out = os.path.join(_HERE, "_ref", "libnvk_ref.so")
    subprocess.check_call(["make", "-C", _HERE, "ref"], stdout=subprocess.DEVNULL,
                          stderr=subprocess.DEVNULL)
    return out if os.path.exists(out) else None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_round_bf16.restype = ctypes.c_float
        _lib.oracle_round_bf16.argtypes = [ctypes.c_float]
        _lib.oracle_round_fp16.restype = ctypes.c_float
        _lib.oracle_round_fp16.argtypes = [ctypes.c_float]
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def default_threads() -> int:
    return max(1, len(os.sched_getaffinity(0)))


def round_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 -> fp32 (vectorised; matches ``oracle_round_bf16``)."""
    u = _f32(x).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    u = ((u + 0x7FFF + lsb) & 0xFFFF0000).astype(np.uint32)
    return u.view(np.float32).reshape(np.shape(x))


def store_kvcache(key: np.ndarray, value: np.ndarray, k_cache: np.ndarray, v_cache: np.ndarray,
                  slot_mapping: np.ndarray) -> None:
    """In-place scatter; any dtype (byte copy).  ``key``/``value``: [N, ...]; caches: [rows, ...]."""
    n = int(slot_mapping.size)
    assert key.flags.c_contiguous and value.flags.c_contiguous
    assert k_cache.flags.c_contiguous and v_cache.flags.c_contiguous
    row_bytes = key.nbytes // n
    cache_rows = k_cache.nbytes // row_bytes
    sm = np.ascontiguousarray(slot_mapping)
    assert sm.dtype in (np.int32, np.int64)
    lib().oracle_store_kvcache(_p(key), _p(value), _p(k_cache), _p(v_cache), _p(sm),
                               ctypes.c_int(1 if sm.dtype == np.int64 else 0),
                               ctypes.c_int64(n), ctypes.c_int64(row_bytes),
                               ctypes.c_int64(cache_rows))


def decode_attention_paged(q, k_cache, v_cache, context_lens, block_tables, num_kv_heads,
                           head_dim, block_size, scale, threads: int | None = None) -> np.ndarray:
    q = _f32(q); k_cache = _f32(k_cache); v_cache = _f32(v_cache)
    cl = _i32(context_lens); bt = _i32(block_tables)
    batch, num_heads = q.shape[0], q.shape[1]
    out = np.empty_like(q)
    lib().oracle_decode_attention_paged(
        _p(q), _p(k_cache), _p(v_cache), _p(cl), _p(bt), ctypes.c_int64(batch),
        ctypes.c_int64(bt.shape[1]), ctypes.c_int(num_heads), ctypes.c_int(num_kv_heads),
        ctypes.c_int(head_dim), ctypes.c_int(block_size), ctypes.c_float(scale), _p(out),
        ctypes.c_int(threads or default_threads()))
    return out


def store_kvcache_int8(key, value, k_cache, v_cache, k_scale, v_scale, slot_mapping) -> None:
    """In place: ``k_cache`` / ``v_cache`` int8 [rows, Hkv, D] (any leading shape), ``k_scale`` / ``v_scale`` float32
    [rows, Hkv] holding the fp16-rounded scales."""
    key = _f32(key); value = _f32(value); sm = _i32(slot_mapping)
    for a, dt in ((k_cache, np.int8), (v_cache, np.int8), (k_scale, np.float32), (v_scale, np.float32)):
        assert a.dtype == dt and a.flags["C_CONTIGUOUS"]
    tokens, hkv, d = key.shape
    lib().oracle_store_kvcache_int8(_p(key), _p(value), _p(k_cache), _p(v_cache), _p(k_scale), _p(v_scale), _p(sm),
                                    ctypes.c_int64(tokens), ctypes.c_int(hkv), ctypes.c_int(d),
                                    ctypes.c_int64(k_cache.size // (hkv * d)))


def decode_attention_paged_int8(q, k_cache, v_cache, k_scale, v_scale, context_lens, block_tables, num_kv_heads,
                                head_dim, block_size, scale, threads: int | None = None) -> np.ndarray:
    q = _f32(q); cl = _i32(context_lens); bt = _i32(block_tables)
    k_scale = _f32(k_scale); v_scale = _f32(v_scale)
    assert k_cache.dtype == np.int8 and v_cache.dtype == np.int8
    k_cache = np.ascontiguousarray(k_cache); v_cache = np.ascontiguousarray(v_cache)
    batch, num_heads = q.shape[0], q.shape[1]
    out = np.empty_like(q)
    lib().oracle_decode_attention_paged_int8(
        _p(q), _p(k_cache), _p(v_cache), _p(k_scale), _p(v_scale), _p(cl), _p(bt), ctypes.c_int64(batch),
        ctypes.c_int64(bt.shape[1]), ctypes.c_int(num_heads), ctypes.c_int(num_kv_heads), ctypes.c_int(head_dim),
        ctypes.c_int(block_size), ctypes.c_float(scale), _p(out), ctypes.c_int(threads or default_threads()))
    return out


def store_kvcache_fp8(key, value, k_cache, v_cache, k_scale, v_scale, slot_mapping) -> None:
    """In place: ``k_cache`` / ``v_cache`` uint8 (e4m3 bytes) [rows, Hkv, D], ``k_scale`` / ``v_scale`` float32 [rows, Hkv]
    holding the fp16-rounded scales."""
    key = _f32(key); value = _f32(value); sm = _i32(slot_mapping)
    for a, dt in ((k_cache, np.uint8), (v_cache, np.uint8), (k_scale, np.float32), (v_scale, np.float32)):
        assert a.dtype == dt and a.flags["C_CONTIGUOUS"]
    tokens, hkv, d = key.shape
    lib().oracle_store_kvcache_fp8(_p(key), _p(value), _p(k_cache), _p(v_cache), _p(k_scale), _p(v_scale), _p(sm),
                                   ctypes.c_int64(tokens), ctypes.c_int(hkv), ctypes.c_int(d),
                                   ctypes.c_int64(k_cache.size // (hkv * d)))


def decode_attention_paged_fp8(q, k_cache, v_cache, k_scale, v_scale, context_lens, block_tables, num_kv_heads,
                               head_dim, block_size, scale) -> np.ndarray:
    q = _f32(q); cl = _i32(context_lens); bt = _i32(block_tables)
    k_scale = _f32(k_scale); v_scale = _f32(v_scale)
    assert k_cache.dtype == np.uint8 and v_cache.dtype == np.uint8
    k_cache = np.ascontiguousarray(k_cache); v_cache = np.ascontiguousarray(v_cache)
    batch, num_heads = q.shape[0], q.shape[1]
    out = np.empty_like(q)
    lib().oracle_decode_attention_paged_fp8(
        _p(q), _p(k_cache), _p(v_cache), _p(k_scale), _p(v_scale), _p(cl), _p(bt), ctypes.c_int64(batch),
        ctypes.c_int64(bt.shape[1]), ctypes.c_int(num_heads), ctypes.c_int(num_kv_heads), ctypes.c_int(head_dim),
        ctypes.c_int(block_size), ctypes.c_float(scale), _p(out))
    return out


def prefill_attention_dense(q, k, v, cu_seqlens_q, cu_seqlens_k, num_kv_heads, head_dim, scale,
                            threads: int | None = None) -> np.ndarray:
    q = _f32(q); k = _f32(k); v = _f32(v)
    out = np.empty_like(q)
    if cu_seqlens_q is None or cu_seqlens_k is None:
        cq = ck = None
        num_seqs = 1
    else:
        cq = _i32(cu_seqlens_q); ck = _i32(cu_seqlens_k)
        num_seqs = cq.size - 1
    lib().oracle_prefill_attention_dense(
        _p(q), _p(k), _p(v), _p(cq) if cq is not None else None,
        _p(ck) if ck is not None else None, ctypes.c_int64(num_seqs),
        ctypes.c_int64(q.shape[0]), ctypes.c_int64(k.shape[0]), ctypes.c_int(q.shape[1]),
        ctypes.c_int(num_kv_heads), ctypes.c_int(head_dim), ctypes.c_float(scale), _p(out),
        ctypes.c_int(threads or default_threads()))
    return out


def prefill_attention_paged(q, k_cache, v_cache, cu_seqlens_q, cu_seqlens_k, block_tables,
                            num_kv_heads, head_dim, block_size, scale,
                            threads: int | None = None) -> np.ndarray:
    q = _f32(q); k_cache = _f32(k_cache); v_cache = _f32(v_cache)
    cq = _i32(cu_seqlens_q); ck = _i32(cu_seqlens_k); bt = _i32(block_tables)
    out = np.empty_like(q)
    lib().oracle_prefill_attention_paged(
        _p(q), _p(k_cache), _p(v_cache), _p(cq), _p(ck), _p(bt), ctypes.c_int64(cq.size - 1),
        ctypes.c_int64(q.shape[0]), ctypes.c_int64(bt.shape[1]), ctypes.c_int(q.shape[1]),
        ctypes.c_int(num_kv_heads), ctypes.c_int(head_dim), ctypes.c_int(block_size),
        ctypes.c_float(scale), _p(out), ctypes.c_int(threads or default_threads()))
    return out


def build_cos_sin_cache(max_position: int, rotary_dim: int, base: float) -> np.ndarray:
    table = np.zeros((max_position, rotary_dim), dtype=np.float32)
    lib().oracle_build_cos_sin_cache(_p(table), ctypes.c_int(max_position),
                                     ctypes.c_int(rotary_dim), ctypes.c_float(base))
    return table


def fused_split_norm_rope_store(qkv, positions, q_norm_weight, k_norm_weight, norm_eps,
                                cos_sin_cache, slot_mapping, k_cache, v_cache, num_q_heads,
                                num_kv_heads, head_dim, round_mode=ROUND_BF16) -> np.ndarray:
    """Writes K/V rows into the fp32 ``k_cache``/``v_cache`` arrays in place; returns q_out."""
    qkv = _f32(qkv); pos = _i32(positions); sm = _i32(slot_mapping)
    qw = _f32(q_norm_weight); kw = _f32(k_norm_weight); cs = _f32(cos_sin_cache)
    assert k_cache.dtype == np.float32 and k_cache.flags.c_contiguous
    assert v_cache.dtype == np.float32 and v_cache.flags.c_contiguous
    rows = qkv.shape[0]
    q_out = np.empty((rows, num_q_heads, head_dim), dtype=np.float32)
    lib().oracle_fused_split_norm_rope_store(
        _p(qkv), _p(pos), _p(qw), _p(kw), ctypes.c_float(norm_eps), _p(cs),
        ctypes.c_int(cs.shape[0]), _p(sm), _p(k_cache), _p(v_cache), ctypes.c_int64(rows),
        ctypes.c_int(num_q_heads), ctypes.c_int(num_kv_heads), ctypes.c_int(head_dim), _p(q_out),
        ctypes.c_int(round_mode))
    return q_out
