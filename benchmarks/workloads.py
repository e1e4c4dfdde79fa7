"""Seeded synthetic inputs in the shapes of the benchmark configurations.

All generators are numpy-only and deterministic in ``seed``; values are N(0,1) * ``value_scale``
rounded to bf16 (held as float32) so that the CUDA path (bf16) and the fp32 oracle see identical
inputs.  Metadata follows the reference's engine contract
(src/engine/model_runner.cpp:525-538, :591-597, :748-769): ``slot = block_id * block_size + offset``,
``context_lens`` include the token being generated, ``block_tables`` rows are zero padded, and a
sequence's blocks are a slice of one random permutation of the pool.
"""
from __future__ import annotations

import math

import numpy as np


def round_bf16(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return u.view(np.float32).reshape(x.shape)


def _normal(rng, shape, value_scale, rounded=True):
    x = (rng.standard_normal(shape, dtype=np.float32) * np.float32(value_scale)).astype(np.float32)
    return round_bf16(x) if rounded else x


def build_block_tables(rng, context_lens, block_size, extra_pool_blocks=0, pad_to=None):
    """Random-permutation block tables: returns (tables [B, max_blocks] int32, pool size)."""
    need = [(int(c) + block_size - 1) // block_size for c in context_lens]
    pool = int(sum(need)) + int(extra_pool_blocks)
    pool = max(pool, 1)
    perm = rng.permutation(pool).astype(np.int32)
    width = max(max(need) if need else 1, 1)
    if pad_to is not None:
        width = max(width, int(pad_to))
    tables = np.zeros((len(need), width), dtype=np.int32)
    at = 0
    for i, n in enumerate(need):
        tables[i, :n] = perm[at:at + n]
        at += n
    return tables, pool


def make_decode_workload(batch, num_heads, num_kv_heads, head_dim, block_size, ctx_lo, ctx_hi, seed,
                         value_scale=1.0, prescale_q=False, rounded=True, pad_blocks_to=None,
                         extra_pool_blocks=0, context_lens=None):
    """One decode step: new-token q/k/v, a paged cache already holding the older tokens, metadata."""
    rng = np.random.default_rng(seed)
    if context_lens is None:
        context_lens = rng.integers(ctx_lo, ctx_hi + 1, size=batch)
    context_lens = np.asarray(context_lens, dtype=np.int32)
    tables, pool = build_block_tables(rng, np.maximum(context_lens, 1), block_size, extra_pool_blocks,
                                      pad_blocks_to)
    k_cache = _normal(rng, (pool, block_size, num_kv_heads, head_dim), value_scale, rounded)
    v_cache = _normal(rng, (pool, block_size, num_kv_heads, head_dim), value_scale, rounded)
    q = _normal(rng, (batch, num_heads, head_dim), value_scale, False)
    if prescale_q:
        q = q * np.float32(1.0 / math.sqrt(head_dim))
    if rounded:
        q = round_bf16(q)
    k_new = _normal(rng, (batch, num_kv_heads, head_dim), value_scale, rounded)
    v_new = _normal(rng, (batch, num_kv_heads, head_dim), value_scale, rounded)
    last = np.maximum(context_lens.astype(np.int64) - 1, 0)
    slots = tables[np.arange(batch), last // block_size].astype(np.int64) * block_size + last % block_size
    slots = np.where(context_lens > 0, slots, -1).astype(np.int32)
    return {
        "q": q, "k_new": k_new, "v_new": v_new, "k_cache": k_cache, "v_cache": v_cache,
        "slot_mapping": slots, "context_lens": context_lens, "block_tables": tables,
        "scale": 1.0 if prescale_q else 1.0 / math.sqrt(head_dim),
        "kv_bytes": int(context_lens.clip(min=0).sum()) * 2 * num_kv_heads * head_dim,  # x element size
    }


def make_prefill_workload(q_lens, prefix_lens, num_heads, num_kv_heads, head_dim, block_size, seed,
                          value_scale=1.0, rounded=True, paged=True):
    """Packed varlen prefill.  Paged: every key (prefix and new tokens) sits in the cache and is
    addressed through ``block_tables``; ``k_new``/``v_new``/``slot_mapping`` describe the new tokens so a
    test can clear those slots and run ``store_kvcache`` first.  Dense: ``k``/``v`` hold all keys."""
    rng = np.random.default_rng(seed)
    q_lens = [int(x) for x in q_lens]
    prefix_lens = [int(x) for x in prefix_lens]
    k_lens = [p + q for p, q in zip(prefix_lens, q_lens)]
    cu_q = np.zeros(len(q_lens) + 1, dtype=np.int32)
    cu_k = np.zeros(len(q_lens) + 1, dtype=np.int32)
    cu_q[1:] = np.cumsum(q_lens)
    cu_k[1:] = np.cumsum(k_lens)
    total_q, total_k = int(cu_q[-1]), int(cu_k[-1])
    q = _normal(rng, (total_q, num_heads, head_dim), value_scale, rounded)
    k_all = _normal(rng, (total_k, num_kv_heads, head_dim), value_scale, rounded)
    v_all = _normal(rng, (total_k, num_kv_heads, head_dim), value_scale, rounded)
    out = {"q": q, "cu_q": cu_q, "cu_k": cu_k, "scale": 1.0 / math.sqrt(head_dim),
           "q_lens": q_lens, "prefix_lens": prefix_lens}
    flops = 0
    for p, n in zip(prefix_lens, q_lens):
        flops += 4 * num_heads * head_dim * (n * p + n * (n + 1) // 2)
    out["flops"] = flops
    if not paged:
        out["k"] = k_all
        out["v"] = v_all
        return out
    tables, pool = build_block_tables(rng, np.maximum(np.asarray(k_lens), 1), block_size)
    k_cache = _normal(rng, (pool, block_size, num_kv_heads, head_dim), value_scale, rounded)
    v_cache = _normal(rng, (pool, block_size, num_kv_heads, head_dim), value_scale, rounded)
    kc = k_cache.reshape(pool * block_size, num_kv_heads, head_dim)
    vc = v_cache.reshape(pool * block_size, num_kv_heads, head_dim)
    slots = np.zeros(total_q, dtype=np.int32)
    k_new = np.zeros((total_q, num_kv_heads, head_dim), dtype=np.float32)
    v_new = np.zeros((total_q, num_kv_heads, head_dim), dtype=np.float32)
    for s, (p, n) in enumerate(zip(prefix_lens, q_lens)):
        pos = np.arange(p + n)
        rows = tables[s, pos // block_size].astype(np.int64) * block_size + pos % block_size
        kc[rows] = k_all[cu_k[s]:cu_k[s + 1]]
        vc[rows] = v_all[cu_k[s]:cu_k[s + 1]]
        slots[cu_q[s]:cu_q[s + 1]] = rows[p:]
        k_new[cu_q[s]:cu_q[s + 1]] = k_all[cu_k[s] + p:cu_k[s + 1]]
        v_new[cu_q[s]:cu_q[s + 1]] = v_all[cu_k[s] + p:cu_k[s + 1]]
    out.update({"k_cache": k_cache, "v_cache": v_cache, "block_tables": tables, "slot_mapping": slots,
                "k_new": k_new, "v_new": v_new})
    return out


def make_prologue_workload(rows, num_q_heads, num_kv_heads, head_dim, cache_rows, max_positions, seed,
                           rope_base=1.0e6):
    """Inputs of the fused decode prologue: packed qkv rows, norm weights, positions, slots."""
    rng = np.random.default_rng(seed)
    cols = (num_q_heads + 2 * num_kv_heads) * head_dim
    qkv = _normal(rng, (rows, cols), 1.0)
    qw = round_bf16((1.0 + 0.1 * rng.standard_normal(head_dim)).astype(np.float32))
    kw = round_bf16((1.0 + 0.1 * rng.standard_normal(head_dim)).astype(np.float32))
    positions = rng.integers(0, max_positions, size=rows).astype(np.int32)
    slots = rng.permutation(cache_rows)[:rows].astype(np.int32)
    return {"qkv": qkv, "q_norm_weight": qw, "k_norm_weight": kw, "positions": positions,
            "slot_mapping": slots, "rope_base": rope_base, "eps": 1e-6}
