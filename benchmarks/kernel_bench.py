"""Single-GPU measurements of the kernels beside paged decode: varlen prefill, store_kvcache at
prefill size, the fused decode prologue, int8-cache decode and the mixed step.  ``bench.py --workload
{prefill,store,prologue,decode_int8,mixed}`` prints one JSON line per run in the same layout as the decode
benchmark (metric / value / roofline / clocks); ``other_kernels`` runs short versions of all of them for the
default benchmark line.

Every workload is seeded synthetic data in the shapes of the Qwen3-8B configurations: 32 query
heads, 8 KV heads, head_dim 128, bf16, 256-token cache blocks.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HQ, HKV, D, BS = 32, 8, 128, 256


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            j = json.load(fh)
        return float(j["hbm_gbs"]), float(j["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def _sustained_tflops():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return float(json.load(fh).get("bf16_tflops_sustained", 0.0)) or None
    return 1400.0


LAST_CLOCKS = None   # clock record of the most recent _time() call: every line below carries it


def _time(torch, fn, steps, warmup, flush=None):
    """Mean and median CUDA-event time of ``fn`` in ms; SM clock and throttle reasons are sampled while it runs."""
    global LAST_CLOCKS
    from .clocks import sampler_for_local_rank
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    sampler = sampler_for_local_rank()
    sampler.start()
    for a, b in evs:
        if flush is not None:
            flush()
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    LAST_CLOCKS = sampler.finish()
    times = sorted(a.elapsed_time(b) for a, b in evs)
    return float(np.mean(times)), float(times[len(times) // 2])


def make_prefill_inputs(torch, dev, seed, num_seqs=16, q_lo=512, q_hi=4096, prefix_frac=0.5):
    """Config 3: ``num_seqs`` sequences of U[q_lo, q_hi] new tokens, packed with cu_seqlens; half of them
    carry a prefix-cache hit of 256..1024 tokens (whole blocks) already sitting in paged blocks."""
    from . import workloads as wl
    rng = np.random.default_rng(seed)
    q_lens = rng.integers(q_lo, q_hi + 1, size=num_seqs)
    hit = rng.permutation(num_seqs)[: int(round(num_seqs * prefix_frac))]
    prefix = np.zeros(num_seqs, dtype=np.int64)
    prefix[hit] = rng.integers(1, 5, size=hit.size) * BS
    k_lens = prefix + q_lens
    cu_q = np.zeros(num_seqs + 1, np.int32)
    cu_k = np.zeros(num_seqs + 1, np.int32)
    cu_q[1:] = np.cumsum(q_lens)
    cu_k[1:] = np.cumsum(k_lens)
    tables, pool = wl.build_block_tables(rng, k_lens, BS)
    slots = np.zeros(int(cu_q[-1]), np.int32)
    prefix_rows = []
    for s in range(num_seqs):
        pos = np.arange(k_lens[s])
        rows = tables[s, pos // BS].astype(np.int64) * BS + pos % BS
        slots[cu_q[s]:cu_q[s + 1]] = rows[prefix[s]:]
        prefix_rows.append(rows[:prefix[s]])
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    bf = torch.bfloat16
    total_q = int(cu_q[-1])
    w = {
        "q": torch.randn((total_q, HQ, D), generator=gen, device=dev).to(bf),
        "k_new": torch.randn((total_q, HKV, D), generator=gen, device=dev).to(bf),
        "v_new": torch.randn((total_q, HKV, D), generator=gen, device=dev).to(bf),
        "k_cache": torch.zeros((pool, BS, HKV, D), device=dev, dtype=bf),
        "v_cache": torch.zeros((pool, BS, HKV, D), device=dev, dtype=bf),
        "cu_q": torch.from_numpy(cu_q).to(dev), "cu_k": torch.from_numpy(cu_k).to(dev),
        "block_tables": torch.from_numpy(tables).to(dev), "slot_mapping": torch.from_numpy(slots).to(dev),
        "q_lens": q_lens, "prefix": prefix, "pool": pool, "scale": 1.0 / math.sqrt(D),
    }
    pr = np.concatenate(prefix_rows) if prefix_rows else np.zeros(0, np.int64)
    if pr.size:
        idx = torch.from_numpy(pr).to(dev)
        w["k_cache"].view(-1, HKV, D)[idx] = torch.randn((pr.size, HKV, D), generator=gen, device=dev).to(bf)
        w["v_cache"].view(-1, HKV, D)[idx] = torch.randn((pr.size, HKV, D), generator=gen, device=dev).to(bf)
    w["out"] = torch.empty_like(w["q"])
    w["flops"] = int(sum(4 * HQ * D * (int(n) * int(p) + int(n) * (int(n) + 1) // 2) for n, p in zip(q_lens, prefix)))
    return w


def bench_prefill(nvk, torch, dev, steps, warmup, num_seqs=16, q_lo=512, q_hi=4096, prefix_frac=0.5):
    w = make_prefill_inputs(torch, dev, 2025, num_seqs, q_lo, q_hi, prefix_frac)
    nvk.store_kvcache(w["k_new"], w["v_new"], w["k_cache"], w["v_cache"], w["slot_mapping"])

    def attn():
        nvk.launch_prefill_attention_paged(w["q"], w["cu_q"], w["k_cache"], w["v_cache"], w["cu_k"],
                                           w["block_tables"], HKV, D, BS, w["scale"], w["out"])

    def store():
        nvk.store_kvcache(w["k_new"], w["v_new"], w["k_cache"], w["v_cache"], w["slot_mapping"])

    mean_ms, med_ms = _time(torch, attn, steps, warmup)
    attn_clocks = LAST_CLOCKS
    st_mean, _ = _time(torch, store, steps, warmup)
    hbm, tf, kind = _peaks()
    achieved = w["flops"] / (mean_ms * 1e-3) / 1e12
    total_q = int(w["q"].shape[0])
    store_bytes = 2 * (2 * total_q * HKV * D * 2) + 4 * total_q
    return {
        "metric": "varlen_prefill_attention_tflops", "value": achieved, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": mean_ms, "median_ms": med_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"varlen causal prefill, Qwen3-8B shape: {num_seqs} sequences of U[{q_lo},{q_hi}] new tokens, "
                               f"{'half' if prefix_frac == 0.5 else str(prefix_frac) + ' of them'} with a 256-1024-token paged prefix, keys read through block_tables",
                   "total_q": total_q, "flops_per_step": w["flops"],
                   "l2": "q/out (2 x %.0f MB) exceed the 126 MB L2" % (total_q * HQ * D * 2 / 1e6)},
        "roofline": {"bound": "tensor", "kernel": "prefill kernel", "achieved": achieved, "peak": tf,
                     "peak_source": f"{kind} cuBLAS bf16 burst", "unit": "TFLOP/s", "frac": achieved / tf,
                     "frac_of_nominal_2250": achieved / 2250.0,
                     "frac_of_sustained": (achieved / _sustained_tflops()) if _sustained_tflops() else None, "traffic": None},
        "store_kvcache": {"ms": st_mean, "bytes": store_bytes, "GBps": store_bytes / (st_mean * 1e-3) / 1e9,
                          "frac_of_" + kind + "_hbm": store_bytes / (st_mean * 1e-3) / 1e9 / hbm},
        "gpu_launches": 2 * steps, "clocks": attn_clocks,
    }


def bench_store(nvk, torch, dev, steps, warmup, tokens=36864):
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    bf = torch.bfloat16
    pool = (tokens + BS - 1) // BS + 64
    key = torch.randn((tokens, HKV, D), generator=gen, device=dev).to(bf)
    value = torch.randn((tokens, HKV, D), generator=gen, device=dev).to(bf)
    kc = torch.zeros((pool, BS, HKV, D), device=dev, dtype=bf)
    vc = torch.zeros_like(kc)
    slots = torch.from_numpy(np.random.default_rng(7).permutation(pool * BS)[:tokens].astype(np.int32)).to(dev)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    mean_ms, med_ms = _time(torch, lambda: nvk.store_kvcache(key, value, kc, vc, slots), steps, warmup,
                            flush=lambda: flush_buf.fill_(1))
    nbytes = 2 * (2 * tokens * HKV * D * 2) + 4 * tokens
    hbm, _, kind = _peaks()
    ach = nbytes / (mean_ms * 1e-3) / 1e9
    clocks = LAST_CLOCKS
    # the slot_mapping a prefill step really produces (prepare_prefill, src/engine/model_runner.cpp:520-548): consecutive
    # tokens fill whole 256-token blocks, the blocks lie anywhere in the pool
    order = np.random.default_rng(8).permutation(pool)[: (tokens + BS - 1) // BS].astype(np.int64)
    blockwise = (order[:, None] * BS + np.arange(BS)[None, :]).reshape(-1)[:tokens].astype(np.int32)
    slots_b = torch.from_numpy(blockwise).to(dev)
    mean_b, _ = _time(torch, lambda: nvk.store_kvcache(key, value, kc, vc, slots_b), steps, warmup, flush=lambda: flush_buf.fill_(1))
    ach_b = nbytes / (mean_b * 1e-3) / 1e9
    LAST_CLOCKS_B = LAST_CLOCKS
    # a contiguous device-to-device copy of the same bytes: what a copy of THIS size reaches (the measured peak is a 2 GB copy)
    src = torch.stack([key, value])
    dst = torch.empty_like(src)
    mean_c, _ = _time(torch, lambda: dst.copy_(src), steps, warmup, flush=lambda: flush_buf.fill_(1))
    ach_c = (nbytes - 4 * tokens) / (mean_c * 1e-3) / 1e9
    return {"same_size_contiguous_copy": {"ms": mean_c, "achieved": ach_c, "unit": "GB/s", "store_over_copy": ach / ach_c,
                                          "note": "torch copy_ of the same K and V rows into a contiguous buffer, same L2 flush"},
            "block_contiguous_slots": {"ms": mean_b, "achieved": ach_b, "unit": "GB/s", "frac": ach_b / hbm, "clocks": LAST_CLOCKS_B,
                                       "note": "whole 256-token blocks in random order, as prepare_prefill lays a prompt out"},
            "metric": "store_kvcache_hbm_bandwidth", "value": ach, "unit": "GB/s", "n_gpus": 1, "steps": steps,
            "warmup": warmup, "ms_per_step": mean_ms, "median_ms": med_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": f"store_kvcache of {tokens} tokens x 8 KV heads x 128 bf16 into random slots",
                       "l2": "a 256 MB buffer is written between timed iterations"},
            "roofline": {"bound": "hbm", "kernel": "store_rows_kernel", "achieved": ach, "peak": hbm,
                         "peak_source": f"{kind} copy bandwidth", "unit": "GB/s", "frac": ach / hbm, "traffic": None},
            "gpu_launches": 2 * steps, "clocks": clocks}


def bench_decode_int8(nvk, torch, dev, steps, warmup, batch=256, ctx_lo=1024, ctx_hi=8192, fmt="int8"):
    """Paged decode at the benchmark shape through the int8 KV cache: a bf16 cache is generated, quantised by the
    library's own store (timed as well), then decoded; the 16-bit decode of the same cache is timed beside it."""
    from . import workloads as wl
    rng = np.random.default_rng(2025)
    ctx = rng.integers(ctx_lo, ctx_hi + 1, size=batch).astype(np.int32)
    tables, pool = wl.build_block_tables(rng, ctx, BS)
    bf = torch.bfloat16
    gen = torch.Generator(device=dev)
    gen.manual_seed(2025)
    rows = pool * BS
    kc16 = torch.empty((pool, BS, HKV, D), device=dev, dtype=bf).normal_(generator=gen)
    vc16 = torch.empty((pool, BS, HKV, D), device=dev, dtype=bf).normal_(generator=gen)
    fp8 = fmt == "fp8"      # e4m3 bytes in the same layout (no counterpart in the reference)
    store_fn = nvk.store_kvcache_fp8 if fp8 else nvk.store_kvcache_int8
    decode_fn = nvk.launch_decode_attention_paged_fp8 if fp8 else nvk.launch_decode_attention_paged_int8
    kc8 = torch.empty((pool, BS, HKV, D), device=dev, dtype=torch.uint8 if fp8 else torch.int8)
    vc8 = torch.empty_like(kc8)
    ks = torch.empty((pool, BS, HKV), device=dev, dtype=torch.float16)
    vs = torch.empty_like(ks)
    slots = torch.arange(rows, dtype=torch.int32, device=dev)
    store = lambda: store_fn(kc16.view(rows, HKV, D), vc16.view(rows, HKV, D), kc8, vc8, ks, vs, slots)  # noqa: E731
    store_ms, _ = _time(torch, store, 5, 2)
    q = torch.randn((batch, HQ, D), generator=gen, device=dev).to(bf)
    out8, out16 = torch.empty_like(q), torch.empty_like(q)
    ctx_dev, tab_dev = torch.from_numpy(ctx).to(dev), torch.from_numpy(tables).to(dev)
    scale = 1.0 / math.sqrt(D)
    ws = torch.empty(max(16, nvk.decode_attention_workspace_bytes(batch, HQ, HKV, D, tables.shape[1], BS)), dtype=torch.uint8, device=dev)
    dec8 = lambda: decode_fn(q, kc8, vc8, ks, vs, ctx_dev, tab_dev, HKV, D, BS, scale, out8, ws)  # noqa: E731
    dec16 = lambda: nvk.launch_decode_attention_paged(q, kc16, vc16, ctx_dev, tab_dev, HKV, D, BS, scale, out16, ws)  # noqa: E731
    mean8, med8 = _time(torch, dec8, steps, warmup)
    clocks8 = LAST_CLOCKS
    mean16, _ = _time(torch, dec16, steps, warmup)
    err = (out8.float() - out16.float()).abs()
    tokens = int(ctx.astype(np.int64).sum())
    used = int(((ctx.astype(np.int64) + BS - 1) // BS).sum())
    bytes8 = tokens * HKV * (2 * D + 2 * 2) + 2 * batch * HQ * D * 2 + 4 * (used + batch)
    bytes16 = tokens * HKV * (2 * D * 2) + 2 * batch * HQ * D * 2 + 4 * (used + batch)
    store_bytes = 2 * rows * HKV * D * 2 + 2 * rows * HKV * (D + 2) + 4 * rows
    hbm, _, kind = _peaks()
    ach = bytes8 / (mean8 * 1e-3) / 1e9
    return {"metric": f"paged_decode_attention_{fmt}_kv_hbm_bandwidth", "value": ach, "unit": "GB/s", "n_gpus": 1, "steps": steps,
            "warmup": warmup, "ms_per_step": mean8, "median_ms": med8, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": f"{fmt} KV, f16 MMA", "data": "synthetic",
            "config": {"workload": f"paged decode attention, {'e4m3' if fp8 else 'int8'} KV cache with fp16 per-(token, head) scales, batch {batch}, "
                                   f"{HQ}/{HKV} heads, head_dim {D}, block_size {BS}, context U[{ctx_lo},{ctx_hi}]",
                       "context_tokens": tokens, "algorithmic_bytes": bytes8, "l2": "the cache (2 x %.1f GB) exceeds the 126 MB L2" % (rows * HKV * D / 1e9)},
            "roofline": {"bound": "hbm", "kernel": "decode_split_int8_kernel<T, fp8>" if fp8 else "decode_split_int8_kernel", "achieved": ach, "peak": hbm,
                         "peak_source": f"{kind} copy bandwidth", "unit": "GB/s", "frac": ach / hbm, "traffic": None},
            "bf16_cache_same_shape": {"ms_per_step": mean16, "GBps": bytes16 / (mean16 * 1e-3) / 1e9, "speedup_of_8_bit_cache": mean16 / mean8},
            "max_abs_diff_vs_bf16_cache": float(err.max()), "mean_abs_diff_vs_bf16_cache": float(err.mean()),
            f"store_kvcache_{fmt}": {"ms": store_ms, "tokens": rows, "bytes": store_bytes, "GBps": store_bytes / (store_ms * 1e-3) / 1e9,
                                   "frac_of_measured_hbm": store_bytes / (store_ms * 1e-3) / 1e9 / hbm},
            "gpu_launches": steps * 2, "clocks": clocks8}


def bench_prologue(nvk, torch, dev, steps, warmup, rows=256):
    """The fused prologue at ``rows`` token rows.  Prefill-sized inputs (larger than L2) are timed launch by launch.  At
    decode sizes a launch lasts a few microseconds and in a decoder it follows the QKV GEMM that has just left its
    packed rows in L2, inside a CUDA graph: so there the figure is the time per launch of a replayed graph of 64 launches
    that rotate over 16 sets of buffers (48 MB of packed rows in total: L2-resident, as after the GEMM)."""
    gen = torch.Generator(device=dev)
    gen.manual_seed(9)
    bf = torch.bfloat16
    qw = torch.ones(D, device=dev, dtype=bf)
    kw = torch.ones(D, device=dev, dtype=bf)
    max_pos = 4096
    inv_freq = 1.0 / (1.0e6 ** (np.arange(0, D, 2, dtype=np.float32) / D))
    ang = np.arange(max_pos, dtype=np.float32)[:, None] * inv_freq[None, :]
    table = torch.from_numpy(np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)).to(dev)
    pos = torch.randint(0, max_pos, (rows,), generator=gen, device=dev, dtype=torch.int32)
    pool = max(64, (rows + BS - 1) // BS)      # every row has its own cache slot
    slots = torch.from_numpy(np.random.default_rng(9).permutation(pool * BS)[:rows].astype(np.int32)).to(dev)
    nbytes = 2 * rows * (HQ + 2 * HKV) * D * 2 + rows * (D * 4 + 8)
    big = rows * (HQ + 2 * HKV) * D * 2 > (128 << 20)
    sets = 1 if big else 16

    def make_set():
        kc = torch.zeros((pool, BS, HKV, D), device=dev, dtype=bf)
        return (torch.randn((rows, (HQ + 2 * HKV) * D), generator=gen, device=dev).to(bf), kc, torch.zeros_like(kc),
                torch.empty((rows, HQ, D), device=dev, dtype=bf))

    bufs = [make_set() for _ in range(sets)]

    def launch(i):
        qkv, kc, vc, q_out = bufs[i % sets]
        nvk.fused_split_norm_rope_store(qkv, pos, qw, kw, 1e-6, table, slots, kc, vc, HQ, HKV, D, q_out)

    copy_line = None
    if big:
        mean_ms, med_ms = _time(torch, lambda: launch(0), steps, warmup)
        how = "the packed qkv input (%d MB) exceeds L2; CUDA events around every launch" % (rows * (HQ + 2 * HKV) * D * 2 >> 20)
        clocks_main = LAST_CLOCKS
        # a contiguous copy of the same packed rows: what a copy of THIS size reaches (the measured peak is a 2 GB copy)
        dst = torch.empty_like(bufs[0][0])
        mean_c, _ = _time(torch, lambda: dst.copy_(bufs[0][0]), steps, warmup)
        ach_c = 2 * rows * (HQ + 2 * HKV) * D * 2 / (mean_c * 1e-3) / 1e9
        copy_line = {"ms": mean_c, "achieved": ach_c, "unit": "GB/s", "prologue_over_copy": (nbytes / (mean_ms * 1e-3) / 1e9) / ach_c,
                     "note": "torch copy_ of the same packed qkv rows into a contiguous buffer"}
        LAST = clocks_main
    else:
        per_graph = 64
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(sets):
                launch(i)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(per_graph):
                launch(i)
        mean_ms, med_ms = _time(torch, graph.replay, steps, warmup)
        mean_ms, med_ms = mean_ms / per_graph, med_ms / per_graph
        how = f"time per launch of a replayed CUDA graph of {per_graph} launches over {sets} buffer sets (L2-resident inputs, as after the QKV GEMM)"
    hbm, _, kind = _peaks()
    ach = nbytes / (mean_ms * 1e-3) / 1e9
    return {"metric": "fused_split_norm_rope_store_hbm_bandwidth", "value": ach, "unit": "GB/s", "n_gpus": 1,
            "steps": steps, "warmup": warmup, "ms_per_step": mean_ms, "median_ms": med_ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"fused split + q/k RMSNorm + RoPE + KV store, {rows} rows of 48 heads x 128", "l2": how},
            "roofline": {"bound": "hbm", "kernel": "fused_prologue_kernel", "achieved": ach, "peak": hbm,
                         "peak_source": f"{kind} copy bandwidth", "unit": "GB/s", "frac": ach / hbm, "traffic": None},
            "same_size_contiguous_copy": copy_line,
            "gpu_launches": steps * (1 if big else 64), "clocks": (LAST if big else LAST_CLOCKS)}


def bench_mixed(nvk, torch, dev, steps, warmup, layers=36, decode_seqs=192, ctx_lo=512, ctx_hi=16384, prefill_seqs=4,
                prefill_len=2048, mem_fraction=0.80, hq=HQ, hkv=HKV, single_launch=False, prefill_blocks_hint=0):
    """Config 4: one continuous-batching step of attention over ``layers`` layer caches -- per layer the store of the
    prefill tokens, the varlen prefill (no prefix), the store of the decode tokens and the paged decode attention,
    all on one stream (the reference never fuses prefill and decode into one launch, src/engine/scheduler.cpp:65-67).
    36 distinct caches of this shape need about 226 GiB, more than one GPU holds, so as many distinct physical
    caches as fit are allocated and the logical layers are mapped onto them round-robin; every physical cache has
    its own block-table permutation and each is far larger than L2, so the reuse brings no cache hits.

    ``single_launch`` runs the same step with ONE attention launch per layer (``nvk_attention_mixed_step``: the
    prefill kernel's persistent blocks also take the decode items; the "true mixed step" the reference lists as
    future work, docs/interview_star.md:54) plus the merge of the decode splits."""
    from . import workloads as wl
    rng = np.random.default_rng(4040)
    ctx = rng.integers(ctx_lo, ctx_hi + 1, size=decode_seqs).astype(np.int32)
    dec_blocks = int(((ctx.astype(np.int64) + BS - 1) // BS).sum())
    pre_blocks = prefill_seqs * ((prefill_len + BS - 1) // BS)
    pool = dec_blocks + pre_blocks
    bytes_per_layer = 2 * pool * BS * hkv * D * 2
    free, _ = torch.cuda.mem_get_info(dev)
    phys = int(max(1, min(layers, (free * mem_fraction) // bytes_per_layer)))
    bf = torch.bfloat16
    gen = torch.Generator(device=dev)
    gen.manual_seed(4040)
    caches = []
    for _ in range(phys):
        perm = rng.permutation(pool).astype(np.int32)
        tables = np.zeros((decode_seqs, int(((ctx.max() + BS - 1) // BS))), np.int32)
        at = 0
        for i, c in enumerate(ctx):
            n = (int(c) + BS - 1) // BS
            tables[i, :n] = perm[at:at + n]
            at += n
        last = ctx.astype(np.int64) - 1
        dslots = (tables[np.arange(decode_seqs), last // BS].astype(np.int64) * BS + last % BS).astype(np.int32)
        pblocks = perm[at:at + pre_blocks].reshape(prefill_seqs, -1)
        pos = np.arange(prefill_len)
        pslots = np.concatenate([pblocks[s, pos // BS].astype(np.int64) * BS + pos % BS for s in range(prefill_seqs)]).astype(np.int32)
        kc = torch.empty((pool, BS, hkv, D), device=dev, dtype=bf).normal_(generator=gen)
        vc = torch.empty((pool, BS, hkv, D), device=dev, dtype=bf).normal_(generator=gen)
        all_tables = np.zeros((prefill_seqs + decode_seqs, tables.shape[1]), np.int32)
        all_tables[:prefill_seqs, :pblocks.shape[1]] = pblocks
        all_tables[prefill_seqs:] = tables
        caches.append({"k": kc, "v": vc, "tables": torch.from_numpy(tables).to(dev), "dslots": torch.from_numpy(dslots).to(dev),
                       "pslots": torch.from_numpy(pslots).to(dev), "all_tables": torch.from_numpy(all_tables).to(dev),
                       "all_slots": torch.from_numpy(np.concatenate([pslots, dslots])).to(dev)})
    total_pq = prefill_seqs * prefill_len
    cu = torch.arange(0, total_pq + 1, prefill_len, dtype=torch.int32, device=dev)
    pq = torch.randn((total_pq, hq, D), generator=gen, device=dev).to(bf)
    pk = torch.randn((total_pq, hkv, D), generator=gen, device=dev).to(bf)
    pv = torch.randn((total_pq, hkv, D), generator=gen, device=dev).to(bf)
    pout = torch.empty_like(pq)
    dq = torch.randn((decode_seqs, hq, D), generator=gen, device=dev).to(bf)
    dk = torch.randn((decode_seqs, hkv, D), generator=gen, device=dev).to(bf)
    dv = torch.randn((decode_seqs, hkv, D), generator=gen, device=dev).to(bf)
    dout = torch.empty_like(dq)
    ctx_dev = torch.from_numpy(ctx).to(dev)
    scale = 1.0 / math.sqrt(D)
    max_blocks = caches[0]["tables"].shape[1]
    ws = torch.empty(max(16, nvk.decode_attention_workspace_bytes(decode_seqs, hq, hkv, D, max_blocks, BS)), dtype=torch.uint8, device=dev)

    ak, av = torch.cat([pk, dk]), torch.cat([pv, dv])   # single launch: one store for the new K / V of both kinds of rows
    flops_est = prefill_seqs * 4 * hq * D * (prefill_len * (prefill_len + 1) // 2)
    bytes_est = int(ctx.astype(np.int64).sum()) * 2 * hkv * D * 2
    t_p, t_d = flops_est / 0.55e15, bytes_est / 6.8e12   # what each half sustains on its share of the SMs
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    prefill_blocks = prefill_blocks_hint or max(1, int(round(sms * t_p / (t_p + t_d))))

    def step_single():
        for layer in range(layers):
            c = caches[layer % phys]
            nvk.store_kvcache(ak, av, c["k"], c["v"], c["all_slots"])
            nvk.attention_mixed_step(pq, cu, pk, pv, cu, None, pout, dq, ctx_dev, c["tables"], dout, c["k"], c["v"], hkv, D, BS,
                                     scale, ws, prefill_blocks)

    def step():
        for layer in range(layers):
            c = caches[layer % phys]
            nvk.store_kvcache(pk, pv, c["k"], c["v"], c["pslots"])
            nvk.launch_prefill_attention_dense(pq, cu, pk, pv, cu, hkv, D, scale, pout)
            nvk.store_kvcache(dk, dv, c["k"], c["v"], c["dslots"])
            nvk.launch_decode_attention_paged(dq, c["k"], c["v"], ctx_dev, c["tables"], hkv, D, BS, scale, dout, ws)

    mean_ms, med_ms = _time(torch, step_single if single_launch else step, steps, warmup)
    dec_bytes = int(ctx.astype(np.int64).sum()) * 2 * hkv * D * 2 + 2 * decode_seqs * hq * D * 2
    pre_bytes = 2 * total_pq * hq * D * 2 + 2 * total_pq * hkv * D * 2
    store_bytes = 2 * (2 * (total_pq + decode_seqs) * hkv * D * 2)
    bytes_layer = dec_bytes + pre_bytes + store_bytes
    flops_layer = prefill_seqs * 4 * hq * D * (prefill_len * (prefill_len + 1) // 2)
    hbm, tf, kind = _peaks()
    ideal_ms = layers * (dec_bytes / (hbm * 1e9) + flops_layer / (tf * 1e12)) * 1e3
    ach = layers * bytes_layer / (mean_ms * 1e-3) / 1e9
    return {"metric": "mixed_step_attention_hbm_bandwidth", "value": ach, "unit": "GB/s", "n_gpus": 1, "steps": steps,
            "warmup": warmup, "ms_per_step": mean_ms, "median_ms": med_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"mixed continuous-batching step, Qwen3-8B attention shape: {prefill_seqs} prefill sequences x "
                                   f"{prefill_len} new tokens + {decode_seqs} decode sequences with context U[{ctx_lo},{ctx_hi}], "
                                   f"{layers} layers per step",
                       "launches": (f"per layer: one store + one mixed prefill / decode launch ({prefill_blocks} of {sms} blocks start on the "
                                    "prefill items) + the merge of the decode splits"
                                    if single_launch else "per layer: store + dense prefill + store + paged decode (split-K + merge)"),
                       "physical_layer_caches": phys, "bytes_per_layer_cache": bytes_per_layer,
                       "note": "logical layers are mapped round-robin onto the physical caches that fit in HBM",
                       "bytes_per_layer": bytes_layer, "prefill_flops_per_layer": flops_layer,
                       "l2": "each layer cache (GiB) exceeds the 126 MB L2"},
            "roofline": {"bound": "hbm", "kernel": ("prefill_tc5_kernel<T, true> (both halves)" if single_launch else "decode_split_kernel (dominant; the prefill kernel second)"), "achieved": ach,
                         "peak": hbm, "peak_source": f"{kind} copy bandwidth", "unit": "GB/s", "frac": ach / hbm,
                         "ideal_ms_per_step": ideal_ms, "frac_of_ideal_time": ideal_ms / mean_ms, "traffic": None},
            "gpu_launches": steps * layers * (3 if single_launch else 5), "clocks": LAST_CLOCKS}


def bench_decode_tp_shape(nvk, torch, dev, steps, warmup, tp=8, batch=256, layers=36, ctx_lo=100, ctx_hi=2048):
    """Paged decode attention at the per-rank shape of a tensor-parallel decoder (``32 / tp`` query heads, ``8 / tp`` KV heads:
    256-byte cache rows at tp = 8) with the contexts of the end-to-end configuration (prompt U[100,1024] plus up to 1024
    generated tokens), timed as in a decoder: ``layers`` attention calls on ``layers`` distinct caches inside one replayed
    CUDA graph; the figure is the time per layer (split-K kernel + merge)."""
    from . import workloads as wl
    hq, hkv = HQ // tp, HKV // tp
    rng = np.random.default_rng(77)
    ctx = rng.integers(ctx_lo, ctx_hi + 1, size=batch).astype(np.int32)
    width = (2 * 1024 + BS - 1) // BS
    tables, pool = wl.build_block_tables(rng, ctx, BS, pad_to=width)
    bf = torch.bfloat16
    gen = torch.Generator(device=dev)
    gen.manual_seed(77)
    caches = [(torch.empty((pool, BS, hkv, D), device=dev, dtype=bf).normal_(generator=gen),
               torch.empty((pool, BS, hkv, D), device=dev, dtype=bf).normal_(generator=gen)) for _ in range(layers)]
    q = torch.randn((batch, hq, D), generator=gen, device=dev).to(bf)
    out = torch.empty_like(q)
    ctx_dev, tab_dev = torch.from_numpy(ctx).to(dev), torch.from_numpy(tables).to(dev)
    scale = 1.0 / math.sqrt(D)
    ws = torch.empty(max(16, nvk.decode_attention_workspace_bytes(batch, hq, hkv, D, tables.shape[1], BS)), dtype=torch.uint8, device=dev)

    def layer(l):
        nvk.launch_decode_attention_paged(q, caches[l][0], caches[l][1], ctx_dev, tab_dev, hkv, D, BS, scale, out, ws)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer(0)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for l in range(layers):
            layer(l)
    mean_ms, med_ms = _time(torch, graph.replay, steps, warmup)
    eager_ms, _ = _time(torch, lambda: [layer(l) for l in range(layers)], max(3, steps // 4), 2)
    tokens = int(ctx.astype(np.int64).sum())
    used = int(((ctx.astype(np.int64) + BS - 1) // BS).sum())
    nbytes = tokens * hkv * D * 2 * 2 + 2 * batch * hq * D * 2 + 4 * (used + batch)
    hbm, _, kind = _peaks()
    per_layer_ms = mean_ms / layers
    ach = nbytes / (per_layer_ms * 1e-3) / 1e9
    return {"metric": "paged_decode_attention_hbm_bandwidth", "value": ach, "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": per_layer_ms, "median_ms": med_ms / layers, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"paged decode attention at the per-rank shape of tp{tp}: batch {batch}, {hq}/{hkv} heads, head_dim {D}, "
                                   f"block_size {BS}, context U[{ctx_lo},{ctx_hi}], table width {tables.shape[1]}",
                       "context_tokens": tokens, "algorithmic_bytes": nbytes,
                       "l2": f"time per layer of a replayed CUDA graph of {layers} calls on {layers} distinct caches "
                             f"({layers * 2 * pool * BS * hkv * D * 2 >> 20} MB in total: beyond L2)"},
            "eager_ms_per_layer": eager_ms / layers,
            "roofline": {"bound": "hbm", "kernel": "decode_split_kernel + decode_merge_kernel", "achieved": ach, "peak": hbm,
                         "peak_source": f"{kind} copy bandwidth", "unit": "GB/s", "frac": ach / hbm, "traffic": None},
            "gpu_launches": steps * layers * 2, "clocks": LAST_CLOCKS}


def bench_linears(nvk, torch, dev, steps, warmup, rows=256, layers=36):
    """The two linears next to attention at decode size, fused with what follows them, against the sequence they replace.
    Every figure is the time per layer of a replayed CUDA graph that walks ``layers`` distinct weight matrices (so weights
    stream from HBM as in a decoder; together they exceed L2).

    * QKV: ``nvk_qkv_linear_norm_rope_store`` against cuBLAS GEMM + ``nvk_fused_split_norm_rope_store``.
    * plain GEMM core: ``nvk_linear`` against ``torch.matmul`` for the QKV and o_proj shapes.
    """
    bf = torch.bfloat16
    gen = torch.Generator(device=dev)
    gen.manual_seed(11)
    hidden = 4096
    n_qkv = (HQ + 2 * HKV) * D
    max_pos = 4096
    inv_freq = 1.0 / (1.0e6 ** (np.arange(0, D, 2, dtype=np.float32) / D))
    ang = np.arange(max_pos, dtype=np.float32)[:, None] * inv_freq[None, :]
    table = torch.from_numpy(np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)).to(dev)
    pos = torch.randint(0, max_pos, (rows,), generator=gen, device=dev, dtype=torch.int32)
    pool = max(64, (rows + BS - 1) // BS)
    slots = torch.from_numpy(np.random.default_rng(11).permutation(pool * BS)[:rows].astype(np.int32)).to(dev)
    qw = torch.ones(D, device=dev, dtype=bf)
    kw = torch.ones(D, device=dev, dtype=bf)
    x = torch.randn((rows, hidden), generator=gen, device=dev).mul_(0.5).to(bf)
    w_qkv = [torch.randn((n_qkv, hidden), generator=gen, device=dev).mul_(0.02).to(bf) for _ in range(layers)]
    w_o = [torch.randn((hidden, HQ * D), generator=gen, device=dev).mul_(0.02).to(bf) for _ in range(layers)]
    kc = torch.zeros((pool, BS, HKV, D), device=dev, dtype=bf)
    vc = torch.zeros_like(kc)
    q_out = torch.empty((rows, HQ, D), device=dev, dtype=bf)
    qkv = torch.empty((rows, n_qkv), device=dev, dtype=bf)
    o_in = torch.randn((rows, HQ * D), generator=gen, device=dev).mul_(0.5).to(bf)
    o_out = torch.empty((rows, hidden), device=dev, dtype=bf)

    def fused_qkv(l):
        nvk.qkv_linear_norm_rope_store(x, w_qkv[l], pos, qw, kw, 1e-6, table, slots, kc, vc, HQ, HKV, D, q_out)

    def unfused_qkv(l):
        torch.matmul(x, w_qkv[l].t(), out=qkv)
        nvk.fused_split_norm_rope_store(qkv, pos, qw, kw, 1e-6, table, slots, kc, vc, HQ, HKV, D, q_out)

    cases = {
        "qkv_fused": fused_qkv,
        "qkv_cublas_then_prologue": unfused_qkv,
        "qkv_gemm_nvk_linear": lambda l: nvk.linear(x, w_qkv[l], qkv),
        "qkv_gemm_cublas": lambda l: torch.matmul(x, w_qkv[l].t(), out=qkv),
        "o_proj_gemm_nvk_linear": lambda l: nvk.linear(o_in, w_o[l], o_out),
        "o_proj_gemm_cublas": lambda l: torch.matmul(o_in, w_o[l].t(), out=o_out),
    }
    out = {}
    clocks = None
    for name, fn in cases.items():
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn(0)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for l in range(layers):
                fn(l)
        mean_ms, med_ms = _time(torch, graph.replay, steps, warmup)
        clocks = LAST_CLOCKS
        wbytes = (n_qkv if name.startswith("qkv") else hidden) * hidden * 2
        out[name] = {"us_per_layer": mean_ms * 1e3 / layers, "median_us_per_layer": med_ms * 1e3 / layers,
                     "weight_GBps": wbytes / (mean_ms * 1e-3 / layers) / 1e9}
        del graph
    status = nvk.gemm_status()
    hbm, _, kind = _peaks()
    best = out["qkv_fused"]
    nbytes = n_qkv * hidden * 2 + rows * hidden * 2 + rows * (HQ + 2 * HKV) * D * 2
    ach = nbytes / (best["us_per_layer"] * 1e-6) / 1e9
    return {"metric": "qkv_linear_norm_rope_store_hbm_bandwidth", "value": ach, "unit": "GB/s", "n_gpus": 1, "steps": steps,
            "warmup": warmup, "ms_per_step": best["us_per_layer"] * 1e-3, "median_ms": best["median_us_per_layer"] * 1e-3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"QKV projection ({hidden} -> {n_qkv}) + split + q/k RMSNorm + RoPE + KV store as one launch, {rows} rows",
                       "l2": f"time per layer of a replayed CUDA graph over {layers} distinct weight matrices ({layers * n_qkv * hidden * 2 >> 20} MB: beyond L2)"},
            "cases": out, "gemm_status": status,
            "roofline": {"bound": "hbm", "kernel": "gemm_tc_kernel<T, qkv prologue epilogue>", "achieved": ach, "peak": hbm,
                         "peak_source": f"{kind} copy bandwidth", "unit": "GB/s", "frac": ach / hbm, "traffic": None},
            "gpu_launches": steps * layers * len(cases), "clocks": clocks}


def other_kernels(nvk, torch, dev, steps=20, warmup=3):
    """Short runs of the kernels beside paged decode, for the default benchmark line: the prefill configuration
    (tensor roofline), store_kvcache at prefill size, the fused prologue at decode and prefill row counts, decode over
    the int8 cache.  Each entry: ms per launch, algorithmic bytes or flops, fraction of the measured peak, clocks."""
    out = {}

    def brief(line, extra=()):
        r = line["roofline"]
        e = {"ms": line["ms_per_step"], "median_ms": line.get("median_ms"), "achieved": r["achieved"], "unit": r["unit"],
             "peak": r["peak"], "frac": r["frac"], "bound": r["bound"], "workload": line["config"]["workload"],
             "clocks": line.get("clocks")}
        for k in extra:
            e[k] = line[k] if k in line else r.get(k)
        return e

    line = bench_prefill(nvk, torch, dev, steps, warmup)
    out["prefill"] = brief(line)
    out["prefill"].update({"flops": line["config"]["flops_per_step"], "frac_of_sustained": line["roofline"]["frac_of_sustained"],
                           "frac_of_nominal_2250": line["roofline"]["frac_of_nominal_2250"]})
    torch.cuda.empty_cache()
    line = bench_prefill(nvk, torch, dev, steps, warmup, num_seqs=32, q_lo=512, q_hi=512, prefix_frac=0.0)
    out["prefill_32x512"] = brief(line)
    out["prefill_32x512"]["flops"] = line["config"]["flops_per_step"]
    torch.cuda.empty_cache()
    line = bench_store(nvk, torch, dev, steps, warmup)
    out["store_kvcache_36864_tokens"] = brief(line, extra=("block_contiguous_slots", "same_size_contiguous_copy"))
    for rows in (256, 16384):
        line = bench_prologue(nvk, torch, dev, steps, warmup, rows=rows)
        out[f"fused_prologue_{rows}_rows"] = brief(line, extra=("same_size_contiguous_copy",))
    torch.cuda.empty_cache()
    line = bench_decode_int8(nvk, torch, dev, steps, warmup)
    out["decode_int8_kv"] = brief(line, extra=("bf16_cache_same_shape", "store_kvcache_int8"))
    torch.cuda.empty_cache()
    line = bench_decode_int8(nvk, torch, dev, steps, warmup, fmt="fp8")
    out["decode_fp8_kv"] = brief(line, extra=("bf16_cache_same_shape", "store_kvcache_fp8"))
    torch.cuda.empty_cache()
    line = bench_decode_tp_shape(nvk, torch, dev, steps, warmup)
    out["decode_tp8_rank_shape_in_graph"] = brief(line, extra=("eager_ms_per_layer",))
    torch.cuda.empty_cache()
    line = bench_linears(nvk, torch, dev, min(steps, 10), warmup)
    out["qkv_linear_fused_prologue_256_rows"] = brief(line, extra=("cases",))
    torch.cuda.empty_cache()
    return out
