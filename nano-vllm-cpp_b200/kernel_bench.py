"""Single-GPU measurements of the kernels beside paged decode: varlen prefill, store_kvcache at
prefill size and the fused decode prologue.  ``bench.py --workload {prefill,store,prologue}`` prints
one JSON line per run in the same layout as the decode benchmark (metric / value / roofline).

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


def _time(torch, fn, steps, warmup, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in evs:
        if flush is not None:
            flush()
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
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


def bench_prefill(nvk, torch, dev, steps, warmup, num_seqs=16, q_lo=512, q_hi=4096):
    w = make_prefill_inputs(torch, dev, 2025, num_seqs, q_lo, q_hi)
    nvk.store_kvcache(w["k_new"], w["v_new"], w["k_cache"], w["v_cache"], w["slot_mapping"])

    def attn():
        nvk.launch_prefill_attention_paged(w["q"], w["cu_q"], w["k_cache"], w["v_cache"], w["cu_k"],
                                           w["block_tables"], HKV, D, BS, w["scale"], w["out"])

    def store():
        nvk.store_kvcache(w["k_new"], w["v_new"], w["k_cache"], w["v_cache"], w["slot_mapping"])

    mean_ms, med_ms = _time(torch, attn, steps, warmup)
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
                               "half with a 256-1024-token paged prefix, keys read through block_tables",
                   "total_q": total_q, "flops_per_step": w["flops"],
                   "l2": "q/out (2 x %.0f MB) exceed the 126 MB L2" % (total_q * HQ * D * 2 / 1e6)},
        "roofline": {"bound": "tensor", "kernel": "prefill kernel", "achieved": achieved, "peak": tf,
                     "peak_source": f"{kind} cuBLAS bf16 burst", "unit": "TFLOP/s", "frac": achieved / tf,
                     "frac_of_nominal_2250": achieved / 2250.0, "traffic": None},
        "store_kvcache": {"ms": st_mean, "bytes": store_bytes, "GBps": store_bytes / (st_mean * 1e-3) / 1e9,
                          "frac_of_" + kind + "_hbm": store_bytes / (st_mean * 1e-3) / 1e9 / hbm},
        "gpu_launches": 2 * steps,
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
    return {"metric": "store_kvcache_hbm_bandwidth", "value": ach, "unit": "GB/s", "n_gpus": 1, "steps": steps,
            "warmup": warmup, "ms_per_step": mean_ms, "median_ms": med_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": f"store_kvcache of {tokens} tokens x 8 KV heads x 128 bf16 into random slots",
                       "l2": "a 256 MB buffer is written between timed iterations"},
            "roofline": {"bound": "hbm", "kernel": "store_rows_kernel", "achieved": ach, "peak": hbm,
                         "peak_source": f"{kind} copy bandwidth", "unit": "GB/s", "frac": ach / hbm, "traffic": None},
            "gpu_launches": steps}


def bench_prologue(nvk, torch, dev, steps, warmup, rows=256):
    gen = torch.Generator(device=dev)
    gen.manual_seed(9)
    bf = torch.bfloat16
    qkv = torch.randn((rows, (HQ + 2 * HKV) * D), generator=gen, device=dev).to(bf)
    qw = torch.ones(D, device=dev, dtype=bf)
    kw = torch.ones(D, device=dev, dtype=bf)
    max_pos = 4096
    inv_freq = 1.0 / (1.0e6 ** (np.arange(0, D, 2, dtype=np.float32) / D))
    ang = np.arange(max_pos, dtype=np.float32)[:, None] * inv_freq[None, :]
    table = torch.from_numpy(np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)).to(dev)
    pos = torch.randint(0, max_pos, (rows,), generator=gen, device=dev, dtype=torch.int32)
    pool = 64
    kc = torch.zeros((pool, BS, HKV, D), device=dev, dtype=bf)
    vc = torch.zeros_like(kc)
    slots = torch.from_numpy(np.random.default_rng(9).permutation(pool * BS)[:rows].astype(np.int32)).to(dev)
    q_out = torch.empty((rows, HQ, D), device=dev, dtype=bf)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    fn = lambda: nvk.fused_split_norm_rope_store(qkv, pos, qw, kw, 1e-6, table, slots, kc, vc, HQ, HKV, D, q_out)  # noqa: E731
    mean_ms, med_ms = _time(torch, fn, steps, warmup, flush=lambda: flush_buf.fill_(1))
    nbytes = 2 * rows * (HQ + 2 * HKV) * D * 2 + rows * (D * 4 + 8)
    hbm, _, kind = _peaks()
    ach = nbytes / (mean_ms * 1e-3) / 1e9
    return {"metric": "fused_split_norm_rope_store_hbm_bandwidth", "value": ach, "unit": "GB/s", "n_gpus": 1,
            "steps": steps, "warmup": warmup, "ms_per_step": mean_ms, "median_ms": med_ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"fused split + q/k RMSNorm + RoPE + KV store, {rows} rows of 48 heads x 128",
                       "l2": "a 256 MB buffer is written between timed iterations"},
            "roofline": {"bound": "hbm", "kernel": "fused_prologue_kernel", "achieved": ach, "peak": hbm,
                         "peak_source": f"{kind} copy bandwidth", "unit": "GB/s", "frac": ach / hbm, "traffic": None},
            "gpu_launches": steps}
