#!/usr/bin/env python
"""Benchmark of the paged-KV decode hot path (store_kvcache + paged decode attention).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload at every N: the Qwen3-8B decode configuration -- 32 query heads, 8 KV heads, head_dim 128,
bf16 paged KV cache with 256-token blocks, batch 256, context lengths uniform in [1024, 8192], block
tables a seeded random permutation of a pool sized for the batch, N(0,1) values, scale 1/sqrt(128).
One step = store_kvcache of the 256 new tokens + paged decode attention over the whole batch.  With
N > 1 every rank owns an independent batch of the same shape (no data-path collective; weak scaling).

``value`` is algorithmic HBM bytes per second with all inputs resident in HBM; ``e2e`` is the same
quantity when each step also uploads its inputs (q / k / v of the new tokens and the step metadata)
from pinned host memory and reads the attention output back.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
import datetime
import json
import math
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

METRIC = "paged_decode_attention_hbm_bandwidth"
UNIT = "GB/s"
CFG = dict(batch=256, num_heads=32, num_kv_heads=8, head_dim=128, block_size=256, ctx_lo=1024, ctx_hi=8192)
# dram__bytes_read.sum + dram__bytes_write.sum of one decode_split_kernel launch divided by its algorithmic bytes, from
# an ncu capture of a batch-32 case of this workload (a full batch is too large to capture; traffic scales with KV bytes).
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.010


def workload_name():
    """The same string in both arms' ``config.workload``."""
    return (f"paged decode attention + store_kvcache, Qwen3-8B shape: batch {CFG['batch']} per GPU, "
            f"{CFG['num_heads']}/{CFG['num_kv_heads']} heads per GPU, head_dim {CFG['head_dim']}, block_size {CFG['block_size']}, "
            f"context U[{CFG['ctx_lo']},{CFG['ctx_hi']}], random-permutation block tables")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


from benchmarks.clocks import ClockSampler, physical_gpu_index  # noqa: E402


def make_workload(torch, dev, seed):
    """Builds the decode configuration on the device (values drawn on the GPU from a seeded generator)."""
    from benchmarks import workloads as wl
    rng = np.random.default_rng(seed)
    ctx = rng.integers(CFG["ctx_lo"], CFG["ctx_hi"] + 1, size=CFG["batch"]).astype(np.int32)
    tables, pool = wl.build_block_tables(rng, ctx, CFG["block_size"])
    last = ctx.astype(np.int64) - 1
    slots = (tables[np.arange(CFG["batch"]), last // CFG["block_size"]].astype(np.int64) * CFG["block_size"]
             + last % CFG["block_size"]).astype(np.int32)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    bf = torch.bfloat16
    shape = (pool, CFG["block_size"], CFG["num_kv_heads"], CFG["head_dim"])
    w = {
        "context_lens_np": ctx, "block_tables_np": tables, "slot_mapping_np": slots, "pool": pool,
    }
    # draw the large caches block-wise to bound the fp32 temporary
    for name in ("k_cache", "v_cache"):
        t = torch.empty(shape, device=dev, dtype=bf)
        step = 256
        for i in range(0, pool, step):
            n = min(step, pool - i)
            t[i:i + n] = torch.randn((n,) + shape[1:], generator=gen, device=dev, dtype=torch.float32).to(bf)
        w[name] = t
    w["q"] = torch.randn((CFG["batch"], CFG["num_heads"], CFG["head_dim"]), generator=gen, device=dev).to(bf)
    w["k_new"] = torch.randn((CFG["batch"], CFG["num_kv_heads"], CFG["head_dim"]), generator=gen, device=dev).to(bf)
    w["v_new"] = torch.randn((CFG["batch"], CFG["num_kv_heads"], CFG["head_dim"]), generator=gen, device=dev).to(bf)
    w["context_lens"] = torch.from_numpy(ctx).to(dev)
    w["block_tables"] = torch.from_numpy(tables).to(dev)
    w["slot_mapping"] = torch.from_numpy(slots).to(dev)
    w["out"] = torch.empty_like(w["q"])
    w["scale"] = 1.0 / math.sqrt(CFG["head_dim"])
    return w


def algorithmic_bytes(ctx, tables):
    """Bytes one step must move: K and V of every context token once per KV head, q and out, the
    metadata actually dereferenced, and the store's read + write of the new rows."""
    hkv, d, hq, b = CFG["num_kv_heads"], CFG["head_dim"], CFG["num_heads"], CFG["batch"]
    kv = int(ctx.astype(np.int64).sum()) * 2 * hkv * d * 2
    q_out = 2 * b * hq * d * 2
    used_entries = int(((ctx.astype(np.int64) + CFG["block_size"] - 1) // CFG["block_size"]).sum())
    meta = used_entries * 4 + b * 4
    store = 2 * (2 * b * hkv * d * 2) + b * 4
    return {"decode": kv + q_out + meta, "store": store, "total": kv + q_out + meta + store}


def cpu_baseline(torch, w, budget_s=12.0):
    """Times the CPU oracle (fp32 restatement of the reference's decode kernel) on a bounded sample:
    the first n sequences of the batch, all heads, all host threads."""
    import oracle
    ctx, tables = w["context_lens_np"], w["block_tables_np"]
    threads = oracle.default_threads()

    def prepare(n):
        blocks = []
        remap = np.zeros((n, tables.shape[1]), dtype=np.int32)
        for b in range(n):
            nb = (int(ctx[b]) + CFG["block_size"] - 1) // CFG["block_size"]
            for j in range(nb):
                remap[b, j] = len(blocks)
                blocks.append(int(tables[b, j]))
        idx = torch.tensor(blocks, device=w["k_cache"].device)
        kc = w["k_cache"][idx].float().cpu().numpy()
        vc = w["v_cache"][idx].float().cpu().numpy()
        q = w["q"][:n].float().cpu().numpy()
        nbytes = int(ctx[:n].astype(np.int64).sum()) * 2 * CFG["num_kv_heads"] * CFG["head_dim"] * 2

        def once():
            t0 = time.perf_counter()
            oracle.decode_attention_paged(q, kc, vc, ctx[:n], remap, CFG["num_kv_heads"], CFG["head_dim"],
                                          CFG["block_size"], w["scale"], threads=threads)
            return time.perf_counter() - t0, nbytes
        return once

    n = min(CFG["batch"], 32)
    run_once = prepare(n)
    run_once()  # warm-up (page faults, thread pool)
    dt, reps, nbytes = 0.0, 0, 0
    while dt < budget_s:
        t, nb = run_once()
        dt += t
        nbytes += nb
        reps += 1
    return {"value": nbytes / dt / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"first {n} of {CFG['batch']} sequences, all {CFG['num_heads']} heads, {reps} passes of the fp32 "
                      f"oracle in {dt:.1f} s; bytes counted at the workload's bf16 element size",
            "qwen3_0p6b_decode_fp32": cpu_reference_config(oracle)}


def cpu_reference_config(oracle, budget_s=4.0):
    """The CPU-runnable configuration, timed on the host cores: single-layer paged decode at the Qwen3-0.6B shape -- 16
    query heads, 8 KV heads, head_dim 128, fp32, batch 8, block_size 256, contexts U[64,1024], q pre-scaled by
    1/sqrt(128) (softmax scale 1), block tables from a seeded permutation of a 64-block pool, the new token stored
    first.  One thread and all threads; bytes are the fp32 K and V actually read."""
    from benchmarks import workloads as wl
    ctx = np.random.default_rng(1234).integers(64, 1025, size=8)
    need = int(((ctx + 255) // 256).sum())
    w = wl.make_decode_workload(batch=8, num_heads=16, num_kv_heads=8, head_dim=128, block_size=256, ctx_lo=64, ctx_hi=1024,
                                seed=1234, value_scale=0.5, prescale_q=True, rounded=False, extra_pool_blocks=64 - need,
                                context_lens=ctx)
    kc, vc = w["k_cache"].copy(), w["v_cache"].copy()
    nbytes = int(w["context_lens"].astype(np.int64).sum()) * 2 * 8 * 128 * 4
    out = {"workload": "16/8 heads, head_dim 128, fp32, batch 8, block_size 256, context U[64,1024], 64-block pool",
           "algorithmic_bytes_per_step": nbytes, "unit": UNIT, "host_threads_available": oracle.default_threads()}
    for label, threads in (("single_thread", 1), ("all_threads", oracle.default_threads())):
        best, spent = float("inf"), 0.0
        while spent < budget_s / 2:
            t0 = time.perf_counter()
            oracle.store_kvcache(w["k_new"], w["v_new"], kc, vc, w["slot_mapping"])
            oracle.decode_attention_paged(w["q"], kc, vc, w["context_lens"], w["block_tables"], 8, 128, 256, w["scale"], threads=threads)
            dt = time.perf_counter() - t0
            best, spent = min(best, dt), spent + dt
        out[label] = {"threads": threads, "ms_per_step": best * 1e3, "value": nbytes / best / 1e9}
    return out


def rank_plan(rank, world, shard):
    """What one rank works on.  ``batch``: an independent batch per rank (same shape, own seed; weak scaling).
    ``kv_heads``: tensor-parallel layout of the reference (src/models/transformer.cpp:75-80) -- every rank holds
    Hkv / world KV heads and their query heads for the SAME sequences, so the step metadata is replicated (same
    seed) and the total work is fixed (strong scaling).  Neither layout needs a collective inside attention."""
    if shard == "kv_heads":
        if CFG["num_kv_heads"] % world != 0:
            raise ValueError("num_kv_heads must be divisible by the number of GPUs")
        return {"seed": 2024, "num_heads": CFG["num_heads"] // world, "num_kv_heads": CFG["num_kv_heads"] // world,
                "scaling": "strong", "parallelism": f"tp{world}: {CFG['num_kv_heads'] // world} KV heads per GPU, replicated metadata, no collective"}
    return {"seed": 2024 + rank, "num_heads": CFG["num_heads"], "num_kv_heads": CFG["num_kv_heads"], "scaling": "weak",
            "parallelism": f"{world} independent batches, one per GPU, no collective"}


def combine_ranks(torch, dist, world, device, times_ms, sums):
    """Max over ranks of every timing, sum over ranks of every additive quantity (bytes, launches)."""
    if world <= 1:
        return list(times_ms), list(sums)
    t = torch.tensor(list(times_ms), device=device, dtype=torch.float64)
    u = torch.tensor(list(sums), device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(u, op=dist.ReduceOp.SUM)
    return [float(x) for x in t], [float(x) for x in u]


def run_ours(args, torch, dist, rank, world, dev):
    nvk = entry.load_package()
    nvk.lib()  # raises if the CUDA library is missing: there is no fallback
    plan = rank_plan(rank, world, args.shard)
    CFG["num_heads"], CFG["num_kv_heads"] = plan["num_heads"], plan["num_kv_heads"]
    w = make_workload(torch, dev, seed=plan["seed"])
    ab = algorithmic_bytes(w["context_lens_np"], w["block_tables_np"])
    ws_bytes = nvk.decode_attention_workspace_bytes(CFG["batch"], CFG["num_heads"], CFG["num_kv_heads"],
                                                    CFG["head_dim"], w["block_tables"].shape[1], CFG["block_size"])
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)

    def store():
        nvk.store_kvcache(w["k_new"], w["v_new"], w["k_cache"], w["v_cache"], w["slot_mapping"])

    def decode():
        nvk.launch_decode_attention_paged(w["q"], w["k_cache"], w["v_cache"], w["context_lens"], w["block_tables"],
                                          CFG["num_kv_heads"], CFG["head_dim"], CFG["block_size"], w["scale"],
                                          w["out"], ws)

    def barrier():
        if world > 1:
            dist.barrier()

    for _ in range(args.warmup):
        store()
        decode()
    torch.cuda.synchronize()

    # ---- timed region: K steps, device-resident inputs --------------------------------------------
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ka = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    kb = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    sampler = ClockSampler(physical_gpu_index(int(os.environ.get("LOCAL_RANK", 0))))
    launches_before = nvk.launch_count
    barrier()
    torch.cuda.synchronize()
    sampler.start()
    ev0.record()
    for i in range(args.steps):
        store()
        ka[i].record()
        decode()
        kb[i].record()
    ev1.record()
    torch.cuda.synchronize()
    barrier()
    clocks = sampler.finish()
    launches = nvk.launch_count - launches_before
    total_ms = ev0.elapsed_time(ev1)
    decode_ms = sum(a.elapsed_time(b) for a, b in zip(ka, kb)) / args.steps

    # ---- end to end: host buffers in, host buffer out, every step ---------------------------------
    host = {k: w[k].cpu().pin_memory() for k in ("q", "k_new", "v_new", "slot_mapping", "context_lens", "block_tables")}
    out_host = torch.empty(w["out"].shape, dtype=w["out"].dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = out_host.numel() * out_host.element_size()

    def e2e_step():
        for k, t in host.items():
            w[k].copy_(t, non_blocking=True)
        store()
        decode()
        out_host.copy_(w["out"], non_blocking=True)
        torch.cuda.synchronize()

    # Pipelined form of the same step (what a serving loop does): two sets of device input / output buffers, the copies of
    # step i + 1 run on a copy stream under the kernels of step i, the result of step i leaves on a third stream.
    # Every step still uploads all its inputs from pinned host memory and downloads its result inside the timed region.
    names = list(host.keys())
    dev_in = [{k: torch.empty_like(w[k]) for k in names} for _ in range(2)]
    dev_out = [torch.empty_like(w["out"]) for _ in range(2)]
    host_out = [torch.empty(w["out"].shape, dtype=w["out"].dtype).pin_memory() for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    s_run = torch.cuda.current_stream(dev)

    def e2e_pipelined(steps, first_event, last_event):
        in_ready = [torch.cuda.Event() for _ in range(2)]
        run_done = [torch.cuda.Event() for _ in range(2)]
        out_done = [torch.cuda.Event() for _ in range(2)]
        with torch.cuda.stream(s_in):
            first_event.record()
        for i in range(steps):
            b = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(run_done[b])           # the kernels of step i - 2 are done with this input set
                for k in names:
                    dev_in[b][k].copy_(host[k], non_blocking=True)
                in_ready[b].record()
            s_run.wait_event(in_ready[b])
            if i >= 2:
                s_run.wait_event(out_done[b])               # the result of step i - 2 has left this output buffer
            d = dev_in[b]
            nvk.store_kvcache(d["k_new"], d["v_new"], w["k_cache"], w["v_cache"], d["slot_mapping"])
            nvk.launch_decode_attention_paged(d["q"], w["k_cache"], w["v_cache"], d["context_lens"], d["block_tables"],
                                              CFG["num_kv_heads"], CFG["head_dim"], CFG["block_size"], w["scale"], dev_out[b], ws)
            run_done[b].record()
            with torch.cuda.stream(s_out):
                s_out.wait_event(run_done[b])
                host_out[b].copy_(dev_out[b], non_blocking=True)
                out_done[b].record()
        with torch.cuda.stream(s_out):
            last_event.record()
        torch.cuda.synchronize()

    e2e_ms = serial_ms = float("nan")
    if not args.no_e2e:
        for _ in range(max(3, args.warmup // 4)):
            e2e_step()
        barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        barrier()
        serial_ms = e0.elapsed_time(e1)
        e2e_pipelined(4, torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        barrier()
        torch.cuda.synchronize()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_pipelined(args.steps, p0, p1)
        barrier()
        e2e_ms = p0.elapsed_time(p1)
        if not torch.equal(host_out[(args.steps - 1) & 1], out_host):
            raise RuntimeError("pipelined end-to-end step produced a different result than the serial one")

    per_rank = gather_per_rank(torch, dist, world, dev, {
        "ms_per_step": total_ms / args.steps, "decode_ms_per_launch": decode_ms, "bytes_per_step": float(ab["total"]),
        "context_tokens": float(w["context_lens_np"].astype(np.int64).sum()), "sm_mhz": float(clocks["sm_mhz"] or 0.0)})
    own_decode_ms = decode_ms
    (total_ms, e2e_ms, decode_ms, serial_ms), (bytes_all, launches) = combine_ranks(
        torch, dist, world, dev, [total_ms, e2e_ms, decode_ms, serial_ms], [float(ab["total"]), float(launches)])
    launches = int(launches)

    peak, peak_kind = measured_peaks()
    achieved = ab["decode"] / (own_decode_ms * 1e-3) / 1e9      # rank 0's own bytes over rank 0's own launch time
    line = {
        "metric": METRIC, "value": bytes_all * args.steps / (total_ms * 1e-3) / 1e9, "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
        "higher_is_better": True, "scaling": plan["scaling"], "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(),
                   "bytes_per_step_per_gpu": ab["total"], "kv_pool_blocks": w["pool"],
                   "l2": "inputs (about 4.8 GB of KV per step) exceed the 126 MB L2; no flush needed",
                   "parallelism": plan["parallelism"]},
        "e2e": {"value": bytes_all * args.steps / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps,
                "pipelining": "copies of step i+1 run on a copy stream under the kernels of step i (two device buffer sets); every "
                              "step uploads all its inputs from pinned host memory and downloads its result inside the timed region",
                "serial_value": bytes_all * args.steps / (serial_ms * 1e-3) / 1e9, "serial_ms_per_step": serial_ms / args.steps},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "kernel": "decode_split_kernel (+ decode_merge_kernel)", "achieved": achieved,
                     "peak": peak, "peak_source": f"{peak_kind} copy bandwidth", "unit": UNIT, "frac": achieved / peak,
                     "frac_of_nominal_8TBs": achieved / 8000.0, "ms_per_launch": own_decode_ms,
                     "algorithmic_bytes_per_launch": ab["decode"],
                     "traffic": (NCU_TRAFFIC_PER_ALGORITHMIC_BYTE * ab["decode"]
                                 if NCU_TRAFFIC_PER_ALGORITHMIC_BYTE else None)},
        "clocks": clocks,
    }
    if world > 1:
        # every rank's own figures: ranks draw different context lengths (seed 2024 + rank), so bytes differ by a few per
        # cent; `value` divides the sum of bytes by the slowest rank's time, `sum_of_rank_rates` adds bytes_r / t_r
        line["per_rank"] = per_rank
        line["sum_of_rank_rates"] = sum(b / (t * 1e-3) / 1e9 for b, t in zip(per_rank["bytes_per_step"], per_rank["ms_per_step"]))
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(torch, w)
    # free the decode workload before anything else is measured in this process
    del dev_in, dev_out, host_out, host, out_host, ws
    w.clear()
    torch.cuda.empty_cache()
    if world == 1 and not args.no_other_kernels:
        from benchmarks import kernel_bench as kb
        line["other_kernels"] = kb.other_kernels(nvk, torch, dev)
        line["gpu_launches_other_kernels"] = "not counted in gpu_launches (outside the timed region)"
    # at N = 1 too: the metric asks for output tokens per second at 1, 2, 4 and 8 GPUs (profiling runs, which pass
    # --no-other-kernels, measure the decode step alone)
    if not args.no_tp_e2e and (world > 1 or not args.no_other_kernels):
        line["tp_e2e"] = tp_e2e(args, nvk, torch, dist, rank, world, dev)
    return line


def tp_e2e(args, nvk, torch, dist, rank, world, dev):
    """The second half of the metric: output tokens per second of the end-to-end Qwen3-8B-shaped decoder, tensor-parallel
    over the N GPUs of this run (KV-head shards; all-reduce after o_proj / down_proj through this library's peer-memory
    kernel in the decode steps).  Returns the figures of benchmarks/e2e_bench.run_e2e, or the error that stopped it."""
    from benchmarks import e2e_bench as eb, e2e_model as em
    sampler = ClockSampler(physical_gpu_index(int(os.environ.get("LOCAL_RANK", 0))))
    sampler.start()
    try:
        full = eb.run_e2e(nvk, torch, dist, rank, world, dev, em.DecoderConfig(layers=args.e2e_layers), num_seqs=args.e2e_seqs,
                          len_lo=min(100, args.e2e_maxlen), len_hi=args.e2e_maxlen, use_graph=True, kv_dtype="bf16",
                          allreduce=args.e2e_allreduce)
    except Exception as exc:   # reported, not fatal: the decode figures of this line stand on their own
        sampler.finish()
        return {"error": f"{type(exc).__name__}: {exc}"}
    keep = ("metric", "value", "unit", "ms_per_step", "scaling", "output_tokens", "prompt_tokens", "total_s", "prefill_s", "decode_s",
            "attention_ms_per_decode_step", "peer_allreduce_status", "prefill_status", "gpu_launches")
    out = {k: full.get(k) for k in keep}
    out["config"] = full["config"]
    out["clocks"] = sampler.finish()
    return out


def gather_per_rank(torch, dist, world, device, values: dict) -> dict:
    """{name: [value of rank 0, value of rank 1, ...]} for a dict of floats."""
    names = sorted(values)
    mine = torch.tensor([float(values[k]) for k in names], device=device, dtype=torch.float64)
    if world <= 1:
        return {k: [float(v)] for k, v in zip(names, mine.tolist())}
    rows = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(rows, mine)
    return {k: [float(r[i]) for r in rows] for i, k in enumerate(names)}


def run_reference(args, torch, dist, rank, world, dev):
    """Reference arm: the reference's own CUDA kernels (store_kvcache + decode_paged_attention_kernel, compiled
    unmodified for sm_100a into oracle/_ref) on the same workload, one rank per GPU with the aggregation of the other arm
    (every rank its own batch, seed 2024 + rank; slowest rank's time, sum of bytes).  The reference has no CPU
    implementation of this path; if the compiled reference is absent the CPU oracle port is timed on rank 0."""
    w = make_workload(torch, dev, seed=2024 + rank)
    ab = algorithmic_bytes(w["context_lens_np"], w["block_tables_np"])
    ref_path = os.path.join(ROOT, "oracle", "_ref", "libnvk_ref.so")
    steps = min(args.steps, 50)   # the reference kernel is two orders of magnitude slower per step
    base = {"impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": world, "steps": steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "data": "synthetic", "config": {"workload": workload_name(), "parallelism": f"{world} independent batches, one per GPU, no collective"}}
    if not os.path.exists(ref_path):
        if rank != 0:
            return None
        cb = cpu_baseline(torch, w, budget_s=20.0)
        base.update({"value": cb["value"], "ms_per_step": None, "dtype": "f32", "cpu_baseline": cb, "n_gpus": 0,
                     "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        return base
    ref = ctypes.CDLL(ref_path)
    ref.nvkref_last_error.restype = ctypes.c_char_p
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    row = CFG["num_kv_heads"] * CFG["head_dim"]

    def step():
        rc = ref.nvkref_store_kvcache(P(w["k_new"]), P(w["v_new"]), P(w["k_cache"]), P(w["v_cache"]),
                                      P(w["slot_mapping"]), 3, ctypes.c_int64(CFG["batch"]), ctypes.c_int64(row),
                                      ctypes.c_int64(w["pool"] * CFG["block_size"]), 1, stream)
        rc |= ref.nvkref_decode_attention_paged(
            P(w["q"]), P(w["k_cache"]), P(w["v_cache"]), P(w["context_lens"]), P(w["block_tables"]),
            ctypes.c_int64(CFG["batch"]), ctypes.c_int64(w["block_tables"].shape[1]), ctypes.c_int64(w["pool"]),
            CFG["num_heads"], CFG["num_kv_heads"], CFG["head_dim"], CFG["block_size"], ctypes.c_float(w["scale"]),
            P(w["out"]), 1, stream)
        if rc:
            raise RuntimeError(ref.nvkref_last_error().decode())

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(physical_gpu_index(int(os.environ.get("LOCAL_RANK", 0))))
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.finish()
    (ms,), (bytes_all,) = combine_ranks(torch, dist, world, dev, [ev0.elapsed_time(ev1)], [float(ab["total"])])
    value = bytes_all * steps / (ms * 1e-3) / 1e9
    base.update({
        "value": value, "ms_per_step": ms / steps, "dtype": "bf16", "gpu_launches": 2 * steps * world, "clocks": clocks,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": 0, "kind": "reference",
                         "sample": "full workload; the reference implements this path only as CUDA kernels, so its "
                                   "own kernels (compiled for sm_100a) run on the GPU, not on host cores"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    return base


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer pass (profiling runs)")
    ap.add_argument("--no-other-kernels", action="store_true", help="N = 1: measure the paged-decode step alone (skips the short runs of the other kernels and the decoder run)")
    ap.add_argument("--no-tp-e2e", action="store_true", help="skip the end-to-end decoder run (tensor-parallel over the N GPUs of the run)")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "store", "prologue", "mixed", "e2e", "decode_int8", "decode_fp8", "linears", "decode_tp"],
                    help="decode is the benchmark; prefill / store / prologue / mixed / decode_int8 time the remaining kernels of the path "
                         "(1 GPU); e2e reports output tokens per second of the whole decoder, tensor-parallel over --gpus")
    ap.add_argument("--e2e-layers", type=int, default=36, help="e2e workload: decoder layers (36 = the named model)")
    ap.add_argument("--e2e-seqs", type=int, default=256, help="e2e workload: number of sequences")
    ap.add_argument("--e2e-maxlen", type=int, default=1024, help="e2e workload: longest prompt / output")
    ap.add_argument("--no-graph", action="store_true", help="e2e workload: run decode steps eagerly")
    ap.add_argument("--e2e-kv", default="bf16", choices=["bf16", "int8", "fp8"], help="e2e workload: KV cache format")
    ap.add_argument("--e2e-linears", default="cublas", choices=["cublas", "fused"],
                    help="e2e workload: decode-step QKV / o_proj / down_proj as cuBLAS GEMMs + kernels, or this library's fused GEMMs")
    ap.add_argument("--e2e-allreduce", default="auto", choices=["auto", "nccl", "peer", "multimem"],
                    help="e2e workload, N > 1: all-reduce of the decode steps through NCCL, the peer-memory kernel or the in-switch "
                         "(multimem) kernel; auto = peer")
    ap.add_argument("--shard", default="batch", choices=["batch", "kv_heads"],
                    help="N > 1: independent batch per GPU (weak scaling) or KV-head tensor-parallel shards (strong)")
    ap.add_argument("--layers", type=int, default=36, help="mixed workload: layer caches per step")
    ap.add_argument("--rows", type=int, default=256, help="prologue workload: token rows")
    ap.add_argument("--mixed-single-launch", action="store_true",
                    help="mixed workload: one attention launch per layer for prefill and decode rows together (nvk_attention_mixed_step)")
    ap.add_argument("--mixed-prefill-blocks", type=int, default=0, help="mixed single launch: blocks that start on the prefill items (0 = from the sizes)")
    ap.add_argument("--seqs", type=int, default=16, help="prefill workload: number of sequences")
    ap.add_argument("--qmax", type=int, default=4096, help="prefill workload: longest new-token run")
    ap.add_argument("--batch", type=int, default=CFG["batch"],
                    help="sequences per GPU; anything but 256 is a profiling-sized case, not the benchmark")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    CFG["batch"] = args.batch

    import torch
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))

    if args.impl == "reference":
        dist = None
        torch.cuda.set_device(local_rank)
        if world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"), timeout=datetime.timedelta(seconds=300))
        line = run_reference(args, torch, dist, rank, world, torch.device(f"cuda:{local_rank}"))
        if rank == 0 and line is not None:
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return 0

    if args.workload == "e2e":
        dist = None
        torch.cuda.set_device(local_rank)
        if world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
        nvk = entry.load_package()
        nvk.lib()
        from benchmarks import e2e_bench as eb, e2e_model as em
        sampler = ClockSampler(physical_gpu_index(local_rank)) if rank == 0 else None
        if sampler:
            sampler.start()
        line = eb.run_e2e(nvk, torch, dist, rank, world, torch.device(f"cuda:{local_rank}"),
                          em.DecoderConfig(layers=args.e2e_layers), num_seqs=args.e2e_seqs,
                          len_lo=min(100, args.e2e_maxlen), len_hi=args.e2e_maxlen, use_graph=not args.no_graph,
                          kv_dtype=args.e2e_kv, allreduce=args.e2e_allreduce, linears=args.e2e_linears)
        if sampler:
            line["clocks"] = sampler.finish()
        if rank == 0:
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return 0

    if args.workload == "mixed" and world > 1:
        # config 4 with all 36 layer caches resident: KV-head shards, one per GPU, no collective inside attention
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
        nvk = entry.load_package()
        nvk.lib()
        from benchmarks import kernel_bench as kb
        dev = torch.device(f"cuda:{local_rank}")
        if CFG["num_kv_heads"] % world:
            raise SystemExit("--gpus must divide the number of KV heads")
        dist.barrier()
        line = kb.bench_mixed(nvk, torch, dev, min(args.steps, 10), min(args.warmup, 3), layers=args.layers,
                              hq=CFG["num_heads"] // world, hkv=CFG["num_kv_heads"] // world,
                              single_launch=args.mixed_single_launch, prefill_blocks_hint=args.mixed_prefill_blocks)
        t = torch.tensor([line["ms_per_step"]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            ms = float(t.item())
            line["value"] = line["value"] * line["ms_per_step"] / ms * world     # bytes of all shards / slowest rank
            line["roofline"]["note"] = "roofline figures are rank 0's shard"
            line.update({"ms_per_step": ms, "n_gpus": world, "scaling": "strong"})
            line["config"]["parallelism"] = f"tp{world}: {CFG['num_kv_heads'] // world} KV heads per GPU, replicated metadata"
            print(json.dumps(line), flush=True)
        dist.destroy_process_group()
        return 0

    if args.workload != "decode":
        if rank != 0:
            return 0
        torch.cuda.set_device(local_rank)
        nvk = entry.load_package()
        nvk.lib()
        from benchmarks import kernel_bench as kb
        dev = torch.device(f"cuda:{local_rank}")
        steps = min(args.steps, 50)
        if args.workload == "prefill":
            line = kb.bench_prefill(nvk, torch, dev, steps, args.warmup, args.seqs, min(512, args.qmax), args.qmax)
        elif args.workload == "store":
            line = kb.bench_store(nvk, torch, dev, steps, args.warmup)
        elif args.workload in ("decode_int8", "decode_fp8"):
            line = kb.bench_decode_int8(nvk, torch, dev, steps, args.warmup, batch=args.batch, fmt=args.workload[7:])
        elif args.workload == "decode_tp":
            line = kb.bench_decode_tp_shape(nvk, torch, dev, steps, args.warmup, batch=args.batch)
        elif args.workload == "linears":
            line = kb.bench_linears(nvk, torch, dev, min(steps, 20), args.warmup, rows=args.rows)
        elif args.workload == "mixed":
            line = kb.bench_mixed(nvk, torch, dev, min(steps, 10), min(args.warmup, 3), layers=args.layers,
                                  single_launch=args.mixed_single_launch, prefill_blocks_hint=args.mixed_prefill_blocks)
        else:
            line = kb.bench_prologue(nvk, torch, dev, steps, args.warmup, rows=args.rows)
        print(json.dumps(line), flush=True)
        return 0

    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"), timeout=datetime.timedelta(seconds=300))
    else:
        torch.cuda.set_device(local_rank)
    dev = torch.device(f"cuda:{local_rank}")
    line = run_ours(args, torch, dist, rank, world, dev)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
