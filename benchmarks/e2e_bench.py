"""Output tokens per second of the end-to-end decoder (``bench.py --workload e2e``), one process per GPU.

Requests, scheduling and block tables come from ``e2e_schedule.py``, the decoder from ``e2e_model.py``.  With N
processes the model is tensor-parallel over N GPUs (KV-head sharding, all-reduce after o_proj / down_proj: this
library's peer-memory kernel in the decode steps unless ``allreduce="nccl"``, NCCL in the prefill steps).
Timed region: from the first prefill step to the last decode step, host scheduling and the per-step host-to-device
metadata copy included, CUDA events on the compute stream, maximum over ranks.
"""
from __future__ import annotations

import time

import numpy as np

from .e2e_model import Decoder, DecoderConfig
from .e2e_schedule import Schedule, blocks_needed, make_requests, plan_prefill_batches

RING = 64   # pinned metadata slots in flight


def run_e2e(nvk, torch, dist, rank, world, dev, cfg: DecoderConfig | None = None, num_seqs=256, len_lo=100, len_hi=1024,
            seed=0, use_graph=True, kv_dtype="bf16", allreduce="auto", linears="cublas"):
    cfg = cfg or DecoderConfig()
    bs = cfg.block_size
    prompts, output_lens = make_requests(num_seqs, cfg.vocab, len_lo, len_hi, seed)
    prompt_lens = np.array([len(p) for p in prompts])
    table_width = (2 * len_hi + bs - 1) // bs
    num_blocks = blocks_needed(prompt_lens, output_lens, bs) + 8
    t0 = time.time()
    comm = None
    allreduce_kind = "NCCL"
    if allreduce == "auto":
        # measured per 2 MiB message, fused form: tagged-word kernel 12.2 / 16.7 us at 2 / 4 ranks and growing with the
        # bytes it sends to every peer; in-switch kernel 16.8 / 17.6 us.  The in-switch kernel has not been timed at 8 ranks,
        # and a rank that dies while bound to a multicast object disturbs its peers' GPUs, so the default stays with the
        # kernel that needs nothing but peer mappings; "multimem" selects the other one.
        allreduce = "peer"
    if allreduce in ("peer", "multimem") and world > 1:
        from .tp_comm import MulticastAllReduce, PeerAllReduce
        if allreduce == "multimem":
            # every rank must take the same path: the ranks agree on whether the multicast object could be made
            try:
                comm = MulticastAllReduce(nvk, torch, dist, dev, rank, world, num_seqs * cfg.hidden, torch.bfloat16)
                made = 1
            except Exception as exc:   # no multicast support on this box: the peer-memory kernel instead
                comm, made = None, 0
                if rank == 0:
                    print(f"# multimem all-reduce unavailable ({type(exc).__name__}: {exc}); using the peer-memory kernel", flush=True)
            agree = torch.tensor([made], device=dev)
            dist.all_reduce(agree, op=dist.ReduceOp.MIN)
            if int(agree.item()) == 0 and comm is not None:
                comm.close()
                comm = None
            if comm is not None:
                allreduce_kind = ("decode steps: in-switch reduction and broadcast (multimem.ld_reduce / multimem.st) fused with the residual "
                                  "add and the RMSNorm (nvk_tp_allreduce_add_rmsnorm_multimem); prefill steps: NCCL")
        if comm is None:
            comm = PeerAllReduce(nvk, torch, dist, dev, rank, world, num_seqs * cfg.hidden, torch.bfloat16)
            allreduce_kind = ("decode steps: peer-memory all-reduce fused with the residual add and the RMSNorm "
                              "(nvk_tp_allreduce_add_rmsnorm); prefill steps: NCCL")
    model = Decoder(nvk, torch, dev, cfg, rank, world, dist, num_blocks=num_blocks, seed=seed, kv_dtype=kv_dtype, peer_comm=comm,
                    linears=linears)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    model.ensure_workspace(num_seqs, table_width)

    # ---- warm-up: one small prefill (cuBLAS / NCCL / tensor-map set-up), then the decode step, then its capture ----
    warm = Schedule(prompts[:4], output_lens[:4], bs, num_blocks, table_width, pool_seed=99)
    model.prefill_step(warm.prefill_arrays([0, 1, 2, 3]))
    width = 3 + table_width
    tokens_static = torch.zeros(num_seqs, device=dev, dtype=torch.int64)
    meta_static = torch.zeros((num_seqs, width), device=dev, dtype=torch.int32)
    meta_static[:, 1] = -1
    graph = None
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            tokens_static.copy_(model.decode_forward(tokens_static, meta_static))
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            tokens_static.copy_(model.decode_forward(tokens_static, meta_static))
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()

    # ---- timed run ------------------------------------------------------------------------------------------------
    sched = Schedule(prompts, output_lens, bs, num_blocks, table_width, pool_seed=1)
    batches = plan_prefill_batches(prompt_lens, cfg.max_num_seqs, cfg.max_num_batched_tokens)
    steps = sched.total_decode_steps()
    meta_pinned = torch.empty((RING, num_seqs, width), dtype=torch.int32).pin_memory()
    meta_np = meta_pinned.numpy()
    slot_free = [torch.cuda.Event() for _ in range(RING)]
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    launches0 = nvk.launch_count
    snapshot = None
    torch.cuda.synchronize()
    ev[0].record()
    for ids in batches:
        first = model.prefill_step(sched.prefill_arrays(ids))
        tokens_static[torch.as_tensor(ids, device=dev)] = first
    ev[1].record()
    active_rows = 0
    for t in range(steps):
        s = t % RING
        if t >= RING:
            slot_free[s].synchronize()
        active_rows += sched.decode_arrays(meta_np[s])
        meta_static.copy_(meta_pinned[s], non_blocking=True)
        slot_free[s].record()
        if graph is not None:
            graph.replay()
        else:
            tokens_static.copy_(model.decode_forward(tokens_static, meta_static))
        if t == steps // 4:
            snapshot = meta_np[s].copy()
    ev[2].record()
    torch.cuda.synchronize()
    total_ms, prefill_ms, decode_ms = ev[0].elapsed_time(ev[2]), ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])
    eager_launches = nvk.launch_count - launches0
    # kernels of this library per step: prologue + prefill attention per layer in prefill; prologue + split + merge in decode
    # (+ the quantising store with an int8 cache, + the two all-reduces per layer with the peer-memory kernel)
    our_launches = (len(batches) * cfg.layers * 2 + steps * cfg.layers * 3) + (len(batches) + steps) * cfg.layers * (1 if model.int8 else 0)
    if comm is not None:   # two fused all-reduce launches per layer in every decode step
        our_launches += steps * cfg.layers * 2

    # ---- attention share of a decode step, on the metadata of a step a quarter into the run ----------------------------
    attn_ms = None
    if snapshot is not None:
        meta_static.copy_(torch.from_numpy(snapshot).to(dev))
        positions, slots, ctx = meta_static[:, 0].contiguous(), meta_static[:, 1].contiguous(), meta_static[:, 2].contiguous()
        slots.fill_(-1)                      # do not disturb the cache: the prologue skips the store for slot -1
        tables = meta_static[:, 3:].contiguous()
        qkv = torch.randn((num_seqs, (model.hq + 2 * model.hkv) * cfg.head_dim), device=dev).to(torch.bfloat16)
        q = torch.empty((num_seqs, model.hq, cfg.head_dim), device=dev, dtype=torch.bfloat16)
        out = torch.empty_like(q)

        attend = model.attend_decode(ctx, tables)
        k_step = torch.empty((num_seqs, model.hkv, cfg.head_dim), device=dev, dtype=torch.bfloat16)
        v_step = torch.empty_like(k_step)
        rows = torch.arange(num_seqs, device=dev, dtype=torch.int32)

        def attention_only():
            for l, w in enumerate(model.layers):
                if model.int8:   # prologue into the dense scratch; the quantising store is skipped (all slots are -1)
                    nvk.fused_split_norm_rope_store(qkv, positions, w["q_norm"], w["k_norm"], cfg.eps, model.cos_sin, rows,
                                                    k_step, v_step, model.hq, model.hkv, cfg.head_dim, q)
                else:
                    nvk.fused_split_norm_rope_store(qkv, positions, w["q_norm"], w["k_norm"], cfg.eps, model.cos_sin, slots,
                                                    model.kv_cache[0, l], model.kv_cache[1, l], model.hq, model.hkv, cfg.head_dim, q)
                attend(l, q, k_step, v_step, out)

        for _ in range(3):
            attention_only()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(10):
            attention_only()
        a1.record()
        torch.cuda.synchronize()
        attn_ms = a0.elapsed_time(a1) / 10

    comm_status = comm.status() if comm is not None else 0
    prefill_status = nvk.prefill_status()     # non-zero: a tensor-core prefill launch gave up a bounded wait (rows incomplete)
    times = torch.tensor([total_ms, prefill_ms, decode_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, prefill_ms, decode_ms = (float(x) for x in times.tolist())
    out_tokens = int(output_lens.sum())
    line = {
        "metric": "qwen3_8b_output_tokens_per_s", "value": out_tokens / (total_ms / 1e3), "unit": "tok/s", "n_gpus": world,
        "steps": len(batches) + steps, "warmup": 4, "ms_per_step": decode_ms / max(steps, 1), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"end-to-end decoder, {cfg.layers} layers, hidden {cfg.hidden}, {cfg.num_heads}/{cfg.num_kv_heads} heads, "
                               f"head_dim {cfg.head_dim}, FFN {cfg.ffn}, vocab {cfg.vocab}, random-init bf16 weights; {num_seqs} sequences, "
                               f"prompt and output lengths U[{len_lo},{len_hi}], greedy, ignore_eos",
                   "parallelism": f"tp{world} (KV-head shards, all-reduce after o_proj / down_proj)",
                   "kv_cache": (("e4m3" if model.fp8 else "int8") + " with fp16 per-(token, head) scales") if model.int8 else "bf16",
                   "allreduce": allreduce_kind,
                   "linears": ("decode steps: QKV projection with split + norm + RoPE + cache store in its epilogue "
                               "(nvk_qkv_linear_norm_rope_store)" + ("; o_proj / down_proj push their partial sums into the all-reduce "
                               "from their epilogue (nvk_tp_row_linear_allreduce_add_rmsnorm)" if comm is not None else "") +
                               "; other linears and prefill steps: cuBLAS" if model.fused_linears else "cuBLAS (torch.matmul)"),
                   "decode": "one captured CUDA graph of %d fixed rows" % num_seqs if graph is not None else "eager",
                   "prefill_batches": len(batches), "decode_steps": steps, "kv_blocks": num_blocks,
                   "l2": "weights (16.4 GB / tp) and KV cache exceed the 126 MB L2"},
        "output_tokens": out_tokens, "prompt_tokens": int(prompt_lens.sum()),
        "total_s": total_ms / 1e3, "prefill_s": prefill_ms / 1e3, "decode_s": decode_ms / 1e3,
        "mean_active_rows": active_rows / max(steps, 1),
        "attention_ms_per_decode_step": attn_ms,
        "attention_share_of_decode_step": (attn_ms / (decode_ms / max(steps, 1))) if attn_ms else None,
        "model_build_s": build_s, "peer_allreduce_status": comm_status, "prefill_status": prefill_status,
        "gemm_status": nvk.gemm_status() if model.fused_linears else None,
        "gpu_launches": our_launches, "gpu_launches_issued_eagerly": eager_launches,
        "e2e": {"value": out_tokens / (total_ms / 1e3), "unit": "tok/s",
                "h2d_bytes_per_step": num_seqs * width * 4, "d2h_bytes_per_step": 0,
                "note": "the timed region already runs through the host scheduler and copies every step's metadata from pinned "
                        "memory; sampled tokens stay on the device (ignore_eos: the host needs no token to schedule)"},
    }
    if comm is not None:
        del graph
        comm.close()
    return line
