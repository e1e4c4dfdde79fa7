"""Child program of tests/test_e2e_tp.py (run under torch.distributed.run, one process per GPU): the tensor-parallel
decoder (KV-head shards, all-reduce after o_proj / down_proj) must produce the hidden states of the single-GPU decoder
built from the same seed, for a prefill step and for decode steps on the cache that step filled."""
import importlib
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", device_id=dev)
    nvk = entry.load_package()
    nvk.lib()
    em = importlib.import_module("benchmarks.e2e_model")
    es = importlib.import_module("benchmarks.e2e_schedule")
    cfg = em.DecoderConfig(layers=2, hidden=512, num_heads=8, num_kv_heads=4, head_dim=128, ffn=1024, vocab=1000,
                           max_model_len=1024, max_num_seqs=8, max_num_batched_tokens=2048)
    rng = np.random.default_rng(9)
    lens, extra = [70, 300], 2
    full = [rng.integers(0, cfg.vocab, size=n + extra) for n in lens]

    def run(model):
        model.ensure_workspace(len(lens), 4)
        s = es.Schedule([f[:n] for f, n in zip(full, lens)], [extra + 1] * len(lens), cfg.block_size, 16, 4)
        a = s.prefill_arrays(list(range(len(lens))))
        up = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(dev)  # noqa: E731
        cu, tables = up(a["cu_seqlens_q"]), up(a["block_tables"])
        hs = [model.forward(up(a["tokens"]), up(a["positions"]), up(a["slot_mapping"]), model.attend_prefill(cu, cu, tables)).float()]
        meta = np.zeros((len(lens), 3 + 4), dtype=np.int32)
        for step in range(extra):
            s.decode_arrays(meta)
            m = torch.from_numpy(meta).to(dev)
            tokens = torch.tensor([int(f[n + step]) for f, n in zip(full, lens)], device=dev)
            hs.append(model.forward(tokens, m[:, 0].contiguous(), m[:, 1].contiguous(),
                                    model.attend_decode(m[:, 2].contiguous(), m[:, 3:].contiguous())).float())
        return hs

    comm = None
    mode = os.environ.get("TP_CHECK_PEER", "0")   # 1: decode-step all-reduces through the peer-memory kernel; 2: and the fused linears
    if mode == "3":   # decode-step all-reduces through the switch (multimem), where the group has a multicast object
        tc = importlib.import_module("benchmarks.tp_comm")
        try:
            comm, made = tc.MulticastAllReduce(nvk, torch, dist, dev, rank, world, 8 * cfg.hidden, torch.bfloat16), 1
        except Exception as exc:
            comm, made = None, 0
            print(f"rank {rank}: multimem unavailable ({type(exc).__name__}: {exc})", flush=True)
        agree = torch.tensor([made], device=dev)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        if int(agree.item()) == 0:
            if comm is not None:
                comm.close()
            if rank == 0:
                print("step 0: skipped, no multicast support\nstep 1: skipped\nstep 2: skipped", flush=True)
            dist.destroy_process_group()
            return 0
    if mode in ("1", "2"):
        tc = importlib.import_module("benchmarks.tp_comm")
        comm = tc.PeerAllReduce(nvk, torch, dist, dev, rank, world, 8 * cfg.hidden, torch.bfloat16)
    sharded = run(em.Decoder(nvk, torch, dev, cfg, rank, world, dist, num_blocks=16, seed=4, peer_comm=comm,
                             linears="fused" if mode == "2" else "cublas"))
    if mode == "2":
        assert nvk.gemm_status() == 0
    if comm is not None:
        assert comm.status() == 0
        comm.close()
    ok = True
    if rank == 0:
        single = run(em.Decoder(nvk, torch, dev, cfg, 0, 1, None, num_blocks=16, seed=4))
        for i, (a, b) in enumerate(zip(sharded, single)):
            err = float((a - b).abs().max())
            ref = float(b.abs().max())
            print(f"step {i}: max |tp - single| {err:.4e} (max |single| {ref:.3f})", flush=True)
            ok = ok and err <= 0.03 * max(1.0, ref)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.broadcast(flag, 0)
    dist.destroy_process_group()
    return 0 if int(flag.item()) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
