"""World-size-2 check of the benchmark's multi-rank logic on CPU (gloo): per-rank work plans and the
max-over-ranks / sum-over-ranks aggregation that produces the whole-job value.  The data path itself needs no
collective (KV heads or batches are sharded, metadata is replicated), so this is all the N > 1 host logic."""
import importlib.util
import os
import socket

import pytest

from util import ROOT

torch = pytest.importorskip("torch")


def _load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, queue):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    bench = _load_bench()
    plan_b = bench.rank_plan(rank, world, "batch")
    plan_t = bench.rank_plan(rank, world, "kv_heads")
    # rank r took (10 + r) ms for the step and moved (100 + r) bytes with 3 launches
    times, sums = bench.combine_ranks(torch, dist, world, torch.device("cpu"), [10.0 + rank, 20.0 - rank], [100.0 + rank, 3.0])
    queue.put((rank, plan_b, plan_t, times, sums))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_agree_on_max_time_and_total_bytes():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(queue.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, plan_b, plan_t, times, sums in results:
        assert times == [11.0, 20.0]          # max over ranks
        assert sums == [201.0, 6.0]           # sum over ranks
        assert plan_b["seed"] == 2024 + rank and plan_b["scaling"] == "weak"
        assert plan_b["num_kv_heads"] == 8 and plan_b["num_heads"] == 32
        assert plan_t["seed"] == 2024 and plan_t["scaling"] == "strong"      # replicated metadata
        assert plan_t["num_kv_heads"] == 4 and plan_t["num_heads"] == 16      # KV heads sharded, group size kept


def test_kv_head_shards_must_divide_evenly():
    bench = _load_bench()
    with pytest.raises(ValueError):
        bench.rank_plan(0, 3, "kv_heads")
    assert bench.combine_ranks(torch, None, 1, torch.device("cpu"), [1.5], [7.0]) == ([1.5], [7.0])
