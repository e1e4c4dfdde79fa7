"""Child program of tests/test_e2e_tp.py (torch.distributed.run, one process per GPU): the peer-memory all-reduce
against NCCL on the same addends -- repeated eager calls (the launch counter in the flags advances), calls replayed from
a CUDA graph, a ragged count, the fused all-reduce + residual add + RMSNorm against NCCL + torch, chains of 32 dependent
launches replayed from a graph (every replay and every rank must end with the same bits), the fp16 instantiations, and
a timing of all of them for the decode-step message (256 x 4096 bf16)."""
import importlib
import os
import sys

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
    tc = importlib.import_module("benchmarks.tp_comm")
    rows, cols = 256, 4096
    comm = tc.PeerAllReduce(nvk, torch, dist, dev, rank, world, rows * cols, torch.bfloat16)
    addend, result = comm.buffers(rows, cols)
    gen = torch.Generator(device=dev)
    gen.manual_seed(100 + rank)
    ok = True

    def compare(tag, n):
        nonlocal ok
        want = addend.view(-1)[:n].clone()
        dist.all_reduce(want)
        torch.cuda.synchronize()
        err = float((result.view(-1)[:n].float() - want.float()).abs().max())
        # two addends: one rounding either way, bit-identical; more: NCCL rounds to bf16 between additions, this kernel once
        # at the end -- allow a few bf16 units in the last place of the largest sum
        tol = 0.0 if world == 2 else 4.0 * 2.0 ** -8 * float(want.float().abs().max())
        if rank == 0:
            print(f"{tag}: max |peer - nccl| = {err:.4e} (allowed {tol:.4e})", flush=True)
        ok = ok and err <= tol

    for it in range(20):                                   # eager calls, fresh data every time
        addend.copy_(torch.randn((rows, cols), generator=gen, device=dev))
        n = rows * cols if it % 3 else 8 * world * (1000 + it)   # also counts that do not fill every block
        comm.all_reduce(n)
        compare(f"eager {it}", n)

    graph = torch.cuda.CUDAGraph()                          # replayed calls: three all-reduces per replay
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        comm.all_reduce(rows * cols)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    with torch.cuda.graph(graph):
        for _ in range(3):
            comm.all_reduce(rows * cols)
    for it in range(5):
        addend.copy_(torch.randn((rows, cols), generator=gen, device=dev))
        graph.replay()
        compare(f"graph {it}", rows * cols)
    # fused form: h = residual + sum, x = rmsnorm(h) * weight, against NCCL + torch on the same data
    weight = (1.0 + 0.1 * torch.randn(cols, generator=gen, device=dev)).to(torch.bfloat16)
    dist.broadcast(weight, 0)
    residual = torch.randn((rows, cols), generator=gen, device=dev).to(torch.bfloat16)
    dist.broadcast(residual, 0)
    for it in range(4):
        addend.copy_(torch.randn((rows, cols), generator=gen, device=dev))
        want_sum = addend.clone()
        dist.all_reduce(want_sum)
        want_h = residual + want_sum
        want_x = torch.nn.functional.rms_norm(want_h, (cols,), weight, 1e-6)
        h_new, x = comm.all_reduce_add_rmsnorm(residual, weight, 1e-6, rows, cols)
        torch.cuda.synchronize()
        eh = float((h_new.float() - want_h.float()).abs().max())
        ex = float((x.float() - want_x.float()).abs().max())
        tol_h = (0.0 if world == 2 else 4.0 * 2.0 ** -8 * float(want_h.float().abs().max()))
        tol_x = 2.0 ** -6 * float(want_x.float().abs().max()) + (0.0 if world == 2 else 0.05)
        if rank == 0:
            print(f"fused {it}: max |h - ref| = {eh:.4e} (allowed {tol_h:.4e}), max |x - ref| = {ex:.4e} (allowed {tol_x:.4e})", flush=True)
        ok = ok and eh <= tol_h and ex <= tol_x
        residual = h_new.clone()      # next round continues from the new hidden state, as a decoder does
    # back-to-back launches with a consumer between them, as in a decoder: round k's addend depends on round k-1's sum,
    # so a launch that read an addend too early or left its result incomplete changes the end of the chain.  Two chains:
    # small integers (every partial sum is exact in bf16 in any order, so any number of ranks must match NCCL bit for
    # bit; the dependency is the parity of the previous sum) and, for two ranks, real-valued data.
    rounds = 32
    scratch_chain = torch.empty((rows, cols), device=dev, dtype=torch.bfloat16)
    int_noise = torch.randint(-2, 3, (rounds, rows, cols), generator=gen, device=dev).to(torch.bfloat16)
    real_noise = torch.randn((rounds, rows, cols), generator=gen, device=dev).to(torch.bfloat16)

    def next_addend(kind, noise_k, prev_sum, out):
        if kind == "integer":
            torch.add(noise_k, torch.remainder(prev_sum, 2), out=out)
        else:
            torch.add(noise_k, prev_sum, alpha=1.0 / world, out=out)

    def run_chain(kind, noise):
        nonlocal ok

        def chain_peer():
            addend.copy_(noise[0])
            for k in range(1, rounds):
                comm.all_reduce(rows * cols)
                next_addend(kind, noise[k], result, addend)
            comm.all_reduce(rows * cols)

        scratch_chain.copy_(noise[0])
        for k in range(1, rounds):
            dist.all_reduce(scratch_chain)
            next_addend(kind, noise[k], scratch_chain, scratch_chain)
        dist.all_reduce(scratch_chain)
        chain_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(chain_graph):
            chain_peer()
        for it in range(6):
            chain_graph.replay()
            torch.cuda.synchronize()
            err = float((result.float() - scratch_chain.float()).abs().max())
            if rank == 0:
                print(f"{kind} chain of {rounds} replay {it}: max |peer - nccl| = {err:.4e} (allowed 0)", flush=True)
            ok = ok and err == 0.0
        del chain_graph

    run_chain("integer", int_noise)
    if world == 2:
        run_chain("real", real_noise)
    noise = real_noise
    # the fused kernel in the same kind of chain: every replay and every rank must end with the same bits
    def chain_fused():
        h = residual_start
        addend.copy_(noise[0])
        for k in range(1, rounds):
            h, x = comm.all_reduce_add_rmsnorm(h, weight, 1e-6, rows, cols)
            torch.add(noise[k], x, alpha=0.25, out=addend)
        return comm.all_reduce_add_rmsnorm(h, weight, 1e-6, rows, cols)

    residual_start = residual.clone()
    fused_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(fused_graph):
        h_end, x_end = chain_fused()
    firsts = None
    for it in range(6):
        fused_graph.replay()
        torch.cuda.synchronize()
        got = torch.cat([h_end.reshape(-1), x_end.reshape(-1)]).clone()
        if firsts is None:
            firsts = got
            gathered = [torch.empty_like(got) for _ in range(world)]
            dist.all_gather(gathered, got)
            same_ranks = all(bool(torch.equal(g, got)) for g in gathered)
            finite = bool(torch.isfinite(got.float()).all())
            if rank == 0:
                print(f"fused chain: identical on all ranks: {same_ranks}, finite: {finite}", flush=True)
            ok = ok and same_ranks and finite
        same = bool(torch.equal(got, firsts))
        if rank == 0:
            print(f"fused chain replay {it}: identical to replay 0: {same}", flush=True)
        ok = ok and same
    # the fp16 instantiations of both kernels, on a second set of peer buffers
    comm16 = tc.PeerAllReduce(nvk, torch, dist, dev, rank, world, rows * cols, torch.float16)
    addend16, result16 = comm16.buffers(rows, cols)
    weight16 = weight.to(torch.float16)
    residual16 = (0.5 * torch.randn((rows, cols), generator=gen, device=dev)).to(torch.float16)
    dist.broadcast(residual16, 0)
    for it in range(3):
        addend16.copy_(torch.randn((rows, cols), generator=gen, device=dev))
        want = addend16.clone()
        dist.all_reduce(want)
        comm16.all_reduce(rows * cols)
        torch.cuda.synchronize()
        err = float((result16.float() - want.float()).abs().max())
        tol = 0.0 if world == 2 else 4.0 * 2.0 ** -11 * float(want.float().abs().max())
        want_h = residual16 + want
        want_x = torch.nn.functional.rms_norm(want_h, (cols,), weight16, 1e-6)
        h16, x16 = comm16.all_reduce_add_rmsnorm(residual16, weight16, 1e-6, rows, cols)
        torch.cuda.synchronize()
        eh = float((h16.float() - want_h.float()).abs().max())
        ex = float((x16.float() - want_x.float()).abs().max())
        tol_h = 0.0 if world == 2 else 4.0 * 2.0 ** -11 * float(want_h.float().abs().max())
        tol_x = 2.0 ** -9 * float(want_x.float().abs().max()) + (0.0 if world == 2 else 0.01)
        if rank == 0:
            print(f"fp16 {it}: max |sum - nccl| = {err:.4e} (allowed {tol:.4e}), max |h - ref| = {eh:.4e} (allowed {tol_h:.4e}), "
                  f"max |x - ref| = {ex:.4e} (allowed {tol_x:.4e})", flush=True)
        ok = ok and err <= tol and eh <= tol_h and ex <= tol_x
    ok = ok and comm16.status() == 0
    comm16.close()
    status = comm.status()
    ok = ok and status == 0

    # timing, 72 per replay as in a decode step of 36 layers
    def timed(fn, reps=20):
        g = torch.cuda.CUDAGraph()
        fn()
        torch.cuda.synchronize()
        dist.barrier()
        with torch.cuda.graph(g):
            for _ in range(72):
                fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps / 72 * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    scratch = torch.randn((rows, cols), generator=gen, device=dev).to(torch.bfloat16)
    us_peer = timed(lambda: comm.all_reduce(rows * cols))
    us_nccl = timed(lambda: dist.all_reduce(scratch))
    res_buf = residual.clone()

    def unfused():
        dist.all_reduce(scratch)
        torch.nn.functional.rms_norm(res_buf + scratch, (cols,), weight, 1e-6)

    us_fused = timed(lambda: comm.all_reduce_add_rmsnorm(res_buf, weight, 1e-6, rows, cols))
    us_unfused = timed(unfused)
    # row-parallel linear whose epilogue pushes the partial sums (o_proj shape: in_features 4096 / world), against
    # cuBLAS GEMM + NCCL + add + rms_norm; then timing over 36 distinct weight matrices (weights stream from HBM)
    k_in = 4096 // world
    w_rows = [(0.02 * torch.randn((cols, k_in), generator=gen, device=dev)).to(torch.bfloat16) for _ in range(36)]
    x_in = (0.5 * torch.randn((rows, k_in), generator=gen, device=dev)).to(torch.bfloat16)
    part = x_in @ w_rows[0].t()
    dist.all_reduce(part)
    want_h = res_buf + part
    want_x = torch.nn.functional.rms_norm(want_h, (cols,), weight, 1e-6)
    h_f, x_f = comm.row_linear_all_reduce_add_rmsnorm(x_in, w_rows[0], res_buf, weight, 1e-6)
    torch.cuda.synchronize()
    eh = float((h_f.float() - want_h.float()).abs().max())
    ex = float((x_f.float() - want_x.float()).abs().max())
    tol_h = 2.0 ** -7 * float(want_h.float().abs().max())
    tol_x = 2.0 ** -6 * float(want_x.float().abs().max())
    gemm_word = nvk.gemm_status()
    if rank == 0:
        print(f"row-parallel linear + all-reduce + add + rmsnorm: max |h - ref| = {eh:.4e} (allowed {tol_h:.4e}), "
              f"max |x - ref| = {ex:.4e} (allowed {tol_x:.4e}), gemm status {gemm_word}", flush=True)
    ok = ok and eh <= tol_h and ex <= tol_x and gemm_word == 0 and comm.status() == 0
    turn = [0]
    addend_buf, _ = comm.buffers(rows, cols)

    def next_w():
        turn[0] += 1
        return w_rows[turn[0] % len(w_rows)]

    def gemm_then_fused():
        torch.matmul(x_in, next_w().t(), out=addend_buf)
        comm.all_reduce_add_rmsnorm(res_buf, weight, 1e-6, rows, cols)

    def gemm_then_nccl():
        torch.matmul(x_in, next_w().t(), out=scratch)
        dist.all_reduce(scratch)
        torch.nn.functional.rms_norm(res_buf + scratch, (cols,), weight, 1e-6)

    us_row_fused = timed(lambda: comm.row_linear_all_reduce_add_rmsnorm(x_in, next_w(), res_buf, weight, 1e-6))
    us_row_two = timed(gemm_then_fused)
    us_row_nccl = timed(gemm_then_nccl)
    ok = ok and nvk.gemm_status() == 0 and comm.status() == 0
    if rank == 0:
        print(f"timing world {world}: row-parallel linear ({k_in} -> {cols}) + all-reduce + add + rmsnorm: pushed from the GEMM epilogue "
              f"{us_row_fused:.2f} us, cuBLAS + fused all-reduce {us_row_two:.2f} us, cuBLAS + NCCL + add + rms_norm {us_row_nccl:.2f} us", flush=True)
    if rank == 0:
        print(f"timing world {world}: peer-memory all-reduce {us_peer:.2f} us, NCCL {us_nccl:.2f} us per 2 MiB message (in a graph)", flush=True)
        print(f"timing world {world}: fused all-reduce + add + rmsnorm {us_fused:.2f} us, NCCL + add + rms_norm {us_unfused:.2f} us", flush=True)
    comm.close()

    # the same two operations through the switch (multimem), where the group has a multicast object
    mm = None
    try:
        mm = tc.MulticastAllReduce(nvk, torch, dist, dev, rank, world, rows * cols, torch.bfloat16)
        made = 1
    except Exception as exc:
        made = 0
        if rank == 0:
            print(f"multimem: unavailable ({type(exc).__name__}: {exc})", flush=True)
    agree = torch.tensor([made], device=dev)
    dist.all_reduce(agree, op=dist.ReduceOp.MIN)
    if int(agree.item()) == 1:
        mm_addend, mm_result = mm.buffers(rows, cols)
        res_mm = residual.clone()
        for it in range(3):
            mm_addend.copy_((0.5 * torch.randn((rows, cols), generator=gen, device=dev)).to(torch.bfloat16))
            # reference: every rank's addend summed in fp32 and rounded once (the switch accumulates in fp32 in an order of
            # its own: one unit of the 16-bit type around that; NCCL rounds at every hop of its ring)
            parts = [torch.empty_like(mm_addend) for _ in range(world)]
            dist.all_gather(parts, mm_addend.clone())
            want = torch.stack([x.float() for x in parts]).sum(dim=0).to(torch.bfloat16)
            mm.all_reduce(rows * cols, cols)
            torch.cuda.synchronize()
            err = float((mm_result.float() - want.float()).abs().max())
            tol = 2.0 ** -7 * float(want.float().abs().max())
            want_h = res_mm + want
            want_x = torch.nn.functional.rms_norm(want_h, (cols,), weight, 1e-6)
            h_mm, x_mm = mm.all_reduce_add_rmsnorm(res_mm, weight, 1e-6, rows, cols)
            torch.cuda.synchronize()
            eh = float((h_mm.float() - want_h.float()).abs().max())
            ex = float((x_mm.float() - want_x.float()).abs().max())
            tol_h = 2.0 ** -7 * float(want_h.float().abs().max())
            tol_x = 2.0 ** -6 * float(want_x.float().abs().max())
            got = torch.cat([h_mm.reshape(-1), x_mm.reshape(-1)]).clone()
            gathered = [torch.empty_like(got) for _ in range(world)]
            dist.all_gather(gathered, got)
            same = all(bool(torch.equal(g, got)) for g in gathered)
            if rank == 0:
                print(f"multimem {it}: max |sum - fp32 sum| = {err:.4e} (allowed {tol:.4e}), max |h - ref| = {eh:.4e} (allowed {tol_h:.4e}), "
                      f"max |x - ref| = {ex:.4e} (allowed {tol_x:.4e}), identical on all ranks: {same}", flush=True)
            ok = ok and err <= tol and eh <= tol_h and ex <= tol_x and same
        us_mm = timed(lambda: mm.all_reduce(rows * cols, cols))
        us_mm_fused = timed(lambda: mm.all_reduce_add_rmsnorm(res_mm, weight, 1e-6, rows, cols))
        st = mm.status()
        ok = ok and st == 0
        if rank == 0:
            print(f"timing world {world}: multimem all-reduce {us_mm:.2f} us, multimem all-reduce + add + rmsnorm {us_mm_fused:.2f} us (status {st})", flush=True)
    if mm is not None:
        mm.close()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    return 0 if int(flag.item()) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
