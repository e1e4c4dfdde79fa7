"""Parity of the peer-memory all-reduce kernels on ONE GPU: ``nvk_tp_allreduce_inprocess`` runs the same device code for
2, 4 or 8 ranks as one cooperative launch over one buffer set per rank (the reference tests its tensor-parallel layers
the same way, with an in-process communicator: src/utils/tensor_parallel.cpp:165-277, tests/test_models.cpp:418-557).

Expected values are plain torch: the fp32 sum of the addends in rank order, rounded once to the 16-bit type; for the
fused form the residual added in the 16-bit type and an fp32 RMSNorm of the rounded row.  The sum must match bit for
bit (same order, one rounding); the norm within one unit of the 16-bit type (the kernel's rsqrt).  Every rank must end
with the same bits, across repeated launches (the launch counter advances) and when replayed from a CUDA graph.
"""
import importlib

import pytest

from util import nvk

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _comm(world, max_elems, dtype):
    tc = importlib.import_module("benchmarks.tp_comm")
    return tc.InProcessAllReduce(nvk(), torch, torch.device("cuda"), world, max_elems, dtype)


def _expected_sum(addends, n, dtype):
    acc = torch.zeros(n, device="cuda", dtype=torch.float32)
    for a in addends:                      # rank order, fp32, one rounding at the end
        acc += a[:n].float()
    return acc.to(dtype)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_plain_sum_matches_torch_bit_for_bit(world, dtype):
    rows, cols = 64, 1024
    comm = _comm(world, rows * cols, dtype)
    gen = torch.Generator(device="cuda").manual_seed(world)
    for it, (r, c) in enumerate([(rows, cols), (rows, cols), (world, 8 * 33), (8, 8 * world), (rows, cols)]):
        n = r * c
        for a in comm.addend:
            a.copy_(torch.randn(a.shape, generator=gen, device="cuda"))
        comm.launch(r, c)
        torch.cuda.synchronize()
        want = _expected_sum(comm.addend, n, dtype)
        for rank in range(world):
            assert torch.equal(comm.result[rank][:n], want), (it, rank)
            assert comm.status(rank) == 0


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_add_rmsnorm_matches_torch(world, dtype):
    rows, cols = 8 * world, 4096
    comm = _comm(world, rows * cols, dtype)
    gen = torch.Generator(device="cuda").manual_seed(100 + world)
    weight = (1.0 + 0.1 * torch.randn(cols, generator=gen, device="cuda")).to(dtype)
    residual = torch.randn((rows, cols), generator=gen, device="cuda").to(dtype)
    residuals = [residual.clone() for _ in range(world)]
    ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    for it in range(3):
        for a in comm.addend:
            a.copy_(0.5 * torch.randn(a.shape, generator=gen, device="cuda"))
        comm.launch(rows, cols, residuals=residuals, weight=weight, eps=1e-6)
        torch.cuda.synchronize()
        total = _expected_sum(comm.addend, rows * cols, dtype).view(rows, cols)
        want_h = residuals[0] + total                                        # added in the 16-bit type
        hf = want_h.float()
        want_x = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * weight.float())
        for rank in range(world):
            h = comm.result[rank].view(rows, cols)
            x = comm.normed[rank].view(rows, cols)
            assert torch.equal(h, want_h), (it, rank)
            assert torch.equal(x, comm.normed[0].view(rows, cols))           # every rank holds the same bits
            err = (x.float() - want_x).abs()
            assert bool((err <= want_x.abs().clamp_min(1e-2) * 2 * ulp).all()), float(err.max())
            assert comm.status(rank) == 0
        residuals = [comm.result[r].view(rows, cols).clone() for r in range(world)]   # the next layer continues from h_new


def test_in_place_residual_and_graph_replay():
    """A decoder keeps its hidden state in the result buffer (residual == out), and decode steps replay a captured graph:
    a chain of dependent launches must give the same bits eagerly and on every replay."""
    world, rows, cols, dtype = 4, 32, 2048, torch.bfloat16
    comm = _comm(world, rows * cols, dtype)
    gen = torch.Generator(device="cuda").manual_seed(7)
    weight = (1.0 + 0.1 * torch.randn(cols, generator=gen, device="cuda")).to(dtype)
    start = torch.randn((rows, cols), generator=gen, device="cuda").to(dtype)
    noise = [[(0.3 * torch.randn((rows * cols,), generator=gen, device="cuda")).to(dtype) for _ in range(world)] for _ in range(6)]

    def chain():
        for r in range(world):
            comm.result[r].copy_(start.view(-1))
        for k in range(6):
            for r in range(world):
                torch.add(noise[k][r], comm.normed[r], alpha=0.25, out=comm.addend[r])   # depends on the previous launch
            comm.launch(rows, cols, residuals=[t.view(rows, cols) for t in comm.result], weight=weight)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for t in comm.normed:
            t.zero_()
        chain()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    eager = [torch.cat([comm.result[r], comm.normed[r]]).clone() for r in range(world)]
    assert all(torch.equal(eager[0], e) for e in eager[1:])
    assert bool(torch.isfinite(eager[0].float()).all())
    graph = torch.cuda.CUDAGraph()
    for t in comm.normed:
        t.zero_()
    with torch.cuda.graph(graph):
        chain()
    for _ in range(3):
        for t in comm.normed:
            t.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.equal(torch.cat([comm.result[r], comm.normed[r]]), eager[0])
    assert all(comm.status(r) == 0 for r in range(world))
