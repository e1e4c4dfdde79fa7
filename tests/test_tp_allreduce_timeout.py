"""Failure detection of the peer-memory all-reduce on one GPU, without a GPU fault.

Every wait of ``nvk_tp_allreduce`` / ``nvk_tp_allreduce_add_rmsnorm`` on a peer is bounded (about one second): when it
runs out the block raises an error word in its own flag area, skips its remaining waits and returns, and the host reads
the word with ``nvk_tp_allreduce_status``.  Here the "peer" of a two-rank group is a second set of buffers on the same
GPU whose flags nothing ever sets (a rank that never joined): the launch must come back by itself, the status must say
which exchange gave up, the CUDA context must stay usable, and argument errors must be refused before any launch.
"""
import ctypes
import time

import pytest

from util import nvk

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _tables(count):
    lib = nvk().lib()
    lib.nvk_tp_allreduce_flag_bytes.restype = ctypes.c_size_t
    flag_bytes = int(lib.nvk_tp_allreduce_flag_bytes())
    bufs = {name: [torch.zeros(count, dtype=torch.bfloat16, device="cuda") for _ in range(2)] for name in ("in", "out", "norm")}
    flags = [torch.zeros(flag_bytes // 4, dtype=torch.int32, device="cuda") for _ in range(2)]
    arr = ctypes.c_void_p * 2
    tabs = {name: arr(*[t.data_ptr() for t in ts]) for name, ts in bufs.items()}
    tabs["flags"] = arr(*[t.data_ptr() for t in flags])
    return lib, bufs, flags, tabs


def _status(lib, flags):
    out = ctypes.c_int(-1)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.nvk_tp_allreduce_status(ctypes.c_void_p(flags[0].data_ptr()), stream, ctypes.byref(out)) == 0
    return out.value


def test_absent_peer_times_out_with_a_status_and_leaves_the_context_usable():
    count = 8 * 2 * 256
    lib, bufs, flags, tabs = _tables(count)
    bufs["in"][0].fill_(1.0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert _status(lib, flags) == 0
    t0 = time.time()
    rc = lib.nvk_tp_allreduce(tabs["in"], tabs["out"], tabs["flags"], ctypes.c_int(0), ctypes.c_int(2), ctypes.c_int64(count),
                              ctypes.c_int(nvk().BF16), stream)
    assert rc == 0, nvk().lib().nvk_last_error()
    torch.cuda.synchronize()                      # returns by itself: the wait is bounded
    waited = time.time() - t0
    assert 0.2 < waited < 20.0, waited
    assert _status(lib, flags) == 1               # gave up in the first exchange (peer never announced its addend)
    assert int(flags[0][0].item()) == 1           # the launch counter still advanced: later launches stay in step
    # the context is alive and the buffers are untouched by the abandoned reduction
    assert float(bufs["out"][0].float().abs().max()) == 0.0
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0


def test_fused_form_times_out_the_same_way():
    rows, cols = 4, 1024
    lib, bufs, flags, tabs = _tables(rows * cols)
    residual = torch.zeros((rows, cols), dtype=torch.bfloat16, device="cuda")
    weight = torch.ones(cols, dtype=torch.bfloat16, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.nvk_tp_allreduce_add_rmsnorm(tabs["in"], tabs["out"], tabs["norm"], tabs["flags"], ctypes.c_void_p(residual.data_ptr()),
                                          ctypes.c_void_p(weight.data_ptr()), ctypes.c_float(1e-6), ctypes.c_int(0), ctypes.c_int(2),
                                          ctypes.c_int(rows), ctypes.c_int(cols), ctypes.c_int(nvk().BF16), stream)
    assert rc == 0, nvk().lib().nvk_last_error()
    torch.cuda.synchronize()
    assert _status(lib, flags) == 1
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0


def test_bad_arguments_are_refused_before_any_launch():
    count = 8 * 2 * 256
    lib, bufs, flags, tabs = _tables(count)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    bf = ctypes.c_int(nvk().BF16)
    call = lambda rank, world, n, dtype=bf: lib.nvk_tp_allreduce(tabs["in"], tabs["out"], tabs["flags"], ctypes.c_int(rank),  # noqa: E731
                                                                 ctypes.c_int(world), ctypes.c_int64(n), dtype, stream)
    assert call(0, 1, count) != 0                 # a group of one has nothing to reduce
    assert call(2, 2, count) != 0                 # rank outside the group
    assert call(0, 2, count + 8) != 0             # not a multiple of 8 * world
    assert call(0, 2, 0) != 0
    assert call(0, 2, count, ctypes.c_int(nvk().F32)) != 0
    residual = torch.zeros((3, 1024), dtype=torch.bfloat16, device="cuda")
    weight = torch.ones(1024, dtype=torch.bfloat16, device="cuda")
    fused = lambda rows, cols: lib.nvk_tp_allreduce_add_rmsnorm(  # noqa: E731
        tabs["in"], tabs["out"], tabs["norm"], tabs["flags"], ctypes.c_void_p(residual.data_ptr()), ctypes.c_void_p(weight.data_ptr()),
        ctypes.c_float(1e-6), ctypes.c_int(0), ctypes.c_int(2), ctypes.c_int(rows), ctypes.c_int(cols), bf, stream)
    assert fused(3, 1024) != 0                    # rows not a multiple of world
    assert fused(2, 1028) != 0                    # cols not a multiple of 8
    assert fused(2, 16384) != 0                   # a row longer than one block handles
    torch.cuda.synchronize()
    assert _status(lib, flags) == 0               # nothing was launched
