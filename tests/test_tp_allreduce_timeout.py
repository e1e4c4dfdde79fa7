"""Failure detection of the peer-memory all-reduce on one GPU, without a GPU fault.

Every wait of ``nvk_tp_allreduce`` / ``nvk_tp_allreduce_add_rmsnorm`` is a wait for a peer's data and is bounded
(``nvk_tp_allreduce_set_wait_limit_ms``).  When it runs out the rank's error word becomes non-zero and stays so: later
launches of that rank return at once, and ``nvk_tp_allreduce_status`` tells the host.  Here the "peer" of a two-rank
group is a second staging area on the same GPU into which nothing is ever pushed (a rank that never joined): the launch
must come back by itself, the status must say which wait gave up, the next launch must not wait again, the CUDA context
must stay usable, a LATE peer must fail fast instead of hanging, and after the documented reset the same buffers must
work again.  Argument errors must be refused before any launch.
"""
import ctypes
import time

import pytest

from util import nvk

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

LIMIT_MS = 400


def _lib():
    import importlib
    lib = nvk().lib()
    importlib.import_module("benchmarks.tp_comm").declare(lib)
    return lib


def _group(count, world=2):
    lib = _lib()
    stage_bytes = int(lib.nvk_tp_allreduce_stage_bytes(count))
    bufs = {name: [torch.zeros(count, dtype=torch.bfloat16, device="cuda") for _ in range(world)] for name in ("in", "out", "norm")}
    stage = [torch.zeros(stage_bytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    flags = [torch.zeros(int(lib.nvk_tp_allreduce_flag_bytes()) // 4, dtype=torch.int32, device="cuda") for _ in range(world)]
    tab = (ctypes.c_void_p * world)(*[t.data_ptr() for t in stage])
    return lib, bufs, stage, flags, tab, stage_bytes


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _status(lib, flags, rank=0):
    out = ctypes.c_int(-1)
    assert lib.nvk_tp_allreduce_status(ctypes.c_void_p(flags[rank].data_ptr()), _stream(), ctypes.byref(out)) == 0
    return out.value


def _launch(lib, bufs, flags, tab, stage_bytes, rank, count):
    return lib.nvk_tp_allreduce(ctypes.c_void_p(bufs["in"][rank].data_ptr()), ctypes.c_void_p(bufs["out"][rank].data_ptr()), tab,
                                ctypes.c_size_t(stage_bytes), ctypes.c_void_p(flags[rank].data_ptr()), ctypes.c_int(rank),
                                ctypes.c_int(2), ctypes.c_int64(count), ctypes.c_int(nvk().BF16), _stream())


@pytest.fixture(autouse=True)
def short_wait_limit():
    lib = _lib()
    lib.nvk_tp_allreduce_set_wait_limit_ms(LIMIT_MS)
    yield
    lib.nvk_tp_allreduce_set_wait_limit_ms(10000)


def test_absent_peer_times_out_once_then_the_error_is_sticky_and_a_late_peer_fails_fast():
    count = 8 * 2 * 256
    lib, bufs, stage, flags, tab, stage_bytes = _group(count)
    bufs["in"][0].fill_(1.0)
    bufs["in"][1].fill_(2.0)
    assert _status(lib, flags) == 0
    t0 = time.time()
    assert _launch(lib, bufs, flags, tab, stage_bytes, 0, count) == 0, lib.nvk_last_error()
    torch.cuda.synchronize()                      # returns by itself: the wait is bounded
    waited = time.time() - t0
    assert 0.5 * LIMIT_MS / 1e3 < waited < 20.0, waited
    assert _status(lib, flags) == 1               # the peer's addend slice never arrived
    assert int(flags[0][0].item()) == 1           # the launch counter still advanced
    # sticky: the next launch does not wait again, and the word is unchanged
    t0 = time.time()
    assert _launch(lib, bufs, flags, tab, stage_bytes, 0, count) == 0
    torch.cuda.synchronize()
    assert time.time() - t0 < 0.05
    assert _status(lib, flags) == 1
    # the late peer: it finds rank 0's slice (pushed before rank 0 gave up), reduces its own chunk, then waits for rank
    # 0's result slice, which rank 0 never produced -- one bounded wait, status 2, no hang and no stale result accepted
    t0 = time.time()
    assert _launch(lib, bufs, flags, tab, stage_bytes, 1, count) == 0
    torch.cuda.synchronize()
    assert 0.5 * LIMIT_MS / 1e3 < time.time() - t0 < 20.0
    assert _status(lib, flags, rank=1) == 2
    # the context is alive
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0
    # documented recovery: with no launch in flight, zero the staging areas and reset the flag areas of every rank ...
    for r in range(2):
        stage[r].zero_()
        assert lib.nvk_tp_allreduce_reset(ctypes.c_void_p(flags[r].data_ptr()), _stream()) == 0
    assert _status(lib, flags, 0) == 0 and _status(lib, flags, 1) == 0
    # ... and the same buffers serve a complete group again (both ranks in one cooperative launch)
    arr = lambda ts: (ctypes.c_void_p * 2)(*[t.data_ptr() for t in ts])  # noqa: E731
    rc = lib.nvk_tp_allreduce_inprocess(arr(bufs["in"]), arr(bufs["out"]), None, tab, ctypes.c_size_t(stage_bytes), arr(flags), None,
                                        None, ctypes.c_float(0.0), ctypes.c_int(2), ctypes.c_int(2), ctypes.c_int(count // 2),
                                        ctypes.c_int(nvk().BF16), _stream())
    assert rc == 0, lib.nvk_last_error()
    torch.cuda.synchronize()
    assert _status(lib, flags, 0) == 0 and _status(lib, flags, 1) == 0
    for r in range(2):
        assert torch.equal(bufs["out"][r], torch.full_like(bufs["out"][r], 3.0))


def test_fused_form_times_out_the_same_way():
    rows, cols = 4, 1024
    lib, bufs, stage, flags, tab, stage_bytes = _group(rows * cols)
    residual = torch.zeros((rows, cols), dtype=torch.bfloat16, device="cuda")
    weight = torch.ones(cols, dtype=torch.bfloat16, device="cuda")
    rc = lib.nvk_tp_allreduce_add_rmsnorm(
        ctypes.c_void_p(bufs["in"][0].data_ptr()), ctypes.c_void_p(bufs["out"][0].data_ptr()), ctypes.c_void_p(bufs["norm"][0].data_ptr()),
        tab, ctypes.c_size_t(stage_bytes), ctypes.c_void_p(flags[0].data_ptr()), ctypes.c_void_p(residual.data_ptr()),
        ctypes.c_void_p(weight.data_ptr()), ctypes.c_float(1e-6), ctypes.c_int(0), ctypes.c_int(2), ctypes.c_int(rows), ctypes.c_int(cols),
        ctypes.c_int(nvk().BF16), _stream())
    assert rc == 0, lib.nvk_last_error()
    torch.cuda.synchronize()
    assert _status(lib, flags) == 1
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0


def test_bad_arguments_are_refused_before_any_launch():
    count = 8 * 2 * 256
    lib, bufs, stage, flags, tab, stage_bytes = _group(count)
    bf = nvk().BF16

    def call(rank, world, n, dtype=bf, nbytes=stage_bytes):
        return lib.nvk_tp_allreduce(ctypes.c_void_p(bufs["in"][0].data_ptr()), ctypes.c_void_p(bufs["out"][0].data_ptr()), tab,
                                    ctypes.c_size_t(nbytes), ctypes.c_void_p(flags[0].data_ptr()), ctypes.c_int(rank), ctypes.c_int(world),
                                    ctypes.c_int64(n), ctypes.c_int(dtype), _stream())

    assert call(0, 1, count) != 0                 # a group of one has nothing to reduce
    assert call(2, 2, count) != 0                 # rank outside the group
    assert call(0, 2, count + 8) != 0             # not a multiple of 8 * world
    assert call(0, 2, 0) != 0
    assert call(0, 2, count, nvk().F32) != 0
    assert call(0, 2, count, nbytes=stage_bytes // 2) != 0      # staging areas too small for the message
    residual = torch.zeros((3, 1024), dtype=torch.bfloat16, device="cuda")
    weight = torch.ones(1024, dtype=torch.bfloat16, device="cuda")

    def fused(rows, cols):
        return lib.nvk_tp_allreduce_add_rmsnorm(
            ctypes.c_void_p(bufs["in"][0].data_ptr()), ctypes.c_void_p(bufs["out"][0].data_ptr()), ctypes.c_void_p(bufs["norm"][0].data_ptr()),
            tab, ctypes.c_size_t(stage_bytes), ctypes.c_void_p(flags[0].data_ptr()), ctypes.c_void_p(residual.data_ptr()),
            ctypes.c_void_p(weight.data_ptr()), ctypes.c_float(1e-6), ctypes.c_int(0), ctypes.c_int(2), ctypes.c_int(rows), ctypes.c_int(cols),
            ctypes.c_int(bf), _stream())

    assert fused(3, 1024) != 0                    # rows not a multiple of world
    assert fused(2, 1028) != 0                    # cols not a multiple of 8
    assert fused(2, 16384) != 0                   # a row longer than one block handles
    torch.cuda.synchronize()
    assert _status(lib, flags) == 0               # nothing was launched
    assert int(flags[0][0].item()) == 0
