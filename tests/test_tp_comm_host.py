"""Host-side checks of the peer all-reduce plumbing that need no GPU: the module imports without CUDA, and the
argument rules of ``PeerAllReduce`` (message size, divisibility by the rank count) are enforced before any launch."""
import importlib

import pytest

from util import entry, nvk


def _module():
    nvk()                                   # registers the package under its importable name
    return importlib.import_module("benchmarks.tp_comm")


def test_module_imports_without_cuda():
    mod = _module()
    assert hasattr(mod, "PeerAllReduce")


class _Unlaunchable:
    """Stands in for the library handle: any attempt to launch fails the test."""

    launch_count = 0

    def lib(self):
        raise AssertionError("a launch was attempted")


def _bare(world, max_elems):
    comm = object.__new__(_module().PeerAllReduce)     # no buffers: only the argument checks are exercised
    comm.world, comm.max_elems, comm.rank = world, max_elems, 0
    comm.nvk, comm.torch = _Unlaunchable(), None
    comm.addend = comm.result = comm.normed = None
    return comm


def test_argument_rules_are_checked_before_any_launch():
    comm = _bare(world=4, max_elems=4096)
    with pytest.raises(ValueError):
        comm.all_reduce(4096 + 32)          # larger than the peer buffers
    with pytest.raises(ValueError):
        comm.all_reduce(40)                 # not a multiple of 8 * world
    with pytest.raises(ValueError):
        comm.all_reduce_add_rmsnorm(None, None, 1e-6, rows=6, cols=64)      # rows not a multiple of world
    with pytest.raises(ValueError):
        comm.all_reduce_add_rmsnorm(None, None, 1e-6, rows=8, cols=1024)    # message larger than the buffers
    with pytest.raises(ValueError):
        comm.buffers(8, 1024)
