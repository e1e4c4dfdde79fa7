"""Peer-memory all-reduce for the tensor-parallel decoder (plumbing around ``nvk_tp_allreduce``).

One process per GPU.  Every rank allocates an addend buffer, a result buffer and a flag area with ``cudaMalloc``
(through cuda-python), publishes their CUDA IPC handles over the existing ``torch.distributed`` group and maps the
peers' buffers with ``cudaIpcOpenMemHandle`` (plain peer mappings over NVLink; no multicast object is created).  The
row-parallel GEMMs write straight into the addend buffer (``torch.matmul(..., out=...)``), the kernel leaves the sum in
the result buffer of every rank.  Replaces ``NcclTensorParallelCommunicator::all_reduce_sum``
(src/utils/tensor_parallel.cpp:331-353 of the reference) for messages of up to ``max_elems`` 16-bit elements.
"""
from __future__ import annotations

import ctypes


class _DeviceBlock:
    """A cudaMalloc'ed range exposed to torch through the CUDA array interface (as int16 elements)."""

    def __init__(self, ptr: int, nbytes: int):
        self.ptr, self.nbytes = ptr, nbytes
        self.__cuda_array_interface__ = {"shape": (nbytes // 2,), "typestr": "<i2", "data": (ptr, False), "version": 2}


def _check(err, what):
    code = int(err)
    if code != 0:
        raise RuntimeError(f"{what} failed with CUDA error {code}")


class PeerAllReduce:
    def __init__(self, nvk, torch, dist, dev, rank: int, world: int, max_elems: int, dtype):
        from cuda.bindings import runtime as cudart
        self.nvk, self.torch, self.dist, self.dev = nvk, torch, dist, dev
        self.rank, self.world, self.max_elems, self.dtype = rank, world, int(max_elems), dtype
        self._cudart = cudart
        lib = nvk.lib()
        lib.nvk_tp_allreduce_flag_bytes.restype = ctypes.c_size_t
        flag_bytes = int(lib.nvk_tp_allreduce_flag_bytes())
        sizes = {"in": self.max_elems * 2, "out": self.max_elems * 2, "norm": self.max_elems * 2,
                 "flags": (flag_bytes + 255) // 256 * 256}
        self._own, handles = {}, {}
        for name, nbytes in sizes.items():
            err, ptr = cudart.cudaMalloc(nbytes)
            _check(err, "cudaMalloc")
            _check(cudart.cudaMemset(ptr, 0, nbytes)[0], "cudaMemset")
            err, handle = cudart.cudaIpcGetMemHandle(ptr)
            _check(err, "cudaIpcGetMemHandle")
            self._own[name] = (int(ptr), nbytes)
            handles[name] = bytes(handle.reserved)
        _check(cudart.cudaDeviceSynchronize()[0], "cudaDeviceSynchronize")
        gathered = [None] * world
        dist.all_gather_object(gathered, handles)
        self._opened = []
        self._ptrs = {name: [0] * world for name in sizes}
        for r in range(world):
            for name in sizes:
                if r == rank:
                    self._ptrs[name][r] = self._own[name][0]
                    continue
                handle = cudart.cudaIpcMemHandle_t()
                handle.reserved = gathered[r][name]
                err, ptr = cudart.cudaIpcOpenMemHandle(handle, cudart.cudaIpcMemLazyEnablePeerAccess)
                _check(err, "cudaIpcOpenMemHandle")
                self._opened.append(int(ptr))
                self._ptrs[name][r] = int(ptr)
        arr = ctypes.c_void_p * world
        self._in_tab = arr(*self._ptrs["in"])
        self._out_tab = arr(*self._ptrs["out"])
        self._flag_tab = arr(*self._ptrs["flags"])
        self._norm_tab = arr(*self._ptrs["norm"])
        self._norm_block = _DeviceBlock(*self._own["norm"])
        self._in_block = _DeviceBlock(*self._own["in"])
        self._out_block = _DeviceBlock(*self._own["out"])
        self.addend = torch.as_tensor(self._in_block, device=dev).view(dtype)    # [max_elems], this rank's addend
        self.result = torch.as_tensor(self._out_block, device=dev).view(dtype)   # [max_elems], the sum
        self.normed = torch.as_tensor(self._norm_block, device=dev).view(dtype)  # [max_elems], rmsnorm of (residual + sum)
        dist.barrier()   # every rank has mapped every buffer before anyone launches

    def buffers(self, rows: int, cols: int):
        """Views of the addend and result buffers shaped [rows, cols]."""
        n = rows * cols
        if n > self.max_elems:
            raise ValueError("message larger than the peer buffers")
        return self.addend[:n].view(rows, cols), self.result[:n].view(rows, cols)

    def all_reduce(self, count: int) -> None:
        """Sums the first ``count`` elements of every rank's addend buffer into every rank's result buffer."""
        nvk, torch = self.nvk, self.torch
        if count % (8 * self.world) != 0 or count > self.max_elems:
            raise ValueError("count must be a multiple of 8 * world and fit the peer buffers")
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        nvk._check(nvk.lib().nvk_tp_allreduce(self._in_tab, self._out_tab, self._flag_tab, ctypes.c_int(self.rank),
                                              ctypes.c_int(self.world), ctypes.c_int64(count),
                                              ctypes.c_int(nvk._dtype_code(self.addend)), stream))
        nvk.launch_count += 1

    def all_reduce_add_rmsnorm(self, residual, weight, eps: float, rows: int, cols: int):
        """``h = residual + sum of every rank's addend``, ``x = rmsnorm(h) * weight`` in one launch; returns views of
        this rank's result and norm buffers shaped [rows, cols].  ``residual`` may be the result buffer itself."""
        nvk, torch = self.nvk, self.torch
        n = rows * cols
        if n > self.max_elems or rows % self.world != 0:
            raise ValueError("rows must be a multiple of world and the message must fit the peer buffers")
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        nvk._check(nvk.lib().nvk_tp_allreduce_add_rmsnorm(
            self._in_tab, self._out_tab, self._norm_tab, self._flag_tab, ctypes.c_void_p(residual.data_ptr()),
            ctypes.c_void_p(weight.data_ptr()), ctypes.c_float(eps), ctypes.c_int(self.rank), ctypes.c_int(self.world),
            ctypes.c_int(rows), ctypes.c_int(cols), ctypes.c_int(nvk._dtype_code(self.addend)), stream))
        nvk.launch_count += 1
        return self.result[:n].view(rows, cols), self.normed[:n].view(rows, cols)

    def status(self) -> int:
        """0 when every wait on the peers completed; 1 / 2 when a peer never arrived (synchronises the stream)."""
        out = ctypes.c_int(0)
        stream = ctypes.c_void_p(self.torch.cuda.current_stream().cuda_stream)
        self.nvk._check(self.nvk.lib().nvk_tp_allreduce_status(ctypes.c_void_p(self._own["flags"][0]), stream, ctypes.byref(out)))
        return int(out.value)

    def close(self) -> None:
        cudart = self._cudart
        self.torch.cuda.synchronize()
        self.dist.barrier()
        for ptr in self._opened:
            cudart.cudaIpcCloseMemHandle(ptr)
        self._opened = []
        self.dist.barrier()   # nobody frees a buffer that a peer still has mapped
        for ptr, _ in self._own.values():
            cudart.cudaFree(ptr)
        self._own = {}
