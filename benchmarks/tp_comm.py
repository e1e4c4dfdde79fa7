"""Peer-memory all-reduce for the tensor-parallel decoder (plumbing around ``nvk_tp_allreduce``).

One process per GPU.  Every rank allocates a staging area and a flag area with ``cudaMalloc`` (through cuda-python),
publishes the staging area's CUDA IPC handle over the existing ``torch.distributed`` group and maps the peers' staging
areas with ``cudaIpcOpenMemHandle`` (plain peer mappings over NVLink; no multicast object is created).  Addend, result
and norm buffers are ordinary torch tensors of the owning rank: peers never touch them, the row-parallel GEMMs write
straight into the addend (``torch.matmul(..., out=...)``) and the kernel leaves the sum in the result buffer.
Replaces ``NcclTensorParallelCommunicator::all_reduce_sum`` (src/utils/tensor_parallel.cpp:331-353 of the reference)
for messages of up to ``max_elems`` 16-bit elements.
"""
from __future__ import annotations

import ctypes


def _check(err, what):
    code = int(err)
    if code != 0:
        raise RuntimeError(f"{what} failed with CUDA error {code}")


def declare(lib) -> None:
    """ctypes signatures of the all-reduce entry points (include/nvk.h)."""
    lib.nvk_tp_allreduce_flag_bytes.restype = ctypes.c_size_t
    lib.nvk_tp_allreduce_stage_bytes.restype = ctypes.c_size_t
    lib.nvk_tp_allreduce_stage_bytes.argtypes = [ctypes.c_int64]
    lib.nvk_tp_allreduce_set_wait_limit_ms.restype = None
    lib.nvk_tp_allreduce_set_wait_limit_ms.argtypes = [ctypes.c_int]


class PeerAllReduce:
    def __init__(self, nvk, torch, dist, dev, rank: int, world: int, max_elems: int, dtype):
        from cuda.bindings import runtime as cudart
        self.nvk, self.torch, self.dist, self.dev = nvk, torch, dist, dev
        self.rank, self.world, self.max_elems, self.dtype = rank, world, int(max_elems), dtype
        self._cudart = cudart
        lib = nvk.lib()
        declare(lib)
        self.stage_bytes = int(lib.nvk_tp_allreduce_stage_bytes(self.max_elems))
        flag_bytes = (int(lib.nvk_tp_allreduce_flag_bytes()) + 255) // 256 * 256
        self._own = {}
        for name, nbytes in (("stage", self.stage_bytes), ("flags", flag_bytes)):
            err, ptr = cudart.cudaMalloc(nbytes)
            _check(err, "cudaMalloc")
            _check(cudart.cudaMemset(ptr, 0, nbytes)[0], "cudaMemset")
            self._own[name] = (int(ptr), nbytes)
        err, handle = cudart.cudaIpcGetMemHandle(self._own["stage"][0])
        _check(err, "cudaIpcGetMemHandle")
        _check(cudart.cudaDeviceSynchronize()[0], "cudaDeviceSynchronize")
        gathered = [None] * world
        dist.all_gather_object(gathered, bytes(handle.reserved))
        self._opened = []
        stage = [0] * world
        for r in range(world):
            if r == rank:
                stage[r] = self._own["stage"][0]
                continue
            h = cudart.cudaIpcMemHandle_t()
            h.reserved = gathered[r]
            err, ptr = cudart.cudaIpcOpenMemHandle(h, cudart.cudaIpcMemLazyEnablePeerAccess)
            _check(err, "cudaIpcOpenMemHandle")
            self._opened.append(int(ptr))
            stage[r] = int(ptr)
        self._stage_tab = (ctypes.c_void_p * world)(*stage)
        self._flags = ctypes.c_void_p(self._own["flags"][0])
        self.addend = torch.zeros(self.max_elems, device=dev, dtype=dtype)   # this rank's addend
        self.result = torch.zeros(self.max_elems, device=dev, dtype=dtype)   # the sum
        self.normed = torch.zeros(self.max_elems, device=dev, dtype=dtype)   # rmsnorm of (residual + sum)
        torch.cuda.synchronize()
        dist.barrier()   # every rank has mapped every staging area before anyone launches

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
        nvk._check(nvk.lib().nvk_tp_allreduce(
            ctypes.c_void_p(self.addend.data_ptr()), ctypes.c_void_p(self.result.data_ptr()), self._stage_tab,
            ctypes.c_size_t(self.stage_bytes), self._flags, ctypes.c_int(self.rank), ctypes.c_int(self.world),
            ctypes.c_int64(count), ctypes.c_int(nvk._dtype_code(self.addend)), stream))
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
            ctypes.c_void_p(self.addend.data_ptr()), ctypes.c_void_p(self.result.data_ptr()),
            ctypes.c_void_p(self.normed.data_ptr()), self._stage_tab, ctypes.c_size_t(self.stage_bytes), self._flags,
            ctypes.c_void_p(residual.data_ptr()), ctypes.c_void_p(weight.data_ptr()), ctypes.c_float(eps),
            ctypes.c_int(self.rank), ctypes.c_int(self.world), ctypes.c_int(rows), ctypes.c_int(cols),
            ctypes.c_int(nvk._dtype_code(self.addend)), stream))
        nvk.launch_count += 1
        return self.result[:n].view(rows, cols), self.normed[:n].view(rows, cols)

    def row_linear_all_reduce_add_rmsnorm(self, x, weight, residual, norm_weight, eps: float):
        """``h = residual + sum over ranks of x @ weight.T``, ``x_norm = rmsnorm(h) * norm_weight``: this library's GEMM whose
        epilogue pushes the partial sums to the ranks that reduce them, then the all-reduce kernel without its own push."""
        nvk, torch = self.nvk, self.torch
        rows, cols = x.shape[0], weight.shape[0]
        n = rows * cols
        if n > self.max_elems or rows % self.world != 0:
            raise ValueError("rows must be a multiple of world and the message must fit the peer buffers")
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        nvk._check(nvk.lib().nvk_tp_row_linear_allreduce_add_rmsnorm(
            ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(weight.data_ptr()), ctypes.c_int64(rows), ctypes.c_int64(cols),
            ctypes.c_int64(weight.shape[1]), ctypes.c_void_p(self.addend.data_ptr()), ctypes.c_void_p(self.result.data_ptr()),
            ctypes.c_void_p(self.normed.data_ptr()), self._stage_tab, ctypes.c_size_t(self.stage_bytes), self._flags,
            ctypes.c_void_p(residual.data_ptr()), ctypes.c_void_p(norm_weight.data_ptr()), ctypes.c_float(eps), ctypes.c_int(self.rank),
            ctypes.c_int(self.world), ctypes.c_int(nvk._dtype_code(self.addend)), stream))
        nvk.launch_count += 2
        return self.result[:n].view(rows, cols), self.normed[:n].view(rows, cols)

    def status(self) -> int:
        """0 when every wait on the peers completed; 1 / 2 when a peer's data never arrived (synchronises the stream)."""
        out = ctypes.c_int(0)
        stream = ctypes.c_void_p(self.torch.cuda.current_stream().cuda_stream)
        self.nvk._check(self.nvk.lib().nvk_tp_allreduce_status(self._flags, stream, ctypes.byref(out)))
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


class MulticastAllReduce:
    """The all-reduce through the NVSwitch (``nvk_tp_allreduce_multimem`` / ``nvk_tp_allreduce_add_rmsnorm_multimem``).  Addend,
    result and norm buffers and the signal area are carved out of one symmetric allocation made with torch's symmetric
    memory (which creates the NVLink multicast object and binds every rank's part to it); the flag area is private.
    Same ``buffers`` / ``all_reduce`` / ``all_reduce_add_rmsnorm`` / ``status`` / ``close`` surface as ``PeerAllReduce``.
    Raises ``RuntimeError`` when the group has no multicast support."""

    def __init__(self, nvk, torch, dist, dev, rank: int, world: int, max_elems: int, dtype):
        import torch.distributed._symmetric_memory as symm_mem
        self.nvk, self.torch, self.dist, self.dev = nvk, torch, dist, dev
        self.rank, self.world, self.max_elems, self.dtype = rank, world, int(max_elems), dtype
        lib = nvk.lib()
        declare(lib)
        lib.nvk_tp_allreduce_signal_bytes.restype = ctypes.c_size_t
        esize = torch.empty((), dtype=dtype).element_size()
        part = (self.max_elems * esize + 4095) // 4096 * 4096
        signal_bytes = (int(lib.nvk_tp_allreduce_signal_bytes()) + 4095) // 4096 * 4096
        total = 3 * part + signal_bytes
        group = dist.group.WORLD
        try:
            symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:   # newer torch enables every group by itself
            pass
        self._buf = symm_mem.empty(total, dtype=torch.uint8, device=dev)
        self._buf.zero_()
        torch.cuda.synchronize()
        self._hdl = symm_mem.rendezvous(self._buf, group.group_name)
        mc = int(getattr(self._hdl, "multicast_ptr", 0) or 0)
        if mc == 0:
            raise RuntimeError("this process group has no NVLink multicast support")
        peers = [int(x) for x in self._hdl.buffer_ptrs]
        self._mc_in, self._mc_out = mc, mc + part
        self._signal_tab = (ctypes.c_void_p * world)(*[x + 3 * part for x in peers])
        view = lambda k: self._buf[k * part: k * part + self.max_elems * esize].view(dtype)  # noqa: E731
        self.addend, self.result, self.normed = view(0), view(1), view(2)
        self._flag_t = torch.zeros(64, device=dev, dtype=torch.int32)
        self._flags = ctypes.c_void_p(self._flag_t.data_ptr())
        torch.cuda.synchronize()
        dist.barrier()

    def buffers(self, rows: int, cols: int):
        n = rows * cols
        if n > self.max_elems:
            raise ValueError("message larger than the symmetric buffers")
        return self.addend[:n].view(rows, cols), self.result[:n].view(rows, cols)

    def all_reduce(self, count: int, cols: int = 0) -> None:
        """Sums the first ``count`` elements of every rank's addend buffer into every rank's result buffer."""
        nvk, torch = self.nvk, self.torch
        cols = cols or min(count // self.world, 4096)
        rows = count // cols
        if rows * cols != count or rows % self.world or cols % 8 or count > self.max_elems:
            raise ValueError("count must split into rows % world == 0 of cols % 8 == 0 elements")
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        nvk._check(nvk.lib().nvk_tp_allreduce_multimem(
            ctypes.c_void_p(self._mc_in), ctypes.c_void_p(self._mc_out), self._signal_tab, self._flags, ctypes.c_int(self.rank),
            ctypes.c_int(self.world), ctypes.c_int(rows), ctypes.c_int(cols), ctypes.c_int(nvk._dtype_code(self.addend)), stream))
        nvk.launch_count += 1

    def all_reduce_add_rmsnorm(self, residual, weight, eps: float, rows: int, cols: int):
        nvk, torch = self.nvk, self.torch
        n = rows * cols
        if n > self.max_elems or rows % self.world != 0:
            raise ValueError("rows must be a multiple of world and the message must fit the symmetric buffers")
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        nvk._check(nvk.lib().nvk_tp_allreduce_add_rmsnorm_multimem(
            ctypes.c_void_p(self._mc_in), ctypes.c_void_p(self._mc_out), ctypes.c_void_p(self.result.data_ptr()),
            ctypes.c_void_p(self.normed.data_ptr()), self._signal_tab, self._flags,
            ctypes.c_void_p(residual.data_ptr()), ctypes.c_void_p(weight.data_ptr()), ctypes.c_float(eps), ctypes.c_int(self.rank),
            ctypes.c_int(self.world), ctypes.c_int(rows), ctypes.c_int(cols), ctypes.c_int(nvk._dtype_code(self.addend)), stream))
        nvk.launch_count += 1
        return self.result[:n].view(rows, cols), self.normed[:n].view(rows, cols)

    def status(self) -> int:
        out = ctypes.c_int(0)
        stream = ctypes.c_void_p(self.torch.cuda.current_stream().cuda_stream)
        self.nvk._check(self.nvk.lib().nvk_tp_allreduce_status(self._flags, stream, ctypes.byref(out)))
        return int(out.value)

    def close(self) -> None:
        # every rank stops launching before any rank lets go of the symmetric allocation
        self.torch.cuda.synchronize()
        self.dist.barrier()
        self.addend = self.result = self.normed = None
        self._hdl = None
        self._buf = None
        self.torch.cuda.synchronize()
        self.dist.barrier()


class InProcessAllReduce:
    """``world`` ranks on ONE device (``nvk_tp_allreduce_inprocess``): a buffer set per rank, one cooperative launch per
    collective.  The counterpart of the reference's in-process communicator (src/utils/tensor_parallel.cpp:165-277)."""

    def __init__(self, nvk, torch, dev, world: int, max_elems: int, dtype):
        self.nvk, self.torch, self.world, self.max_elems, self.dtype = nvk, torch, world, int(max_elems), dtype
        lib = nvk.lib()
        declare(lib)
        self.stage_bytes = int(lib.nvk_tp_allreduce_stage_bytes(self.max_elems))
        flag_words = int(lib.nvk_tp_allreduce_flag_bytes()) // 4
        mk = lambda: [torch.zeros(self.max_elems, device=dev, dtype=dtype) for _ in range(world)]  # noqa: E731
        self.addend, self.result, self.normed = mk(), mk(), mk()
        self.stage = [torch.zeros(self.stage_bytes, device=dev, dtype=torch.uint8) for _ in range(world)]
        self.flags = [torch.zeros(flag_words, device=dev, dtype=torch.int32) for _ in range(world)]
        self._tab = lambda ts: (ctypes.c_void_p * world)(*[t.data_ptr() for t in ts])  # noqa: E731

    def launch(self, rows: int, cols: int, residuals=None, weight=None, eps: float = 1e-6) -> None:
        """Plain sum when ``residuals`` is None, else the fused form with one residual tensor per rank."""
        nvk, torch = self.nvk, self.torch
        fused = residuals is not None
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        nvk._check(nvk.lib().nvk_tp_allreduce_inprocess(
            self._tab(self.addend), self._tab(self.result), self._tab(self.normed) if fused else None, self._tab(self.stage),
            ctypes.c_size_t(self.stage_bytes), self._tab(self.flags), self._tab(residuals) if fused else None,
            ctypes.c_void_p(weight.data_ptr()) if fused else None, ctypes.c_float(eps), ctypes.c_int(self.world),
            ctypes.c_int(rows), ctypes.c_int(cols), ctypes.c_int(nvk._dtype_code(self.addend[0])), stream))
        nvk.launch_count += 1

    def row_linear_launch(self, xs, weights, residuals, norm_weight, eps: float = 1e-6) -> None:
        """Every rank's row-parallel GEMM (its epilogue pushing the partial sums) and the fused all-reduce that skips its push."""
        nvk, torch = self.nvk, self.torch
        rows, cols = xs[0].shape[0], weights[0].shape[0]
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        nvk._check(nvk.lib().nvk_tp_row_linear_allreduce_add_rmsnorm_inprocess(
            self._tab(xs), self._tab(weights), ctypes.c_int64(rows), ctypes.c_int64(cols), ctypes.c_int64(weights[0].shape[1]),
            self._tab(self.addend), self._tab(self.result), self._tab(self.normed), self._tab(self.stage),
            ctypes.c_size_t(self.stage_bytes), self._tab(self.flags), self._tab(residuals), ctypes.c_void_p(norm_weight.data_ptr()),
            ctypes.c_float(eps), ctypes.c_int(self.world), ctypes.c_int(nvk._dtype_code(self.addend[0])), stream))
        nvk.launch_count += self.world + 1

    def status(self, rank: int = 0) -> int:
        out = ctypes.c_int(0)
        stream = ctypes.c_void_p(self.torch.cuda.current_stream().cuda_stream)
        self.nvk._check(self.nvk.lib().nvk_tp_allreduce_status(ctypes.c_void_p(self.flags[rank].data_ptr()), stream, ctypes.byref(out)))
        return int(out.value)
