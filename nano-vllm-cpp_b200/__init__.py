"""Python test/bench driver over the C ABI of ``libnvk.so`` (``include/nvk.h``).

The product is the shared library; this module only loads it with ``ctypes`` and passes raw
device pointers of torch tensors (torch is plumbing: device memory and streams).  The function
names and argument order mirror the reference's operator API
(include/kernels/kvcache.h:7-12, include/kernels/attention.h:7-41,
include/kernels/split_qkv.h:22-33).  There is no fallback: if the CUDA library is missing or a
call fails, an exception is raised (``ValueError`` for invalid arguments, ``RuntimeError`` for
CUDA errors -- the reference throws std::invalid_argument / std::runtime_error).

The directory name contains a hyphen, so import it with :func:`load_package` from
``__graft_entry__`` (or ``importlib``) rather than with an ``import`` statement.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libnvk.so")

F16, BF16, F32, I32, I64, I8 = 0, 1, 2, 3, 4, 5
OK, ERR_INVALID_ARGUMENT, ERR_CUDA, ERR_UNSUPPORTED = 0, 1, 2, 3

EXPORTED_SYMBOLS = (
    "nvk_abi_version", "nvk_last_error", "nvk_store_kvcache", "nvk_fused_split_norm_rope_store",
    "nvk_decode_attention_workspace_bytes", "nvk_decode_attention_paged",
    "nvk_prefill_attention_varlen", "nvk_decode_attention_paged_static",
    "nvk_store_kvcache_int8", "nvk_decode_attention_paged_int8",
    "nvk_tp_allreduce_flag_bytes", "nvk_tp_allreduce_stage_bytes", "nvk_tp_allreduce_set_wait_limit_ms", "nvk_tp_allreduce",
    "nvk_tp_allreduce_status", "nvk_tp_allreduce_reset", "nvk_tp_allreduce_add_rmsnorm", "nvk_tp_allreduce_inprocess",
    "nvk_prefill_status", "nvk_decode_attention_static_scratch_bytes", "nvk_attention_mixed_step",
    "nvk_linear", "nvk_qkv_linear_norm_rope_store", "nvk_tp_row_linear_allreduce_add_rmsnorm",
    "nvk_tp_row_linear_allreduce_add_rmsnorm_inprocess", "nvk_gemm_status",
    "nvk_tp_allreduce_signal_bytes", "nvk_tp_allreduce_multimem", "nvk_tp_allreduce_add_rmsnorm_multimem",
    "nvk_store_kvcache_fp8", "nvk_decode_attention_paged_fp8",
)

_lib = None
launch_count = 0  # kernels launched through this module (claimed by the benchmark)


class NvkLibraryMissing(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """Loads ``libnvk.so``; raises if it has not been built (no CPU or library fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NvkLibraryMissing(
                f"{LIB_PATH} not found: build it with `python nano-vllm-cpp_b200/build.py` "
                "(or __graft_entry__.build()); there is no fallback path")
        L = ctypes.CDLL(LIB_PATH)
        L.nvk_last_error.restype = ctypes.c_char_p
        L.nvk_abi_version.restype = ctypes.c_int
        L.nvk_decode_attention_workspace_bytes.restype = ctypes.c_size_t
        L.nvk_decode_attention_workspace_bytes.argtypes = [
            ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int]
        L.nvk_decode_attention_static_scratch_bytes.restype = ctypes.c_size_t
        _lib = L
    return _lib


def _check(rc: int) -> None:
    if rc == OK:
        return
    msg = lib().nvk_last_error().decode()
    if rc in (ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED):
        raise ValueError(msg)
    raise RuntimeError(msg)


def _dtype_code(t) -> int:
    import torch
    return {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32, torch.int32: I32,
            torch.int64: I64, torch.int8: I8}[t.dtype]


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _stream():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _index(name, t):
    """(pointer, dtype code) of an index tensor; int32 and int64 are accepted, as by the reference's kernels."""
    if t is None:
        return ctypes.c_void_p(0), ctypes.c_int(I32)
    import torch
    if t.dtype not in (torch.int32, torch.int64):
        raise ValueError(f"{name} must be int32 or int64")
    return _ptr(t), ctypes.c_int(_dtype_code(t))


def _require_cuda(name, t):
    if t is None:
        raise ValueError(f"{name} must be defined")
    if not t.is_cuda:
        raise ValueError(f"{name} must live on CUDA")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def store_kvcache(key, value, k_cache, v_cache, slot_mapping) -> None:
    """``store_kvcache`` (include/kernels/kvcache.h:7-12): in-place scatter into the paged cache."""
    global launch_count
    for n, t in (("key", key), ("value", value), ("k_cache", k_cache), ("v_cache", v_cache),
                 ("slot_mapping", slot_mapping)):
        _require_cuda(n, t)
    if not (key.dtype == value.dtype == k_cache.dtype == v_cache.dtype):
        raise ValueError("key and value must have the same dtype")
    n = slot_mapping.numel()
    if n <= 0:
        raise ValueError("slot_mapping must contain at least one element")
    if key.numel() % n or key.numel() != value.numel():
        raise ValueError("key cannot be flattened by the provided leading count")
    row = key.numel() // n
    if k_cache.numel() % row or k_cache.numel() != v_cache.numel():
        raise ValueError("k_cache does not contain an integer number of cache rows")
    _check(lib().nvk_store_kvcache(
        _ptr(key), _ptr(value), _ptr(k_cache), _ptr(v_cache), _ptr(slot_mapping),
        ctypes.c_int(_dtype_code(slot_mapping)), ctypes.c_int64(n), ctypes.c_int64(row),
        ctypes.c_int64(k_cache.numel() // row), ctypes.c_int(_dtype_code(key)), _stream()))
    launch_count += 1


def fused_split_norm_rope_store(qkv, positions, q_norm_weight, k_norm_weight, norm_eps, cos_sin_cache,
                                slot_mapping, k_cache, v_cache, num_q_heads, num_kv_heads, head_dim,
                                q_out) -> None:
    """``fused_split_norm_rope_store`` (include/kernels/split_qkv.h:22-33).  ``slot_mapping=None`` writes k / v of
    row r to row r of ``k_cache`` / ``v_cache`` (plain [rows, Hkv, D] tensors); both norm weights ``None`` skips the
    RMSNorm -- the two forms that serve the reference's unfused route (split_qkv, optional norm, rotary)."""
    global launch_count
    for n, t in (("qkv", qkv), ("positions", positions), ("cos_sin_cache", cos_sin_cache),
                 ("k_cache", k_cache), ("v_cache", v_cache), ("q_out", q_out)):
        _require_cuda(n, t)
    for n, t in (("q_norm_weight", q_norm_weight), ("k_norm_weight", k_norm_weight), ("slot_mapping", slot_mapping)):
        if t is not None:
            _require_cuda(n, t)
    row = num_kv_heads * head_dim
    _check(lib().nvk_fused_split_norm_rope_store(
        _ptr(qkv), _ptr(positions), _ptr(q_norm_weight), _ptr(k_norm_weight), ctypes.c_float(norm_eps),
        _ptr(cos_sin_cache), ctypes.c_int64(cos_sin_cache.shape[0]), _ptr(slot_mapping), _ptr(k_cache),
        _ptr(v_cache), ctypes.c_int64(k_cache.numel() // row), ctypes.c_int64(qkv.shape[0]),
        ctypes.c_int(num_q_heads), ctypes.c_int(num_kv_heads), ctypes.c_int(head_dim), _ptr(q_out),
        ctypes.c_int(_dtype_code(qkv)), _stream()))
    launch_count += 1


def decode_attention_workspace_bytes(batch, num_heads, num_kv_heads, head_dim, max_blocks, block_size) -> int:
    return int(lib().nvk_decode_attention_workspace_bytes(batch, num_heads, num_kv_heads, head_dim,
                                                          max_blocks, block_size))


def launch_decode_attention_paged(query, k_cache, v_cache, context_lens, block_tables, num_kv_heads,
                                  head_dim, block_size, scale, output, workspace=None) -> None:
    """``launch_decode_attention_paged`` (include/kernels/attention.h:31-41).

    ``workspace`` (a uint8 CUDA tensor of ``decode_attention_workspace_bytes`` bytes) plays the role
    of the allocator argument of ``flash_attn_decode_kvcache`` (include/kernels/flash_attn.h:39-50).
    """
    global launch_count
    for n, t in (("query", query), ("k_cache", k_cache), ("v_cache", v_cache),
                 ("context_lens", context_lens), ("block_tables", block_tables), ("output", output)):
        _require_cuda(n, t)
    batch, num_heads = query.shape[0], query.shape[1]
    num_cache_blocks = k_cache.numel() // (block_size * num_kv_heads * head_dim)
    _check(lib().nvk_decode_attention_paged(
        _ptr(query), _ptr(k_cache), _ptr(v_cache), *_index("context_lens", context_lens),
        *_index("block_tables", block_tables), ctypes.c_int64(batch), ctypes.c_int64(block_tables.shape[1]), ctypes.c_int64(num_cache_blocks),
        ctypes.c_int(num_heads), ctypes.c_int(num_kv_heads), ctypes.c_int(head_dim),
        ctypes.c_int(block_size), ctypes.c_float(scale), _ptr(output), ctypes.c_int(_dtype_code(query)),
        _ptr(workspace), ctypes.c_size_t(workspace.numel() * workspace.element_size() if workspace is not None else 0),
        _stream()))
    ws_need = decode_attention_workspace_bytes(batch, num_heads, num_kv_heads, head_dim,
                                               block_tables.shape[1], block_size)
    launch_count += 2 if (workspace is not None and ws_need > 0) else 1


def launch_decode_attention_paged_static(query, k_cache, v_cache, context_lens, block_tables, num_kv_heads,
                                         head_dim, block_size, scale, output) -> None:
    """Decode attention for callers that may not allocate: split-K scratch comes from a 32 MiB array
    inside the library (``nvk_decode_attention_paged_static``).  Calls on one device must not overlap."""
    global launch_count
    for n, t in (("query", query), ("k_cache", k_cache), ("v_cache", v_cache),
                 ("context_lens", context_lens), ("block_tables", block_tables), ("output", output)):
        _require_cuda(n, t)
    batch, num_heads = query.shape[0], query.shape[1]
    num_cache_blocks = k_cache.numel() // (block_size * num_kv_heads * head_dim)
    _check(lib().nvk_decode_attention_paged_static(
        _ptr(query), _ptr(k_cache), _ptr(v_cache), *_index("context_lens", context_lens),
        *_index("block_tables", block_tables), ctypes.c_int64(batch), ctypes.c_int64(block_tables.shape[1]), ctypes.c_int64(num_cache_blocks),
        ctypes.c_int(num_heads), ctypes.c_int(num_kv_heads), ctypes.c_int(head_dim),
        ctypes.c_int(block_size), ctypes.c_float(scale), _ptr(output), ctypes.c_int(_dtype_code(query)),
        _stream()))
    launch_count += 2


def store_kvcache_int8(key, value, k_cache, v_cache, k_scale, v_scale, slot_mapping) -> None:
    """``store_kvcache_int8`` (include/kernels/kvcache.h:14-24): quantising scatter into int8 caches + fp16 scales."""
    global launch_count
    import torch
    for n, t in (("key", key), ("value", value), ("k_cache", k_cache), ("v_cache", v_cache), ("k_scale", k_scale),
                 ("v_scale", v_scale), ("slot_mapping", slot_mapping)):
        _require_cuda(n, t)
    if k_cache.dtype != torch.int8 or v_cache.dtype != torch.int8:
        raise ValueError("store_kvcache_int8 requires int8 caches")
    if k_scale.dtype != torch.float16 or v_scale.dtype != torch.float16:
        raise ValueError("store_kvcache_int8 requires float16 scales")
    if key.dim() != 3:
        raise ValueError("key must be rank-3 for int8 store")
    if slot_mapping.dtype.itemsize != 4:
        raise ValueError("slot_mapping must be int32")
    hkv, d = key.shape[1], key.shape[2]
    _check(lib().nvk_store_kvcache_int8(
        _ptr(key), _ptr(value), _ptr(k_cache), _ptr(v_cache), _ptr(k_scale), _ptr(v_scale), _ptr(slot_mapping),
        ctypes.c_int64(slot_mapping.numel()), ctypes.c_int(hkv), ctypes.c_int(d),
        ctypes.c_int64(k_cache.numel() // (hkv * d)), ctypes.c_int(_dtype_code(key)), _stream()))
    launch_count += 1


def launch_decode_attention_paged_int8(query, k_cache, v_cache, k_scale, v_scale, context_lens, block_tables,
                                       num_kv_heads, head_dim, block_size, scale, output, workspace=None) -> None:
    """``launch_decode_attention_paged_int8`` (include/kernels/attention.h:43-56), with the optional split-K workspace
    of :func:`launch_decode_attention_paged`."""
    global launch_count
    for n, t in (("query", query), ("k_cache", k_cache), ("v_cache", v_cache), ("k_scale", k_scale), ("v_scale", v_scale),
                 ("context_lens", context_lens), ("block_tables", block_tables), ("output", output)):
        _require_cuda(n, t)
    batch, num_heads = query.shape[0], query.shape[1]
    num_cache_blocks = k_cache.numel() // (block_size * num_kv_heads * head_dim)
    _check(lib().nvk_decode_attention_paged_int8(
        _ptr(query), _ptr(k_cache), _ptr(v_cache), _ptr(k_scale), _ptr(v_scale), *_index("context_lens", context_lens),
        *_index("block_tables", block_tables), ctypes.c_int64(batch), ctypes.c_int64(block_tables.shape[1]), ctypes.c_int64(num_cache_blocks),
        ctypes.c_int(num_heads), ctypes.c_int(num_kv_heads), ctypes.c_int(head_dim), ctypes.c_int(block_size),
        ctypes.c_float(scale), _ptr(output), ctypes.c_int(_dtype_code(query)), _ptr(workspace),
        ctypes.c_size_t(workspace.numel() * workspace.element_size() if workspace is not None else 0), _stream()))
    ws_need = decode_attention_workspace_bytes(batch, num_heads, num_kv_heads, head_dim, block_tables.shape[1], block_size)
    launch_count += 2 if (workspace is not None and ws_need > 0) else 1


def store_kvcache_fp8(key, value, k_cache, v_cache, k_scale, v_scale, slot_mapping) -> None:
    """Quantising scatter into e4m3 caches (uint8 or float8_e4m3fn tensors) + fp16 scales (``nvk_store_kvcache_fp8``)."""
    global launch_count
    import torch
    for n, t in (("key", key), ("value", value), ("k_cache", k_cache), ("v_cache", v_cache), ("k_scale", k_scale),
                 ("v_scale", v_scale), ("slot_mapping", slot_mapping)):
        _require_cuda(n, t)
    if k_cache.element_size() != 1 or v_cache.element_size() != 1:
        raise ValueError("store_kvcache_fp8 requires one-byte caches")
    if k_scale.dtype != torch.float16 or v_scale.dtype != torch.float16:
        raise ValueError("store_kvcache_fp8 requires float16 scales")
    if key.dim() != 3:
        raise ValueError("key must be rank-3 for the fp8 store")
    if slot_mapping.dtype.itemsize != 4:
        raise ValueError("slot_mapping must be int32")
    hkv, d = key.shape[1], key.shape[2]
    _check(lib().nvk_store_kvcache_fp8(
        _ptr(key), _ptr(value), _ptr(k_cache), _ptr(v_cache), _ptr(k_scale), _ptr(v_scale), _ptr(slot_mapping),
        ctypes.c_int64(slot_mapping.numel()), ctypes.c_int(hkv), ctypes.c_int(d),
        ctypes.c_int64(k_cache.numel() // (hkv * d)), ctypes.c_int(_dtype_code(key)), _stream()))
    launch_count += 1


def launch_decode_attention_paged_fp8(query, k_cache, v_cache, k_scale, v_scale, context_lens, block_tables,
                                      num_kv_heads, head_dim, block_size, scale, output, workspace=None) -> None:
    """Paged decode attention over an e4m3 cache (``nvk_decode_attention_paged_fp8``)."""
    global launch_count
    for n, t in (("query", query), ("k_cache", k_cache), ("v_cache", v_cache), ("k_scale", k_scale), ("v_scale", v_scale),
                 ("context_lens", context_lens), ("block_tables", block_tables), ("output", output)):
        _require_cuda(n, t)
    batch, num_heads = query.shape[0], query.shape[1]
    num_cache_blocks = k_cache.numel() // (block_size * num_kv_heads * head_dim)
    _check(lib().nvk_decode_attention_paged_fp8(
        _ptr(query), _ptr(k_cache), _ptr(v_cache), _ptr(k_scale), _ptr(v_scale), *_index("context_lens", context_lens),
        *_index("block_tables", block_tables), ctypes.c_int64(batch), ctypes.c_int64(block_tables.shape[1]), ctypes.c_int64(num_cache_blocks),
        ctypes.c_int(num_heads), ctypes.c_int(num_kv_heads), ctypes.c_int(head_dim), ctypes.c_int(block_size),
        ctypes.c_float(scale), _ptr(output), ctypes.c_int(_dtype_code(query)), _ptr(workspace),
        ctypes.c_size_t(workspace.numel() * workspace.element_size() if workspace is not None else 0), _stream()))
    ws_need = decode_attention_workspace_bytes(batch, num_heads, num_kv_heads, head_dim, block_tables.shape[1], block_size)
    launch_count += 2 if (workspace is not None and ws_need > 0) else 1


def _prefill(query, key, value, k_cache, v_cache, cu_q, cu_k, block_tables, num_kv_heads, head_dim,
             block_size, scale, output, max_seqlen_q=0) -> None:
    global launch_count
    _require_cuda("query", query)
    _require_cuda("output", output)
    num_seqs = (cu_q.numel() - 1) if cu_q is not None else 1
    total_k = key.shape[0] if key is not None else 0
    max_blocks = block_tables.shape[1] if block_tables is not None else 0
    ncb = (k_cache.numel() // (block_size * num_kv_heads * head_dim)) if k_cache is not None else 0
    _check(lib().nvk_prefill_attention_varlen(
        _ptr(query), _ptr(key), _ptr(value), _ptr(k_cache), _ptr(v_cache), *_index("cu_seqlens_q", cu_q),
        *_index("cu_seqlens_k", cu_k), *_index("block_tables", block_tables), ctypes.c_int64(num_seqs), ctypes.c_int64(query.shape[0]), ctypes.c_int64(total_k),
        ctypes.c_int64(max_blocks), ctypes.c_int64(ncb), ctypes.c_int(max_seqlen_q),
        ctypes.c_int(query.shape[1]), ctypes.c_int(num_kv_heads), ctypes.c_int(head_dim),
        ctypes.c_int(block_size), ctypes.c_float(scale), _ptr(output), ctypes.c_int(_dtype_code(query)),
        _stream()))
    launch_count += 1


def launch_prefill_attention_dense(query, cu_seqlens_q, key, value, cu_seqlens_k, num_kv_heads, head_dim,
                                   scale, output) -> None:
    """``launch_prefill_attention_dense`` (include/kernels/attention.h:7-16)."""
    _require_cuda("key", key)
    _require_cuda("value", value)
    _prefill(query, key, value, None, None, cu_seqlens_q, cu_seqlens_k, None, num_kv_heads, head_dim, 1,
             scale, output)


def launch_prefill_attention_paged(query, cu_seqlens_q, k_cache, v_cache, cu_seqlens_k, block_tables,
                                   num_kv_heads, head_dim, block_size, scale, output) -> None:
    """``launch_prefill_attention_paged`` (include/kernels/attention.h:18-29)."""
    if cu_seqlens_q is None or cu_seqlens_k is None:
        raise ValueError("paged prefill attention requires cu_seqlens_q and cu_seqlens_k")
    _require_cuda("k_cache", k_cache)
    _require_cuda("v_cache", v_cache)
    _require_cuda("block_tables", block_tables)
    _prefill(query, None, None, k_cache, v_cache, cu_seqlens_q, cu_seqlens_k, block_tables, num_kv_heads,
             head_dim, block_size, scale, output)


def prefill_status() -> int:
    """Reads and clears the error word of the tensor-core prefill kernels on the current device (synchronises the
    current stream): 0 = every launch since the last call completed normally."""
    out = ctypes.c_int(0)
    _check(lib().nvk_prefill_status(_stream(), ctypes.byref(out)))
    return int(out.value)


def decode_attention_static_scratch_bytes() -> int:
    return int(lib().nvk_decode_attention_static_scratch_bytes())


def attention_mixed_step(p_query, cu_seqlens_q, p_key, p_value, cu_seqlens_k, p_block_tables, p_output, d_query, context_lens,
                         d_block_tables, d_output, k_cache, v_cache, num_kv_heads, head_dim, block_size, scale, workspace,
                         prefill_blocks=0) -> None:
    """One launch for a step with prefill rows and decode rows (``nvk_attention_mixed_step``).  Dense prefill keys:
    ``p_key`` / ``p_value`` given and ``p_block_tables`` None; paged: the other way round."""
    global launch_count
    for n, t in (("p_query", p_query), ("p_output", p_output), ("d_query", d_query), ("d_output", d_output), ("k_cache", k_cache),
                 ("v_cache", v_cache), ("context_lens", context_lens), ("d_block_tables", d_block_tables), ("workspace", workspace)):
        _require_cuda(n, t)
    num_seqs = (cu_seqlens_q.numel() - 1) if cu_seqlens_q is not None else 1
    ncb = k_cache.numel() // (block_size * num_kv_heads * head_dim)
    _check(lib().nvk_attention_mixed_step(
        _ptr(p_query), _ptr(p_key), _ptr(p_value), _ptr(k_cache), _ptr(v_cache), *_index("cu_seqlens_q", cu_seqlens_q),
        *_index("cu_seqlens_k", cu_seqlens_k), *_index("p_block_tables", p_block_tables), ctypes.c_int64(num_seqs),
        ctypes.c_int64(p_query.shape[0]), ctypes.c_int64(p_key.shape[0] if p_key is not None else 0),
        ctypes.c_int64(p_block_tables.shape[1] if p_block_tables is not None else 0), ctypes.c_int(0), _ptr(p_output), _ptr(d_query),
        *_index("context_lens", context_lens), *_index("d_block_tables", d_block_tables), ctypes.c_int64(d_query.shape[0]),
        ctypes.c_int64(d_block_tables.shape[1]), _ptr(d_output), ctypes.c_int64(ncb), ctypes.c_int(p_query.shape[1]),
        ctypes.c_int(num_kv_heads), ctypes.c_int(head_dim), ctypes.c_int(block_size), ctypes.c_float(scale),
        ctypes.c_int(_dtype_code(p_query)), _ptr(workspace), ctypes.c_size_t(workspace.numel() * workspace.element_size()),
        ctypes.c_int(prefill_blocks), _stream()))
    launch_count += 2


def linear(x, weight, out) -> None:
    """``out = x @ weight.T`` on this library's tcgen05 GEMM (``nvk_linear``); weight [out_features, in_features]."""
    global launch_count
    for n, t in (("x", x), ("weight", weight), ("out", out)):
        _require_cuda(n, t)
    _check(lib().nvk_linear(_ptr(x), _ptr(weight), _ptr(out), ctypes.c_int64(x.shape[0]), ctypes.c_int64(weight.shape[0]),
                            ctypes.c_int64(weight.shape[1]), ctypes.c_int(_dtype_code(x)), _stream()))
    launch_count += 1


def qkv_linear_norm_rope_store(x, qkv_weight, positions, q_norm_weight, k_norm_weight, norm_eps, cos_sin_cache, slot_mapping,
                               k_cache, v_cache, num_q_heads, num_kv_heads, head_dim, q_out) -> None:
    """QKV projection + split + q / k RMSNorm + RoPE + cache store as one launch (``nvk_qkv_linear_norm_rope_store``)."""
    global launch_count
    for n, t in (("x", x), ("qkv_weight", qkv_weight), ("positions", positions), ("cos_sin_cache", cos_sin_cache),
                 ("k_cache", k_cache), ("v_cache", v_cache), ("q_out", q_out)):
        _require_cuda(n, t)
    row = num_kv_heads * head_dim
    _check(lib().nvk_qkv_linear_norm_rope_store(
        _ptr(x), _ptr(qkv_weight), ctypes.c_int64(x.shape[0]), ctypes.c_int64(x.shape[1]), _ptr(positions), _ptr(q_norm_weight),
        _ptr(k_norm_weight), ctypes.c_float(norm_eps), _ptr(cos_sin_cache), ctypes.c_int64(cos_sin_cache.shape[0]),
        _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), ctypes.c_int64(k_cache.numel() // row), ctypes.c_int(num_q_heads),
        ctypes.c_int(num_kv_heads), ctypes.c_int(head_dim), _ptr(q_out), ctypes.c_int(_dtype_code(x)), _stream()))
    launch_count += 1


def gemm_status() -> int:
    """Reads and clears the error word of the GEMM kernels on the current device (synchronises the current stream)."""
    out = ctypes.c_int(0)
    _check(lib().nvk_gemm_status(_stream(), ctypes.byref(out)))
    return int(out.value)
