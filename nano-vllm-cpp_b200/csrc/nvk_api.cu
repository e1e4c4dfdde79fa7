// extern "C" entry points declared in include/nvk.h: argument validation (the checks the
// reference performs in src/kernels/kvcache.cu:146-190, src/kernels/attention.cu:679-681 and
// src/kernels/kernel_types.cu:24-110) and dispatch to the kernels of this library.
#include "nvk_internal.cuh"

#include <string>

namespace nvk {

namespace {
thread_local std::string g_last_error;
}

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

int check_launch(const char* what) {
    const cudaError_t e = cudaPeekAtLastError();
    if (e == cudaSuccess) return NVK_OK;
    return fail(NVK_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

namespace {

bool is_compute_dtype(int dtype) { return dtype == NVK_F16 || dtype == NVK_BF16 || dtype == NVK_F32; }
bool is_index_dtype(int dtype) { return dtype == NVK_I32 || dtype == NVK_I64; }
IndexArray index_array(const void* p, int dtype) { return IndexArray(p, dtype == NVK_I64 ? 1 : 0); }

}  // namespace
}  // namespace nvk

using namespace nvk;

extern "C" {

int nvk_abi_version(void) { return 2; }

const char* nvk_last_error(void) { return g_last_error.c_str(); }

int nvk_store_kvcache(const void* key, const void* value, void* k_cache, void* v_cache,
                      const void* slot_mapping, int slot_dtype, int64_t num_tokens, int64_t row_elems,
                      int64_t cache_rows, int dtype, void* stream) {
    if (!key || !value || !k_cache || !v_cache || !slot_mapping)
        return fail(NVK_ERR_INVALID_ARGUMENT, "store_kvcache: key, value, k_cache, v_cache and slot_mapping must be defined");
    if (!is_compute_dtype(dtype)) return fail(NVK_ERR_INVALID_ARGUMENT, "key must be float16, bfloat16, or float32");
    if (slot_dtype != NVK_I32 && slot_dtype != NVK_I64)
        return fail(NVK_ERR_INVALID_ARGUMENT, "slot_mapping must be int32 or int64");
    if (num_tokens <= 0) return fail(NVK_ERR_INVALID_ARGUMENT, "slot_mapping must contain at least one element");
    if (row_elems <= 0) return fail(NVK_ERR_INVALID_ARGUMENT, "key cannot be flattened by the provided leading count");
    if (cache_rows <= 0) return fail(NVK_ERR_INVALID_ARGUMENT, "k_cache does not contain an integer number of cache rows");
    return launch_store_kvcache(key, value, k_cache, v_cache, slot_mapping, slot_dtype == NVK_I64, num_tokens,
                                row_elems * static_cast<int64_t>(dtype_size(dtype)), cache_rows,
                                static_cast<cudaStream_t>(stream));
}

int nvk_fused_split_norm_rope_store(const void* qkv, const int32_t* positions, const void* q_norm_weight,
                                    const void* k_norm_weight, float norm_eps, const float* cos_sin_cache,
                                    int64_t max_positions, const int32_t* slot_mapping, void* k_cache,
                                    void* v_cache, int64_t cache_rows, int64_t rows, int num_q_heads,
                                    int num_kv_heads, int head_dim, void* q_out, int dtype, void* stream) {
    if (dtype != NVK_F16 && dtype != NVK_BF16)
        return fail(NVK_ERR_INVALID_ARGUMENT, "fused_split_norm_rope_store only supports bf16/fp16");
    if (!qkv || !positions || !cos_sin_cache || !k_cache || !v_cache || !q_out)
        return fail(NVK_ERR_INVALID_ARGUMENT, "fused_split_norm_rope_store: all tensors must be defined");
    if ((q_norm_weight == nullptr) != (k_norm_weight == nullptr))
        return fail(NVK_ERR_INVALID_ARGUMENT, "fused_split_norm_rope_store: q_norm_weight and k_norm_weight go together");
    if (rows < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || max_positions <= 0 || cache_rows <= 0)
        return fail(NVK_ERR_INVALID_ARGUMENT, "fused_split_norm_rope_store: sizes must be positive");
    if (rows == 0) return NVK_OK;
    if (!aligned_to(qkv, 16) || !aligned_to(q_out, 16) || !aligned_to(k_cache, 16) || !aligned_to(v_cache, 16) ||
        !aligned_to(q_norm_weight, 16) || !aligned_to(k_norm_weight, 16) || !aligned_to(cos_sin_cache, 16))
        return fail(NVK_ERR_UNSUPPORTED, "fused_split_norm_rope_store: tensors must be 16-byte aligned");
    return launch_fused_prologue(qkv, positions, q_norm_weight, k_norm_weight, norm_eps, cos_sin_cache,
                                 max_positions, slot_mapping, k_cache, v_cache, cache_rows, rows, num_q_heads,
                                 num_kv_heads, head_dim, q_out, dtype, static_cast<cudaStream_t>(stream));
}

size_t nvk_decode_attention_workspace_bytes(int64_t batch, int num_heads, int num_kv_heads, int head_dim,
                                            int64_t max_blocks, int block_size) {
    return decode_mma_workspace_bytes(batch, num_heads, num_kv_heads, head_dim, max_blocks, block_size);
}

int nvk_decode_attention_paged(const void* query, const void* k_cache, const void* v_cache,
                               const void* context_lens, int context_lens_dtype, const void* block_tables,
                               int block_tables_dtype, int64_t batch, int64_t max_blocks, int64_t num_cache_blocks,
                               int num_heads, int num_kv_heads, int head_dim, int block_size, float scale,
                               void* output, int dtype, void* workspace, size_t workspace_bytes, void* stream) {
    if (!query || !k_cache || !v_cache || !context_lens || !block_tables || !output)
        return fail(NVK_ERR_INVALID_ARGUMENT, "decode attention requires KV cache, context_lens, and block_tables");
    if (!is_index_dtype(context_lens_dtype) || !is_index_dtype(block_tables_dtype))
        return fail(NVK_ERR_INVALID_ARGUMENT, "context_lens and block_tables must be int32 or int64");
    if (!is_compute_dtype(dtype)) return fail(NVK_ERR_INVALID_ARGUMENT, "unsupported dtype for decode_attention_paged");
    if (batch < 0 || max_blocks <= 0 || num_cache_blocks <= 0 || num_heads <= 0 || num_kv_heads <= 0 ||
        head_dim <= 0 || block_size <= 0)
        return fail(NVK_ERR_INVALID_ARGUMENT, "attention dimensions must be positive");
    if (num_heads % num_kv_heads != 0)
        return fail(NVK_ERR_INVALID_ARGUMENT, "num_heads must be divisible by num_kv_heads");
    if (batch == 0) return NVK_OK;
    DecodeArgs a{query, k_cache, v_cache, index_array(context_lens, context_lens_dtype),
                 index_array(block_tables, block_tables_dtype), output, batch, max_blocks, num_cache_blocks,
                 num_heads, num_kv_heads, head_dim, block_size, scale, dtype, workspace, workspace_bytes,
                 static_cast<cudaStream_t>(stream)};
    if (decode_mma_supported(a)) {
        if (workspace != nullptr) {
            const size_t need = decode_mma_workspace_bytes(batch, num_heads, num_kv_heads, head_dim, max_blocks, block_size);
            if (workspace_bytes < need)
                return fail(NVK_ERR_INVALID_ARGUMENT, "decode attention: workspace of %zu bytes given, %zu needed",
                            workspace_bytes, need);
            if (!aligned_to(workspace, 16))
                return fail(NVK_ERR_INVALID_ARGUMENT, "decode attention: workspace must be 16-byte aligned");
        }
        return launch_decode_mma(a);
    }
    return launch_rowwise_decode(a);
}

int nvk_store_kvcache_int8(const void* key, const void* value, void* k_cache, void* v_cache, void* k_scale,
                           void* v_scale, const int32_t* slot_mapping, int64_t num_tokens, int num_kv_heads,
                           int head_dim, int64_t cache_rows, int dtype, void* stream) {
    if (!key || !value || !k_cache || !v_cache || !k_scale || !v_scale || !slot_mapping)
        return fail(NVK_ERR_INVALID_ARGUMENT, "store_kvcache_int8: every tensor must be defined");
    if (!is_compute_dtype(dtype)) return fail(NVK_ERR_INVALID_ARGUMENT, "unsupported input dtype for store_kvcache_int8");
    if (num_kv_heads <= 0 || head_dim <= 0 || cache_rows <= 0)
        return fail(NVK_ERR_INVALID_ARGUMENT, "store_kvcache_int8: dimensions must be positive");
    if (num_tokens <= 0) return NVK_OK;   // the reference returns without a launch (kvcache.cu:327)
    if (!aligned_to(key, dtype == NVK_F32 ? 4 : 16) || !aligned_to(value, dtype == NVK_F32 ? 4 : 16) ||
        !aligned_to(k_cache, 8) || !aligned_to(v_cache, 8) || !aligned_to(k_scale, 2) || !aligned_to(v_scale, 2))
        return fail(NVK_ERR_INVALID_ARGUMENT, "store_kvcache_int8: misaligned tensor");
    return launch_store_int8(key, value, k_cache, v_cache, k_scale, v_scale, slot_mapping, num_tokens, num_kv_heads,
                             head_dim, cache_rows, dtype, static_cast<cudaStream_t>(stream));
}

int nvk_decode_attention_paged_int8(const void* query, const void* k_cache, const void* v_cache, const void* k_scale,
                                    const void* v_scale, const void* context_lens, int context_lens_dtype,
                                    const void* block_tables, int block_tables_dtype, int64_t batch, int64_t max_blocks,
                                    int64_t num_cache_blocks, int num_heads, int num_kv_heads, int head_dim,
                                    int block_size, float scale, void* output, int dtype, void* workspace,
                                    size_t workspace_bytes, void* stream) {
    if (!query || !k_cache || !v_cache || !k_scale || !v_scale || !context_lens || !block_tables || !output)
        return fail(NVK_ERR_INVALID_ARGUMENT, "decode attention (int8) requires KV cache, scales, context_lens, and block_tables");
    if (!is_index_dtype(context_lens_dtype) || !is_index_dtype(block_tables_dtype))
        return fail(NVK_ERR_INVALID_ARGUMENT, "context_lens and block_tables must be int32 or int64");
    if (!is_compute_dtype(dtype)) return fail(NVK_ERR_INVALID_ARGUMENT, "unsupported query dtype for decode_attention_paged_int8");
    if (batch < 0 || max_blocks <= 0 || num_cache_blocks <= 0 || num_heads <= 0 || num_kv_heads <= 0 ||
        head_dim <= 0 || block_size <= 0)
        return fail(NVK_ERR_INVALID_ARGUMENT, "attention dimensions must be positive");
    if (num_heads % num_kv_heads != 0)
        return fail(NVK_ERR_INVALID_ARGUMENT, "num_heads must be divisible by num_kv_heads");
    if (batch == 0) return NVK_OK;
    DecodeInt8Args a{{query, k_cache, v_cache, index_array(context_lens, context_lens_dtype),
                      index_array(block_tables, block_tables_dtype), output, batch, max_blocks, num_cache_blocks,
                      num_heads, num_kv_heads, head_dim, block_size, scale, dtype, workspace, workspace_bytes,
                      static_cast<cudaStream_t>(stream)},
                     k_scale, v_scale};
    if (decode_int8_mma_supported(a)) {
        if (workspace != nullptr) {
            const size_t need = decode_mma_workspace_bytes(batch, num_heads, num_kv_heads, head_dim, max_blocks, block_size);
            if (workspace_bytes < need)
                return fail(NVK_ERR_INVALID_ARGUMENT, "decode attention (int8): workspace of %zu bytes given, %zu needed",
                            workspace_bytes, need);
            if (!aligned_to(workspace, 16))
                return fail(NVK_ERR_INVALID_ARGUMENT, "decode attention (int8): workspace must be 16-byte aligned");
        }
        return launch_decode_int8_mma(a);
    }
    return launch_rowwise_decode_int8(a);
}

int nvk_store_kvcache_fp8(const void* key, const void* value, void* k_cache, void* v_cache, void* k_scale, void* v_scale,
                          const int32_t* slot_mapping, int64_t num_tokens, int num_kv_heads, int head_dim, int64_t cache_rows,
                          int dtype, void* stream) {
    if (!key || !value || !k_cache || !v_cache || !k_scale || !v_scale || !slot_mapping)
        return fail(NVK_ERR_INVALID_ARGUMENT, "store_kvcache_fp8 requires key, value, caches, scales and slot_mapping");
    if (dtype != NVK_F16 && dtype != NVK_BF16) return fail(NVK_ERR_UNSUPPORTED, "store_kvcache_fp8: key / value must be F16 or BF16");
    if (num_tokens < 0 || num_kv_heads <= 0 || head_dim <= 0 || cache_rows <= 0)
        return fail(NVK_ERR_INVALID_ARGUMENT, "store_kvcache_fp8: sizes must be positive");
    if (!aligned_to(key, 16) || !aligned_to(value, 16) || !aligned_to(k_cache, 8) || !aligned_to(v_cache, 8))
        return fail(NVK_ERR_INVALID_ARGUMENT, "store_kvcache_fp8: key / value must be 16-byte aligned, the caches 8-byte aligned");
    if (num_tokens == 0) return NVK_OK;
    return launch_store_fp8(key, value, k_cache, v_cache, k_scale, v_scale, slot_mapping, num_tokens, num_kv_heads, head_dim,
                            cache_rows, dtype, static_cast<cudaStream_t>(stream));
}

int nvk_decode_attention_paged_fp8(const void* query, const void* k_cache, const void* v_cache, const void* k_scale,
                                   const void* v_scale, const void* context_lens, int context_lens_dtype,
                                   const void* block_tables, int block_tables_dtype, int64_t batch, int64_t max_blocks,
                                   int64_t num_cache_blocks, int num_heads, int num_kv_heads, int head_dim,
                                   int block_size, float scale, void* output, int dtype, void* workspace,
                                   size_t workspace_bytes, void* stream) {
    if (!query || !k_cache || !v_cache || !k_scale || !v_scale || !context_lens || !block_tables || !output)
        return fail(NVK_ERR_INVALID_ARGUMENT, "decode attention (fp8) requires KV cache, scales, context_lens, and block_tables");
    if (!is_index_dtype(context_lens_dtype) || !is_index_dtype(block_tables_dtype))
        return fail(NVK_ERR_INVALID_ARGUMENT, "context_lens and block_tables must be int32 or int64");
    if (batch < 0 || max_blocks <= 0 || num_cache_blocks <= 0 || num_heads <= 0 || num_kv_heads <= 0 ||
        head_dim <= 0 || block_size <= 0)
        return fail(NVK_ERR_INVALID_ARGUMENT, "attention dimensions must be positive");
    if (num_heads % num_kv_heads != 0)
        return fail(NVK_ERR_INVALID_ARGUMENT, "num_heads must be divisible by num_kv_heads");
    if (batch == 0) return NVK_OK;
    DecodeInt8Args a{{query, k_cache, v_cache, index_array(context_lens, context_lens_dtype),
                      index_array(block_tables, block_tables_dtype), output, batch, max_blocks, num_cache_blocks,
                      num_heads, num_kv_heads, head_dim, block_size, scale, dtype, workspace, workspace_bytes,
                      static_cast<cudaStream_t>(stream)},
                     k_scale, v_scale, true};
    if (!decode_int8_mma_supported(a))
        return fail(NVK_ERR_UNSUPPORTED, "decode attention (fp8): F16 / BF16 queries, head_dim 128, at most 8 query heads per KV head, "
                                         "block_size a multiple of 16 (and a workspace beyond 8 cache blocks per sequence)");
    if (workspace != nullptr) {
        const size_t need = decode_mma_workspace_bytes(batch, num_heads, num_kv_heads, head_dim, max_blocks, block_size);
        if (workspace_bytes < need)
            return fail(NVK_ERR_INVALID_ARGUMENT, "decode attention (fp8): workspace of %zu bytes given, %zu needed", workspace_bytes, need);
        if (!aligned_to(workspace, 16)) return fail(NVK_ERR_INVALID_ARGUMENT, "decode attention (fp8): workspace must be 16-byte aligned");
    }
    return launch_decode_int8_mma(a);
}

int nvk_prefill_attention_varlen(const void* query, const void* key, const void* value, const void* k_cache,
                                 const void* v_cache, const void* cu_seqlens_q, int cu_seqlens_q_dtype,
                                 const void* cu_seqlens_k, int cu_seqlens_k_dtype, const void* block_tables,
                                 int block_tables_dtype, int64_t num_seqs, int64_t total_q, int64_t total_k,
                                 int64_t max_blocks, int64_t num_cache_blocks, int max_seqlen_q, int num_heads,
                                 int num_kv_heads, int head_dim, int block_size, float scale, void* output,
                                 int dtype, void* stream) {
    if (!query || !output) return fail(NVK_ERR_INVALID_ARGUMENT, "prefill attention: query and output must be defined");
    if (!is_compute_dtype(dtype)) return fail(NVK_ERR_INVALID_ARGUMENT, "unsupported dtype for prefill attention");
    if (num_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || total_q < 0)
        return fail(NVK_ERR_INVALID_ARGUMENT, "attention dimensions must be positive");
    if (num_heads % num_kv_heads != 0)
        return fail(NVK_ERR_INVALID_ARGUMENT, "num_heads must be divisible by num_kv_heads");
    if ((cu_seqlens_q && !is_index_dtype(cu_seqlens_q_dtype)) || (cu_seqlens_k && !is_index_dtype(cu_seqlens_k_dtype)) ||
        (block_tables && !is_index_dtype(block_tables_dtype)))
        return fail(NVK_ERR_INVALID_ARGUMENT, "cu_seqlens and block_tables must be int32 or int64");
    const bool paged = block_tables != nullptr;
    if (paged) {
        if (!cu_seqlens_q || !cu_seqlens_k)
            return fail(NVK_ERR_INVALID_ARGUMENT, "paged prefill attention requires cu_seqlens_q and cu_seqlens_k");
        if (!k_cache || !v_cache) return fail(NVK_ERR_INVALID_ARGUMENT, "paged prefill attention requires k_cache and v_cache");
        if (max_blocks <= 0 || num_cache_blocks <= 0 || block_size <= 0)
            return fail(NVK_ERR_INVALID_ARGUMENT, "paged prefill attention: block sizes must be positive");
    } else {
        if (!key || !value) return fail(NVK_ERR_INVALID_ARGUMENT, "prefill attention: key and value must be defined");
        if (total_k < 0) return fail(NVK_ERR_INVALID_ARGUMENT, "prefill attention: total_k must be non-negative");
        if ((cu_seqlens_q == nullptr) != (cu_seqlens_k == nullptr)) { cu_seqlens_q = nullptr; cu_seqlens_k = nullptr; }
    }
    if (cu_seqlens_q && num_seqs <= 0) return fail(NVK_ERR_INVALID_ARGUMENT, "prefill attention: num_seqs must be positive");
    if (total_q == 0) return NVK_OK;
    PrefillArgs a{query, key, value, k_cache, v_cache, index_array(cu_seqlens_q, cu_seqlens_q_dtype),
                  index_array(cu_seqlens_k, cu_seqlens_k_dtype), index_array(block_tables, block_tables_dtype), output, num_seqs,
                  total_q, total_k, max_blocks, num_cache_blocks, max_seqlen_q, num_heads, num_kv_heads, head_dim,
                  block_size, scale, dtype, static_cast<cudaStream_t>(stream)};
    if (prefill_tc_supported(a)) return launch_prefill_tc(a);
    if (prefill_mma_supported(a)) return launch_prefill_mma(a);
    return launch_rowwise_prefill(a);
}

int nvk_attention_mixed_step(const void* p_query, const void* p_key, const void* p_value, const void* k_cache, const void* v_cache,
                             const void* cu_seqlens_q, int cu_seqlens_q_dtype, const void* cu_seqlens_k, int cu_seqlens_k_dtype,
                             const void* p_block_tables, int p_block_tables_dtype, int64_t num_seqs, int64_t total_q,
                             int64_t total_k, int64_t p_max_blocks, int max_seqlen_q, void* p_output, const void* d_query,
                             const void* context_lens, int context_lens_dtype, const void* d_block_tables,
                             int d_block_tables_dtype, int64_t batch, int64_t d_max_blocks, void* d_output,
                             int64_t num_cache_blocks, int num_heads, int num_kv_heads, int head_dim, int block_size, float scale,
                             int dtype, void* workspace, size_t workspace_bytes, int prefill_blocks, void* stream) {
    if (!p_query || !p_output || !d_query || !d_output || !k_cache || !v_cache || !context_lens || !d_block_tables)
        return fail(NVK_ERR_INVALID_ARGUMENT, "mixed step: queries, outputs, the KV cache, context_lens and the decode block tables must be defined");
    if (!is_index_dtype(context_lens_dtype) || !is_index_dtype(d_block_tables_dtype) || (cu_seqlens_q && !is_index_dtype(cu_seqlens_q_dtype)) ||
        (cu_seqlens_k && !is_index_dtype(cu_seqlens_k_dtype)) || (p_block_tables && !is_index_dtype(p_block_tables_dtype)))
        return fail(NVK_ERR_INVALID_ARGUMENT, "mixed step: index tensors must be int32 or int64");
    if (num_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || block_size <= 0 || num_cache_blocks <= 0 || total_q <= 0 || batch <= 0 ||
        d_max_blocks <= 0)
        return fail(NVK_ERR_INVALID_ARGUMENT, "mixed step: sizes must be positive (a step without prefill rows or without decode rows takes the single-purpose entry point)");
    if (num_heads % num_kv_heads != 0) return fail(NVK_ERR_INVALID_ARGUMENT, "num_heads must be divisible by num_kv_heads");
    const bool paged = p_block_tables != nullptr;
    if (paged && (!cu_seqlens_q || !cu_seqlens_k || p_max_blocks <= 0))
        return fail(NVK_ERR_INVALID_ARGUMENT, "paged prefill attention requires cu_seqlens_q and cu_seqlens_k");
    if (!paged && (!p_key || !p_value)) return fail(NVK_ERR_INVALID_ARGUMENT, "prefill attention: key and value must be defined");
    if ((cu_seqlens_q == nullptr) != (cu_seqlens_k == nullptr)) { cu_seqlens_q = nullptr; cu_seqlens_k = nullptr; }
    if (cu_seqlens_q && num_seqs <= 0) return fail(NVK_ERR_INVALID_ARGUMENT, "prefill attention: num_seqs must be positive");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    PrefillArgs pa{p_query, p_key, p_value, k_cache, v_cache, index_array(cu_seqlens_q, cu_seqlens_q_dtype),
                   index_array(cu_seqlens_k, cu_seqlens_k_dtype), index_array(p_block_tables, p_block_tables_dtype), p_output, num_seqs,
                   total_q, total_k, p_max_blocks, num_cache_blocks, max_seqlen_q, num_heads, num_kv_heads, head_dim, block_size, scale,
                   dtype, st};
    DecodeArgs da{d_query, k_cache, v_cache, index_array(context_lens, context_lens_dtype), index_array(d_block_tables, d_block_tables_dtype),
                  d_output, batch, d_max_blocks, num_cache_blocks, num_heads, num_kv_heads, head_dim, block_size, scale, dtype, workspace,
                  workspace_bytes, st};
    const size_t need = decode_mma_workspace_bytes(batch, num_heads, num_kv_heads, head_dim, d_max_blocks, block_size);
    if (workspace == nullptr || workspace_bytes < need || !aligned_to(workspace, 16))
        return fail(NVK_ERR_INVALID_ARGUMENT, "mixed step: a 16-byte aligned workspace of %zu bytes is needed (nvk_decode_attention_workspace_bytes)", need);
    if (!mixed_step_supported(pa, da))
        return fail(NVK_ERR_UNSUPPORTED, "mixed step: needs F16 / BF16, head_dim 128, an even number of query heads per KV head, at most 8, and "
                                         "paged block sizes that are multiples of 128; call the prefill and decode entry points instead");
    return launch_mixed_step(pa, da, prefill_blocks);
}

}  // extern "C"
