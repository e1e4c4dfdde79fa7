// Operator wrappers: the reference's C++ kernel API (include/kernels/*.h of nano-vllm-cpp) implemented
// as argument checks + one call into the C ABI of libnvk.so (include/nvk.h).  Error behaviour follows
// the reference: std::invalid_argument for bad operands (src/kernels/kvcache.cu:146-190,
// src/kernels/kernel_types.cu:24-110), std::runtime_error for CUDA failures.
#include "kernels/attention.h"
#include "kernels/flash_attn.h"
#include "kernels/kernel_types.h"
#include "kernels/kvcache.h"
#include "kernels/split_qkv.h"

#include "nvk.h"

#include <stdexcept>
#include <string>

namespace nano_vllm {

// ---- checks -----------------------------------------------------------------------------------------
void ensure_cuda_tensor(const char* name, const Tensor& tensor) {
    if (!tensor.defined()) throw std::invalid_argument(std::string(name) + " must be defined");
    if (tensor.device().type != DeviceType::kCUDA) throw std::invalid_argument(std::string(name) + " must live on CUDA");
    if (!tensor.is_contiguous()) throw std::invalid_argument(std::string(name) + " must be contiguous");
}

void ensure_same_device(const char* lhs_name, const Tensor& lhs, const char* rhs_name, const Tensor& rhs) {
    if (lhs.device() != rhs.device())
        throw std::invalid_argument(std::string(lhs_name) + " and " + rhs_name + " must be on the same device");
}

void ensure_same_shape(const char* lhs_name, const Tensor& lhs, const char* rhs_name, const Tensor& rhs) {
    if (lhs.sizes() != rhs.sizes())
        throw std::invalid_argument(std::string(lhs_name) + " and " + rhs_name + " must have the same shape");
}

void ensure_same_dtype(const char* lhs_name, const Tensor& lhs, const char* rhs_name, const Tensor& rhs) {
    if (lhs.dtype() != rhs.dtype())
        throw std::invalid_argument(std::string(lhs_name) + " and " + rhs_name + " must have the same dtype");
}

void validate_supported_dtype(const char* name, ScalarType dtype) {
    if (dtype != ScalarType::kFloat16 && dtype != ScalarType::kBFloat16 && dtype != ScalarType::kFloat32)
        throw std::invalid_argument(std::string(name) + " must be float16, bfloat16, or float32");
}

MatrixShape flatten_by_leading_count(const char* name, const Tensor& tensor, int64_t leading_count) {
    if (leading_count <= 0) throw std::invalid_argument(std::string(name) + " must have a positive leading count");
    const int64_t total = static_cast<int64_t>(tensor.numel());
    const int64_t cols = total / leading_count;
    if (cols <= 0 || cols * leading_count != total)
        throw std::invalid_argument(std::string(name) + " cannot be flattened by the provided leading count");
    return {leading_count, cols};
}

int64_t cache_rows_from_tensor(const char* name, const Tensor& tensor, int64_t row_width) {
    if (row_width <= 0) throw std::invalid_argument(std::string(name) + " row width must be positive");
    const int64_t total = static_cast<int64_t>(tensor.numel());
    const int64_t rows = total / row_width;
    if (rows <= 0 || rows * row_width != total)
        throw std::invalid_argument(std::string(name) + " does not contain an integer number of cache rows");
    return rows;
}

void throw_on_nvk_status(int status) {
    if (status == NVK_OK) return;
    if (status == NVK_ERR_CUDA) throw std::runtime_error(nvk_last_error());
    throw std::invalid_argument(nvk_last_error());
}

namespace {

int code(ScalarType t) { return static_cast<int>(t); }

const int32_t* int32_data(const char* name, const Tensor& t) {
    ensure_cuda_tensor(name, t);
    if (t.dtype() != ScalarType::kInt32) throw std::invalid_argument(std::string(name) + " must be int32");
    return t.data_as<int32_t>();
}

// An index tensor of either width (the reference's attention kernels take int32 or int64 for each of cu_seqlens_q,
// cu_seqlens_k, context_lens and block_tables on its own, src/kernels/attention.cu:644-660, :708-735).
struct IndexRef { const void* ptr; int dtype; };
IndexRef index_data(const char* name, const Tensor& t) {
    ensure_cuda_tensor(name, t);
    if (t.dtype() != ScalarType::kInt32 && t.dtype() != ScalarType::kInt64)
        throw std::invalid_argument(std::string(name) + " must be int32 or int64");
    return {t.data(), code(t.dtype())};
}

int64_t cache_blocks(const Tensor& cache, int block_size, int num_kv_heads, int head_dim) {
    const int64_t per_block = static_cast<int64_t>(block_size) * num_kv_heads * head_dim;
    if (per_block <= 0) throw std::invalid_argument("attention dimensions must be positive");
    return static_cast<int64_t>(cache.numel()) / per_block;
}

void check_qo(const Tensor& query, const Tensor& output) {
    ensure_cuda_tensor("query", query);
    ensure_cuda_tensor("output", output);
    ensure_same_device("query", query, "output", output);
    ensure_same_dtype("query", query, "output", output);
    ensure_same_shape("query", query, "output", output);
    if (query.dim() != 3) throw std::invalid_argument("attention expects [tokens, heads, head_dim] tensors");
}

}  // namespace

// ---- store_kvcache ----------------------------------------------------------------------------------
void store_kvcache(const Tensor& key, const Tensor& value, Tensor& k_cache, Tensor& v_cache, const Tensor& slot_mapping,
                   cudaStream_t stream) {
    ensure_cuda_tensor("key", key);
    ensure_cuda_tensor("value", value);
    ensure_cuda_tensor("k_cache", k_cache);
    ensure_cuda_tensor("v_cache", v_cache);
    ensure_cuda_tensor("slot_mapping", slot_mapping);
    ensure_same_device("key", key, "value", value);
    ensure_same_device("key", key, "k_cache", k_cache);
    ensure_same_device("key", key, "v_cache", v_cache);
    ensure_same_device("key", key, "slot_mapping", slot_mapping);
    ensure_same_dtype("key", key, "value", value);
    ensure_same_dtype("key", key, "k_cache", k_cache);
    ensure_same_dtype("key", key, "v_cache", v_cache);
    validate_supported_dtype("key", key.dtype());
    if (slot_mapping.dtype() != ScalarType::kInt32 && slot_mapping.dtype() != ScalarType::kInt64)
        throw std::invalid_argument("slot_mapping must be int32 or int64");
    const int64_t tokens = static_cast<int64_t>(slot_mapping.numel());
    if (tokens <= 0) throw std::invalid_argument("slot_mapping must contain at least one element");
    const MatrixShape k = flatten_by_leading_count("key", key, tokens);
    const MatrixShape v = flatten_by_leading_count("value", value, tokens);
    if (k.cols != v.cols) throw std::invalid_argument("key and value must have the same flattened row width");
    const int64_t k_rows = cache_rows_from_tensor("k_cache", k_cache, k.cols);
    const int64_t v_rows = cache_rows_from_tensor("v_cache", v_cache, k.cols);
    if (k_rows != v_rows) throw std::invalid_argument("k_cache and v_cache must contain the same number of slots");
    throw_on_nvk_status(nvk_store_kvcache(key.data(), value.data(), k_cache.data(), v_cache.data(), slot_mapping.data(),
                                          code(slot_mapping.dtype()), tokens, k.cols, k_rows, code(key.dtype()), stream));
}

void store_kvcache_int8(const Tensor& key, const Tensor& value, Tensor& k_cache, Tensor& v_cache, Tensor& k_scale,
                        Tensor& v_scale, const Tensor& slot_mapping, cudaStream_t stream) {
    ensure_cuda_tensor("key", key);
    ensure_cuda_tensor("value", value);
    ensure_cuda_tensor("k_cache", k_cache);
    ensure_cuda_tensor("v_cache", v_cache);
    ensure_cuda_tensor("k_scale", k_scale);
    ensure_cuda_tensor("v_scale", v_scale);
    ensure_cuda_tensor("slot_mapping", slot_mapping);
    validate_supported_dtype("key", key.dtype());
    ensure_same_dtype("key", key, "value", value);
    if (k_cache.dtype() != ScalarType::kInt8 || v_cache.dtype() != ScalarType::kInt8)
        throw std::invalid_argument("store_kvcache_int8 requires int8 caches");
    if (k_scale.dtype() != ScalarType::kFloat16 || v_scale.dtype() != ScalarType::kFloat16)
        throw std::invalid_argument("store_kvcache_int8 requires float16 scales");
    if (slot_mapping.dtype() != ScalarType::kInt32) throw std::invalid_argument("slot_mapping must be int32 for the int8 store");
    const int64_t tokens = static_cast<int64_t>(slot_mapping.numel());
    if (tokens <= 0) return;   // the reference returns without a launch
    if (key.dim() != 3) throw std::invalid_argument("key must be rank-3 for int8 store");
    ensure_same_shape("key", key, "value", value);
    if (key.sizes()[0] != tokens) throw std::invalid_argument("key rows must match slot_mapping");
    const int heads = static_cast<int>(key.sizes()[1]);
    const int head_dim = static_cast<int>(key.sizes()[2]);
    const int64_t row = static_cast<int64_t>(heads) * head_dim;
    const int64_t rows = cache_rows_from_tensor("k_cache", k_cache, row);
    if (cache_rows_from_tensor("v_cache", v_cache, row) != rows)
        throw std::invalid_argument("k_cache and v_cache must contain the same number of slots");
    if (static_cast<int64_t>(k_scale.numel()) != rows * heads || static_cast<int64_t>(v_scale.numel()) != rows * heads)
        throw std::invalid_argument("k_scale and v_scale must hold one value per cache row and KV head");
    throw_on_nvk_status(nvk_store_kvcache_int8(key.data(), value.data(), k_cache.data(), v_cache.data(), k_scale.data(),
                                               v_scale.data(), static_cast<const int32_t*>(slot_mapping.data()), tokens, heads,
                                               head_dim, rows, code(key.dtype()), stream));
}

// ---- fused decode prologue ---------------------------------------------------------------------------
void fused_split_norm_rope_store(const Tensor& qkv, const Tensor& positions, const Tensor& q_norm_weight,
                                 const Tensor& k_norm_weight, float norm_eps, const Tensor& cos_sin_cache,
                                 const Tensor& slot_mapping, Tensor& k_cache, Tensor& v_cache, int num_q_heads,
                                 int num_kv_heads, int head_dim, Tensor& q_out, cudaStream_t stream) {
    if (qkv.defined() && qkv.dtype() != ScalarType::kBFloat16 && qkv.dtype() != ScalarType::kFloat16)
        throw std::invalid_argument("fused_split_norm_rope_store only supports bf16/fp16");
    ensure_cuda_tensor("qkv", qkv);
    ensure_cuda_tensor("q_norm_weight", q_norm_weight);
    ensure_cuda_tensor("k_norm_weight", k_norm_weight);
    ensure_cuda_tensor("cos_sin_cache", cos_sin_cache);
    ensure_cuda_tensor("k_cache", k_cache);
    ensure_cuda_tensor("v_cache", v_cache);
    ensure_cuda_tensor("q_out", q_out);
    if (cos_sin_cache.dtype() != ScalarType::kFloat32 || cos_sin_cache.dim() != 2)
        throw std::invalid_argument("cos_sin_cache must be a [max_positions, head_dim] float32 tensor");
    const int64_t row_width = static_cast<int64_t>(num_kv_heads) * head_dim;
    throw_on_nvk_status(nvk_fused_split_norm_rope_store(
        qkv.data(), int32_data("positions", positions), q_norm_weight.data(), k_norm_weight.data(), norm_eps,
        cos_sin_cache.data_as<float>(), cos_sin_cache.sizes()[0], int32_data("slot_mapping", slot_mapping),
        k_cache.data(), v_cache.data(), cache_rows_from_tensor("k_cache", k_cache, row_width), qkv.sizes()[0],
        num_q_heads, num_kv_heads, head_dim, q_out.data(), code(qkv.dtype()), stream));
}

// ---- decode -------------------------------------------------------------------------------------------
namespace {

void decode_common(const Tensor& query, const Tensor& k_cache, const Tensor& v_cache, const Tensor& context_lens,
                   const Tensor& block_tables, int num_kv_heads, int head_dim, int block_size, float scale,
                   Tensor& output, DeviceAllocator* allocator, cudaStream_t stream) {
    check_qo(query, output);
    ensure_cuda_tensor("k_cache", k_cache);
    ensure_cuda_tensor("v_cache", v_cache);
    ensure_same_dtype("query", query, "k_cache", k_cache);
    ensure_same_dtype("query", query, "v_cache", v_cache);
    const IndexRef lens = index_data("context_lens", context_lens);
    const IndexRef tables = index_data("block_tables", block_tables);
    if (block_tables.dim() != 2) throw std::invalid_argument("block_tables must be [batch, max_blocks]");
    const int64_t batch = query.sizes()[0];
    const int heads = static_cast<int>(query.sizes()[1]);
    const int64_t max_blocks = block_tables.sizes()[1];
    const int64_t blocks = cache_blocks(k_cache, block_size, num_kv_heads, head_dim);
    if (allocator != nullptr) {
        const size_t need = nvk_decode_attention_workspace_bytes(batch, heads, num_kv_heads, head_dim, max_blocks, block_size);
        Memory::Ptr scratch = need > 0 ? allocator->allocate(need, query.device()) : nullptr;
        throw_on_nvk_status(nvk_decode_attention_paged(query.data(), k_cache.data(), v_cache.data(), lens.ptr, lens.dtype,
                                                       tables.ptr, tables.dtype, batch, max_blocks, blocks, heads,
                                                       num_kv_heads, head_dim, block_size, scale, output.data(),
                                                       code(query.dtype()), scratch ? scratch->data() : nullptr, need, stream));
        return;   // the scratch block returns to the allocator's cache; stream order keeps it valid for this launch
    }
    const size_t need = nvk_decode_attention_workspace_bytes(batch, heads, num_kv_heads, head_dim, max_blocks, block_size);
    if (need > 0 && need <= nvk_decode_attention_static_scratch_bytes()) {
        throw_on_nvk_status(nvk_decode_attention_paged_static(query.data(), k_cache.data(), v_cache.data(), lens.ptr,
                                                              lens.dtype, tables.ptr, tables.dtype, batch, max_blocks,
                                                              blocks, heads, num_kv_heads, head_dim, block_size, scale,
                                                              output.data(), code(query.dtype()), stream));
        return;
    }
    throw_on_nvk_status(nvk_decode_attention_paged(query.data(), k_cache.data(), v_cache.data(), lens.ptr, lens.dtype,
                                                   tables.ptr, tables.dtype, batch, max_blocks, blocks, heads, num_kv_heads,
                                                   head_dim, block_size, scale, output.data(), code(query.dtype()), nullptr,
                                                   0, stream));
}

}  // namespace

void launch_decode_attention_paged(const Tensor& query, const Tensor& k_cache, const Tensor& v_cache,
                                   const Tensor& context_lens, const Tensor& block_tables, int num_kv_heads, int head_dim,
                                   int block_size, float scale, Tensor& output, cudaStream_t stream) {
    decode_common(query, k_cache, v_cache, context_lens, block_tables, num_kv_heads, head_dim, block_size, scale, output,
                  nullptr, stream);
}

void flash_attn_decode_kvcache(const Tensor& query, const Tensor& k_cache, const Tensor& v_cache,
                               const Tensor& context_lens, const Tensor& block_tables, int num_kv_heads, int head_dim,
                               int block_size, float scale, Tensor& output, DeviceAllocator& allocator,
                               cudaStream_t stream) {
    decode_common(query, k_cache, v_cache, context_lens, block_tables, num_kv_heads, head_dim, block_size, scale, output,
                  &allocator, stream);
}

void launch_decode_attention_paged_int8(const Tensor& query, const Tensor& k_cache, const Tensor& v_cache,
                                        const Tensor& k_scale, const Tensor& v_scale, const Tensor& context_lens,
                                        const Tensor& block_tables, int num_kv_heads, int head_dim, int block_size,
                                        float scale, Tensor& output, cudaStream_t stream) {
    check_qo(query, output);
    validate_supported_dtype("query", query.dtype());
    ensure_cuda_tensor("k_cache", k_cache);
    ensure_cuda_tensor("v_cache", v_cache);
    ensure_cuda_tensor("k_scale", k_scale);
    ensure_cuda_tensor("v_scale", v_scale);
    ensure_cuda_tensor("context_lens", context_lens);
    ensure_cuda_tensor("block_tables", block_tables);
    if (k_cache.dtype() != ScalarType::kInt8 || v_cache.dtype() != ScalarType::kInt8)
        throw std::invalid_argument("int8 decode attention requires int8 caches");
    if (k_scale.dtype() != ScalarType::kFloat16 || v_scale.dtype() != ScalarType::kFloat16)
        throw std::invalid_argument("int8 decode attention requires float16 scales");
    const IndexRef lens = index_data("context_lens", context_lens);
    const IndexRef tables = index_data("block_tables", block_tables);
    if (block_tables.dim() != 2 || block_tables.sizes()[0] != query.sizes()[0])
        throw std::invalid_argument("block_tables must be [batch, max_blocks]");
    if (static_cast<int64_t>(context_lens.numel()) != query.sizes()[0])
        throw std::invalid_argument("context_lens must hold one entry per sequence");
    if (query.sizes()[2] != head_dim) throw std::invalid_argument("query head_dim does not match head_dim");
    const int64_t batch = query.sizes()[0];
    const int heads = static_cast<int>(query.sizes()[1]);
    const int64_t max_blocks = block_tables.sizes()[1];
    const int64_t per_block = static_cast<int64_t>(block_size) * num_kv_heads * head_dim;
    if (per_block <= 0 || static_cast<int64_t>(k_cache.numel()) % per_block != 0 || k_cache.numel() != v_cache.numel())
        throw std::invalid_argument("int8 caches do not hold a whole number of blocks");
    const int64_t blocks = static_cast<int64_t>(k_cache.numel()) / per_block;
    if (static_cast<int64_t>(k_scale.numel()) != blocks * block_size * num_kv_heads || k_scale.numel() != v_scale.numel())
        throw std::invalid_argument("k_scale and v_scale must hold one value per cache row and KV head");
    // no allocator in this signature (as in the reference): the call runs without split-K scratch
    throw_on_nvk_status(nvk_decode_attention_paged_int8(
        query.data(), k_cache.data(), v_cache.data(), k_scale.data(), v_scale.data(), lens.ptr, lens.dtype, tables.ptr,
        tables.dtype, batch, max_blocks, blocks, heads, num_kv_heads, head_dim, block_size, scale, output.data(), code(query.dtype()), nullptr, 0, stream));
}

// ---- prefill ------------------------------------------------------------------------------------------
void launch_prefill_attention_dense(const Tensor& query, const Tensor* cu_seqlens_q, const Tensor& key,
                                    const Tensor& value, const Tensor* cu_seqlens_k, int num_kv_heads, int head_dim,
                                    float scale, Tensor& output, cudaStream_t stream) {
    check_qo(query, output);
    ensure_cuda_tensor("key", key);
    ensure_cuda_tensor("value", value);
    ensure_same_dtype("query", query, "key", key);
    ensure_same_dtype("query", query, "value", value);
    const bool varlen = cu_seqlens_q != nullptr && cu_seqlens_k != nullptr;   // either missing: one sequence
    const IndexRef cq = varlen ? index_data("cu_seqlens_q", *cu_seqlens_q) : IndexRef{nullptr, NVK_I32};
    const IndexRef ck = varlen ? index_data("cu_seqlens_k", *cu_seqlens_k) : IndexRef{nullptr, NVK_I32};
    const int64_t seqs = varlen ? static_cast<int64_t>(cu_seqlens_q->numel()) - 1 : 1;
    throw_on_nvk_status(nvk_prefill_attention_varlen(query.data(), key.data(), value.data(), nullptr, nullptr, cq.ptr,
                                                     cq.dtype, ck.ptr, ck.dtype, nullptr, NVK_I32, seqs, query.sizes()[0],
                                                     key.sizes()[0], 0, 0, 0,
                                                     static_cast<int>(query.sizes()[1]), num_kv_heads, head_dim, 1, scale,
                                                     output.data(), code(query.dtype()), stream));
}

void launch_prefill_attention_paged(const Tensor& query, const Tensor* cu_seqlens_q, const Tensor& k_cache,
                                    const Tensor& v_cache, const Tensor* cu_seqlens_k, const Tensor& block_tables,
                                    int num_kv_heads, int head_dim, int block_size, float scale, Tensor& output,
                                    cudaStream_t stream) {
    if (cu_seqlens_q == nullptr || cu_seqlens_k == nullptr)
        throw std::invalid_argument("paged prefill attention requires cu_seqlens_q and cu_seqlens_k");
    check_qo(query, output);
    ensure_cuda_tensor("k_cache", k_cache);
    ensure_cuda_tensor("v_cache", v_cache);
    ensure_same_dtype("query", query, "k_cache", k_cache);
    if (block_tables.defined() && block_tables.dim() != 2)
        throw std::invalid_argument("block_tables must be [num_seqs, max_blocks]");
    const IndexRef tables = index_data("block_tables", block_tables);
    const IndexRef cq = index_data("cu_seqlens_q", *cu_seqlens_q), ck = index_data("cu_seqlens_k", *cu_seqlens_k);
    throw_on_nvk_status(nvk_prefill_attention_varlen(
        query.data(), nullptr, nullptr, k_cache.data(), v_cache.data(), cq.ptr, cq.dtype, ck.ptr, ck.dtype, tables.ptr,
        tables.dtype, static_cast<int64_t>(cu_seqlens_q->numel()) - 1,
        query.sizes()[0], 0, block_tables.sizes()[1], cache_blocks(k_cache, block_size, num_kv_heads, head_dim), 0,
        static_cast<int>(query.sizes()[1]), num_kv_heads, head_dim, block_size, scale, output.data(),
        code(query.dtype()), stream));
}

void throw_if_prefill_error(cudaStream_t stream) {
    int word = 0;
    throw_on_nvk_status(nvk_prefill_status(stream, &word));
    if (word != 0)
        throw std::runtime_error("prefill attention: a bounded wait inside the tensor-core kernel ran out (code " +
                                 std::to_string(word) + "); output rows of that launch are incomplete");
}

bool flash_attn_available() { return true; }

void flash_attn_varlen_fwd(const Tensor& query, const Tensor& key, const Tensor& value, const Tensor& cu_seqlens_q,
                           const Tensor& cu_seqlens_k, int /*max_seqlen_q*/, int /*max_seqlen_k*/, float scale,
                           bool is_causal, Tensor& output, DeviceAllocator& /*allocator*/, cudaStream_t stream) {
    if (!is_causal) throw std::invalid_argument("unsupported: non-causal varlen attention");
    const int num_kv_heads = key.defined() && key.dim() == 3 ? static_cast<int>(key.sizes()[1]) : 0;
    const int head_dim = query.defined() && query.dim() == 3 ? static_cast<int>(query.sizes()[2]) : 0;
    launch_prefill_attention_dense(query, &cu_seqlens_q, key, value, &cu_seqlens_k, num_kv_heads, head_dim, scale, output,
                                   stream);
}

}  // namespace nano_vllm
