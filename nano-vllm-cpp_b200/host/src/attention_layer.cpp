// Attention layer over this library's kernels (interface: layers/attention.h; behaviour of
// src/layers/attention.cpp:44-283 of the reference).  The reference picks between its own scalar
// kernels, a dlopen'ed FlashAttention-2 and int8 variants; here there is one backend, so the dispatch
// reduces to prefill (paged / dense) versus decode.
#include "layers/attention.h"

#include "kernels/attention.h"
#include "kernels/flash_attn.h"
#include "kernels/kvcache.h"
#include "utils/context.h"

#include <cmath>
#include <stdexcept>
#include <string>

namespace nano_vllm {

namespace {

void require_cuda_contiguous(const char* name, const Tensor& t) {
    if (!t.defined()) throw std::invalid_argument(std::string(name) + " must be defined");
    if (t.device().type != DeviceType::kCUDA) throw std::invalid_argument(std::string(name) + " must live on CUDA");
    if (!t.is_contiguous()) throw std::invalid_argument(std::string(name) + " must be contiguous");
}

void require_compute_dtype(const char* name, const Tensor& t) {
    const ScalarType d = t.dtype();
    if (d != ScalarType::kFloat32 && d != ScalarType::kFloat16 && d != ScalarType::kBFloat16)
        throw std::invalid_argument(std::string(name) + " must be float32, float16, or bfloat16");
}

void require_index_tensor(const char* name, const Tensor& t) {
    require_cuda_contiguous(name, t);
    if (t.dtype() != ScalarType::kInt32 && t.dtype() != ScalarType::kInt64)
        throw std::invalid_argument(std::string(name) + " must be int32 or int64");
}

}  // namespace

Attention::Attention(int num_heads, int num_kv_heads, int head_dim, int block_size)
    : num_heads_(num_heads), num_kv_heads_(num_kv_heads), head_dim_(head_dim), block_size_(block_size) {
    if (num_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || block_size <= 0)
        throw std::invalid_argument("attention dimensions must be positive");
    if (num_heads % num_kv_heads != 0) throw std::invalid_argument("num_heads must be divisible by num_kv_heads");
    scale_ = 1.0f / std::sqrt(static_cast<float>(head_dim));
}

void Attention::set_kv_cache(const Tensor& k_cache, const Tensor& v_cache) {
    require_cuda_contiguous("k_cache", k_cache);
    require_cuda_contiguous("v_cache", v_cache);
    require_compute_dtype("k_cache", k_cache);
    require_compute_dtype("v_cache", v_cache);
    if (k_cache.sizes() != v_cache.sizes()) throw std::invalid_argument("k_cache and v_cache must have the same shape");
    k_cache_ = k_cache;
    v_cache_ = v_cache;
    is_int8_ = false;
}

void Attention::set_kv_cache_int8(const Tensor& k_cache, const Tensor& v_cache, const Tensor& k_scale, const Tensor& v_scale) {
    require_cuda_contiguous("k_cache", k_cache);
    require_cuda_contiguous("v_cache", v_cache);
    require_cuda_contiguous("k_scale", k_scale);
    require_cuda_contiguous("v_scale", v_scale);
    if (k_cache.dtype() != ScalarType::kInt8 || v_cache.dtype() != ScalarType::kInt8)
        throw std::invalid_argument("int8 KV cache tensors must be int8");
    if (k_scale.dtype() != ScalarType::kFloat16 || v_scale.dtype() != ScalarType::kFloat16)
        throw std::invalid_argument("int8 KV cache scales must be float16");
    k_cache_ = k_cache;
    v_cache_ = v_cache;
    k_scale_ = k_scale;
    v_scale_ = v_scale;
    is_int8_ = true;
}

Tensor Attention::forward(const Tensor& query, const Tensor& key, const Tensor& value, DeviceAllocator& allocator,
                          cudaStream_t stream) {
    require_cuda_contiguous("query", query);
    require_cuda_contiguous("key", key);
    require_cuda_contiguous("value", value);
    require_compute_dtype("query", query);
    require_compute_dtype("key", key);
    require_compute_dtype("value", value);
    if (query.dim() != 3 || key.dim() != 3 || value.dim() != 3)
        throw std::invalid_argument("attention expects [tokens, heads, head_dim] tensors");
    if (query.sizes()[1] != num_heads_ || key.sizes()[1] != num_kv_heads_ || value.sizes()[1] != num_kv_heads_)
        throw std::invalid_argument("attention tensor heads do not match the configured head counts");
    if (query.sizes()[2] != head_dim_ || key.sizes()[2] != head_dim_ || value.sizes()[2] != head_dim_)
        throw std::invalid_argument("attention tensor head_dim does not match the configured head_dim");
    if (key.sizes() != value.sizes()) throw std::invalid_argument("key and value must have the same shape");

    const Context& ctx = get_context();
    if (ctx.cu_seqlens_q.defined()) require_index_tensor("cu_seqlens_q", ctx.cu_seqlens_q);
    if (ctx.cu_seqlens_k.defined()) require_index_tensor("cu_seqlens_k", ctx.cu_seqlens_k);
    if (ctx.slot_mapping.defined()) require_index_tensor("slot_mapping", ctx.slot_mapping);
    if (ctx.context_lens.defined()) require_index_tensor("context_lens", ctx.context_lens);
    if (ctx.block_tables.defined()) require_index_tensor("block_tables", ctx.block_tables);

    // new K/V go into the cache first: both prefill-with-prefix and decode read them back from it
    if (k_cache_.defined() && ctx.slot_mapping.defined()) {
        if (is_int8_) {
            store_kvcache_int8(key, value, k_cache_, v_cache_, k_scale_, v_scale_, ctx.slot_mapping, stream);
        } else {
            store_kvcache(key, value, k_cache_, v_cache_, ctx.slot_mapping, stream);
        }
    }

    Tensor output = Tensor::empty(query.sizes(), query.dtype(), query.device(), allocator);
    const bool paged = k_cache_.defined() && v_cache_.defined() && ctx.block_tables.defined();
    if (ctx.is_prefill) {
        const Tensor* cu_q = ctx.cu_seqlens_q.defined() ? &ctx.cu_seqlens_q : nullptr;
        const Tensor* cu_k = ctx.cu_seqlens_k.defined() ? &ctx.cu_seqlens_k : nullptr;
        if (paged && !is_int8_) {   // an int8 cache is only read by decode: prefill attends over the dense K / V it was given
            if (cu_k == nullptr) throw std::invalid_argument("prefill attention with block_tables requires cu_seqlens_k");
            launch_prefill_attention_paged(query, cu_q, k_cache_, v_cache_, cu_k, ctx.block_tables, num_kv_heads_,
                                           head_dim_, block_size_, scale_, output, stream);
        } else {
            launch_prefill_attention_dense(query, cu_q, key, value, cu_k, num_kv_heads_, head_dim_, scale_, output, stream);
        }
        return output;
    }
    if (!paged || !ctx.context_lens.defined())
        throw std::invalid_argument("decode attention requires KV cache, context_lens, and block_tables");
    if (is_int8_) {
        launch_decode_attention_paged_int8(query, k_cache_, v_cache_, k_scale_, v_scale_, ctx.context_lens, ctx.block_tables,
                                           num_kv_heads_, head_dim_, block_size_, scale_, output, stream);
        return output;
    }
    flash_attn_decode_kvcache(query, k_cache_, v_cache_, ctx.context_lens, ctx.block_tables, num_kv_heads_, head_dim_,
                              block_size_, scale_, output, allocator, stream);
    return output;
}

Tensor Attention::forward_decode_flash_only(const Tensor& query, DeviceAllocator& allocator, cudaStream_t stream) {
    const Context& ctx = get_context();
    if (!k_cache_.defined() || !v_cache_.defined() || !ctx.block_tables.defined() || !ctx.context_lens.defined())
        throw std::invalid_argument("forward_decode_flash_only requires KV cache, context_lens, and block_tables");
    require_cuda_contiguous("query", query);
    Tensor output = Tensor::empty(query.sizes(), query.dtype(), query.device(), allocator);
    if (is_int8_) {
        launch_decode_attention_paged_int8(query, k_cache_, v_cache_, k_scale_, v_scale_, ctx.context_lens, ctx.block_tables,
                                           num_kv_heads_, head_dim_, block_size_, scale_, output, stream);
        return output;
    }
    flash_attn_decode_kvcache(query, k_cache_, v_cache_, ctx.context_lens, ctx.block_tables, num_kv_heads_, head_dim_,
                              block_size_, scale_, output, allocator, stream);
    return output;
}

}  // namespace nano_vllm
