// TransformerAttention: the fused-versus-unfused choice of src/models/transformer.cpp:114-156 of the reference over
// this library's prologue kernel and Attention layer (interface: models/transformer_attention.h).
#include "models/transformer_attention.h"

#include "kernels/kernel_types.h"
#include "kernels/split_qkv.h"
#include "utils/context.h"

#include "nvk.h"

#include <cmath>
#include <stdexcept>
#include <vector>

namespace nano_vllm {

namespace {

bool is_half_type(ScalarType t) { return t == ScalarType::kBFloat16 || t == ScalarType::kFloat16; }

}  // namespace

void split_norm_rope(const Tensor& qkv, const Tensor& positions, const Tensor& q_norm_weight, const Tensor& k_norm_weight,
                     float norm_eps, const Tensor& cos_sin_cache, int num_q_heads, int num_kv_heads, int head_dim,
                     Tensor& q, Tensor& k, Tensor& v, cudaStream_t stream) {
    ensure_cuda_tensor("qkv", qkv);
    ensure_cuda_tensor("positions", positions);
    ensure_cuda_tensor("cos_sin_cache", cos_sin_cache);
    ensure_cuda_tensor("q", q);
    ensure_cuda_tensor("k", k);
    ensure_cuda_tensor("v", v);
    if (!is_half_type(qkv.dtype())) throw std::invalid_argument("split_norm_rope only supports bf16/fp16");
    if (positions.dtype() != ScalarType::kInt32) throw std::invalid_argument("positions must be int32");
    if (q_norm_weight.defined() != k_norm_weight.defined())
        throw std::invalid_argument("q_norm_weight and k_norm_weight must both be defined or both undefined");
    if (cos_sin_cache.dtype() != ScalarType::kFloat32 || cos_sin_cache.dim() != 2)
        throw std::invalid_argument("cos_sin_cache must be a [max_positions, head_dim] float32 tensor");
    const int64_t rows = qkv.sizes()[0];
    if (static_cast<int64_t>(k.numel()) != rows * num_kv_heads * head_dim || k.numel() != v.numel() ||
        static_cast<int64_t>(q.numel()) != rows * num_q_heads * head_dim)
        throw std::invalid_argument("q, k and v do not match the packed qkv tensor");
    throw_on_nvk_status(nvk_fused_split_norm_rope_store(
        qkv.data(), positions.data_as<int32_t>(), q_norm_weight.defined() ? q_norm_weight.data() : nullptr,
        k_norm_weight.defined() ? k_norm_weight.data() : nullptr, norm_eps, cos_sin_cache.data_as<float>(),
        cos_sin_cache.sizes()[0], /*slot_mapping=*/nullptr, k.data(), v.data(), /*cache_rows=*/rows, rows, num_q_heads,
        num_kv_heads, head_dim, q.data(), static_cast<int>(qkv.dtype()), stream));
}

TransformerAttention::TransformerAttention(int num_heads, int num_kv_heads, int head_dim, int block_size, int max_position,
                                           float rope_theta, const Tensor& q_norm_weight, const Tensor& k_norm_weight,
                                           float norm_eps, Device device, DeviceAllocator& allocator)
    : num_heads_(num_heads), num_kv_heads_(num_kv_heads), head_dim_(head_dim), norm_eps_(norm_eps),
      q_norm_weight_(q_norm_weight), k_norm_weight_(k_norm_weight),
      attn_(num_heads, num_kv_heads, head_dim, block_size) {
    if (max_position <= 0) throw std::invalid_argument("rotary embedding dimensions must be positive");
    if (head_dim % 2 != 0) throw std::invalid_argument("rotary_dim must be even");
    if (q_norm_weight.defined() != k_norm_weight.defined())
        throw std::invalid_argument("q_norm_weight and k_norm_weight must both be defined or both undefined");
    cos_sin_cache_ = Tensor::empty({max_position, head_dim}, ScalarType::kFloat32, device, allocator);
    std::vector<float> host(static_cast<size_t>(max_position) * static_cast<size_t>(head_dim), 0.0f);
    const int half = head_dim / 2;
    for (int idx = 0; idx < half; ++idx) {
        const float inv_freq = 1.0f / std::pow(rope_theta, static_cast<float>(2 * idx) / static_cast<float>(head_dim));
        for (int pos = 0; pos < max_position; ++pos) {
            const float angle = static_cast<float>(pos) * inv_freq;
            host[static_cast<size_t>(pos) * head_dim + idx] = std::cos(angle);
            host[static_cast<size_t>(pos) * head_dim + idx + half] = std::sin(angle);
        }
    }
    allocator.copy_to_device_async(cos_sin_cache_.data(), host.data(), cos_sin_cache_.nbytes(), nullptr);
    allocator.synchronize_stream(nullptr);
}

bool TransformerAttention::fused_eligible(const Tensor& qkv) const {
    const Context& ctx = get_context();
    return !ctx.is_prefill && !attn_.is_int8() && has_qk_norm() && ctx.slot_mapping.defined() && is_half_type(qkv.dtype());
}

Tensor TransformerAttention::forward(const Tensor& positions, const Tensor& qkv, DeviceAllocator& allocator,
                                     cudaStream_t stream) {
    ensure_cuda_tensor("qkv", qkv);
    if (qkv.dim() != 2 || qkv.sizes()[1] != static_cast<int64_t>(num_heads_ + 2 * num_kv_heads_) * head_dim_)
        throw std::invalid_argument("qkv must be [rows, (num_heads + 2 * num_kv_heads) * head_dim]");
    const int64_t rows = qkv.sizes()[0];
    Tensor q = Tensor::empty({rows, num_heads_, head_dim_}, qkv.dtype(), qkv.device(), allocator);
    last_fused_ = fused_eligible(qkv);
    if (last_fused_) {
        const Context& ctx = get_context();
        fused_split_norm_rope_store(qkv, positions, q_norm_weight_, k_norm_weight_, norm_eps_, cos_sin_cache_,
                                    ctx.slot_mapping, attn_.k_cache(), attn_.v_cache(), num_heads_, num_kv_heads_, head_dim_,
                                    q, stream);
        return attn_.forward_decode_flash_only(q, allocator, stream);
    }
    Tensor k = Tensor::empty({rows, num_kv_heads_, head_dim_}, qkv.dtype(), qkv.device(), allocator);
    Tensor v = Tensor::empty({rows, num_kv_heads_, head_dim_}, qkv.dtype(), qkv.device(), allocator);
    split_norm_rope(qkv, positions, q_norm_weight_, k_norm_weight_, norm_eps_, cos_sin_cache_, num_heads_, num_kv_heads_,
                    head_dim_, q, k, v, stream);
    return attn_.forward(q, k, v, allocator, stream);
}

}  // namespace nano_vllm
