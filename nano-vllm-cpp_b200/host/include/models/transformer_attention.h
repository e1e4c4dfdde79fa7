// The attention part of a decoder layer between its two linears: the body of TransformerAttention::forward
// (src/models/transformer.cpp:114-156 of the reference) after qkv_proj and before o_proj.  The linears are cuBLAS
// calls of the engine and stay there; what lives here is the choice the reference makes per call:
//
//   fused    decode step, 16-bit cache, q / k norm present, slot_mapping defined, bf16 / fp16 activations
//            (transformer.cpp:125-128): fused_split_norm_rope_store writes K / V straight into the paged cache,
//            then Attention::forward_decode_flash_only;
//   unfused  everything else (prefill, int8 cache, no q / k norm): split -> norm -> rope into dense q / k / v, then
//            Attention::forward, which stores K / V and dispatches on the Context.
//
// Both routes run the same prologue kernel (the unfused one with identity slots into dense k / v tensors), so for
// the same inputs they leave the same bytes in the cache.
#pragma once

#include "layers/attention.h"
#include "utils/cuda_allocator.h"
#include "utils/tensor.h"

namespace nano_vllm {

class TransformerAttention {
public:
    // q_norm_weight / k_norm_weight: [head_dim] tensors of the model dtype, or both undefined (no q / k norm).
    // The rotary table [max_position, head_dim] fp32 = [cos | sin] is built here as RotaryEmbedding does
    // (src/layers/rotary_embedding.cpp:35-47).
    TransformerAttention(int num_heads, int num_kv_heads, int head_dim, int block_size, int max_position, float rope_theta,
                         const Tensor& q_norm_weight, const Tensor& k_norm_weight, float norm_eps, Device device,
                         DeviceAllocator& allocator);

    // qkv: [rows, (num_heads + 2 num_kv_heads) * head_dim], positions: [rows] int32.
    // Returns the attention output [rows, num_heads, head_dim] (the input of o_proj).
    Tensor forward(const Tensor& positions, const Tensor& qkv, DeviceAllocator& allocator, cudaStream_t stream = nullptr);

    // The rule of transformer.cpp:125-128 for the current Context and this qkv dtype.
    bool fused_eligible(const Tensor& qkv) const;
    // Which route the last forward took (tests).
    bool last_forward_was_fused() const { return last_fused_; }

    void set_kv_cache(const Tensor& k_cache, const Tensor& v_cache) { attn_.set_kv_cache(k_cache, v_cache); }
    void set_kv_cache_int8(const Tensor& k_cache, const Tensor& v_cache, const Tensor& k_scale, const Tensor& v_scale) {
        attn_.set_kv_cache_int8(k_cache, v_cache, k_scale, v_scale);
    }
    Attention& attn() { return attn_; }
    const Tensor& cos_sin_cache() const { return cos_sin_cache_; }
    bool has_qk_norm() const { return q_norm_weight_.defined() && k_norm_weight_.defined(); }

private:
    int num_heads_, num_kv_heads_, head_dim_;
    float norm_eps_;
    Tensor q_norm_weight_, k_norm_weight_, cos_sin_cache_;
    Attention attn_;
    bool last_fused_ = false;
};

// split_qkv + optional q / k RMSNorm + neox RoPE into dense tensors (the three kernels of transformer.cpp:144-153 in
// one launch): q [rows, Hq, D], k and v [rows, Hkv, D].  Norm weights may both be undefined.
void split_norm_rope(const Tensor& qkv, const Tensor& positions, const Tensor& q_norm_weight, const Tensor& k_norm_weight,
                     float norm_eps, const Tensor& cos_sin_cache, int num_q_heads, int num_kv_heads, int head_dim,
                     Tensor& q, Tensor& k, Tensor& v, cudaStream_t stream = nullptr);

}  // namespace nano_vllm
