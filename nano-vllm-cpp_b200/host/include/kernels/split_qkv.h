// Fused decode prologue (signature of include/kernels/split_qkv.h:22-33 of the reference).
#pragma once

#include "utils/tensor.h"

namespace nano_vllm {

// split packed qkv + RMSNorm(q, k) + neox RoPE(q, k); q -> q_out, k / v -> cache row slot_mapping[row].
void fused_split_norm_rope_store(const Tensor& qkv, const Tensor& positions, const Tensor& q_norm_weight,
                                 const Tensor& k_norm_weight, float norm_eps, const Tensor& cos_sin_cache,
                                 const Tensor& slot_mapping, Tensor& k_cache, Tensor& v_cache, int num_q_heads,
                                 int num_kv_heads, int head_dim, Tensor& q_out, cudaStream_t stream = nullptr);

}  // namespace nano_vllm
