// The reference reaches FlashAttention-2 through these three entry points
// (include/kernels/flash_attn.h:15-50).  Here they are served by this library's own kernels, so
// flash_attn_available() is always true and the attention layer always takes its fast branches.
#pragma once

#include "utils/cuda_allocator.h"
#include "utils/tensor.h"

namespace nano_vllm {

void flash_attn_varlen_fwd(const Tensor& query, const Tensor& key, const Tensor& value, const Tensor& cu_seqlens_q,
                           const Tensor& cu_seqlens_k, int max_seqlen_q, int max_seqlen_k, float scale, bool is_causal,
                           Tensor& output, DeviceAllocator& allocator, cudaStream_t stream = nullptr);

bool flash_attn_available();

// Split-K scratch is taken from `allocator` (a bump allocator during graph capture).
void flash_attn_decode_kvcache(const Tensor& query, const Tensor& k_cache, const Tensor& v_cache,
                               const Tensor& context_lens, const Tensor& block_tables, int num_kv_heads, int head_dim,
                               int block_size, float scale, Tensor& output, DeviceAllocator& allocator,
                               cudaStream_t stream = nullptr);

}  // namespace nano_vllm
