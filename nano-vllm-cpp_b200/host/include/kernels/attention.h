// Attention operators (signatures of include/kernels/attention.h:7-56 of the reference).
#pragma once

#include "utils/tensor.h"

namespace nano_vllm {

void launch_prefill_attention_dense(const Tensor& query, const Tensor* cu_seqlens_q, const Tensor& key,
                                    const Tensor& value, const Tensor* cu_seqlens_k, int num_kv_heads, int head_dim,
                                    float scale, Tensor& output, cudaStream_t stream = nullptr);

void launch_prefill_attention_paged(const Tensor& query, const Tensor* cu_seqlens_q, const Tensor& k_cache,
                                    const Tensor& v_cache, const Tensor* cu_seqlens_k, const Tensor& block_tables,
                                    int num_kv_heads, int head_dim, int block_size, float scale, Tensor& output,
                                    cudaStream_t stream = nullptr);

// No allocator in this signature: split-K scratch comes from the library's built-in array
// (nvk_decode_attention_paged_static) when the problem fits nvk_decode_attention_static_scratch_bytes(), otherwise the
// call runs unsplit.  Two rules follow from sharing that array, neither of which the reference's function has:
// calls whose kernels may overlap on one device (different streams) race on it and must be serialised by the caller,
// and the first call on a device looks the array's address up, which must not happen inside a stream capture -- make
// one call (or construct an Attention layer and run a warm-up step, as a graph runner does anyway) before capturing.
void launch_decode_attention_paged(const Tensor& query, const Tensor& k_cache, const Tensor& v_cache,
                                   const Tensor& context_lens, const Tensor& block_tables, int num_kv_heads,
                                   int head_dim, int block_size, float scale, Tensor& output,
                                   cudaStream_t stream = nullptr);

// Decode attention over an int8 cache with fp16 scales (include/kernels/attention.h:43-56 of the reference).
void launch_decode_attention_paged_int8(const Tensor& query, const Tensor& k_cache, const Tensor& v_cache,
                                        const Tensor& k_scale, const Tensor& v_scale, const Tensor& context_lens,
                                        const Tensor& block_tables, int num_kv_heads, int head_dim, int block_size,
                                        float scale, Tensor& output, cudaStream_t stream = nullptr);

// The tensor-core prefill kernel bounds every internal wait; a launch whose wait ran out leaves rows unwritten and
// records the fact on the device.  This call synchronises `stream`, and throws std::runtime_error if any prefill launch
// since the previous call gave up (call it where the engine synchronises anyway, e.g. after a prefill step).
void throw_if_prefill_error(cudaStream_t stream = nullptr);

}  // namespace nano_vllm
