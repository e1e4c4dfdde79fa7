// Attention layer (interface of include/layers/attention.h:8-46 of the reference): validates the
// operands, writes new K/V into the paged cache and dispatches on the thread's Context.
#pragma once

#include "utils/cuda_allocator.h"
#include "utils/tensor.h"

namespace nano_vllm {

class Attention {
public:
    Attention(int num_heads, int num_kv_heads, int head_dim, int block_size);

    void set_kv_cache(const Tensor& k_cache, const Tensor& v_cache);
    // int8 caches [blocks, block_size, Hkv, D] with fp16 scales [blocks, block_size, Hkv]: new K/V are quantised on
    // store, decode reads them through launch_decode_attention_paged_int8, prefill attends over the dense K/V.
    void set_kv_cache_int8(const Tensor& k_cache, const Tensor& v_cache, const Tensor& k_scale, const Tensor& v_scale);

    // Prefill or decode according to get_context(); stores key/value first when a cache and a
    // slot_mapping are present.  Returns a freshly allocated [tokens, heads, head_dim] tensor.
    Tensor forward(const Tensor& query, const Tensor& key, const Tensor& value, DeviceAllocator& allocator,
                   cudaStream_t stream = nullptr);

    // Decode without the store (the fused prologue already wrote K/V).
    Tensor forward_decode_flash_only(const Tensor& query, DeviceAllocator& allocator, cudaStream_t stream = nullptr);

    Tensor& k_cache() { return k_cache_; }
    Tensor& v_cache() { return v_cache_; }
    const Tensor& k_cache() const { return k_cache_; }
    const Tensor& v_cache() const { return v_cache_; }
    Tensor& k_scale() { return k_scale_; }
    Tensor& v_scale() { return v_scale_; }
    bool is_int8() const { return is_int8_; }

private:
    int num_heads_ = 0;
    int num_kv_heads_ = 0;
    int head_dim_ = 0;
    int block_size_ = 0;
    float scale_ = 1.0f;
    Tensor k_cache_;
    Tensor v_cache_;
    Tensor k_scale_;
    Tensor v_scale_;
    bool is_int8_ = false;
};

}  // namespace nano_vllm
