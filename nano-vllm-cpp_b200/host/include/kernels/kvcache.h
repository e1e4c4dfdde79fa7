// store_kvcache operator (signature of include/kernels/kvcache.h:7-12 of the reference).
#pragma once

#include "utils/tensor.h"

namespace nano_vllm {

// cache row slot_mapping[t] <- key / value row t; slots < 0 or beyond the cache are skipped.
void store_kvcache(const Tensor& key, const Tensor& value, Tensor& k_cache, Tensor& v_cache,
                   const Tensor& slot_mapping, cudaStream_t stream = nullptr);

// int8 KV cache (include/kernels/kvcache.h:14-24 of the reference): key / value [tokens, Hkv, D] are quantised per
// (token, KV head) into int8 caches [.., Hkv, D] with one fp16 scale each in k_scale / v_scale [.., Hkv].
void store_kvcache_int8(const Tensor& key, const Tensor& value, Tensor& k_cache, Tensor& v_cache, Tensor& k_scale,
                        Tensor& v_scale, const Tensor& slot_mapping, cudaStream_t stream = nullptr);

}  // namespace nano_vllm
