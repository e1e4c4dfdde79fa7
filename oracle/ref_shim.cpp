// TEST INFRASTRUCTURE ONLY.  C shim over the reference's own C++ operator API
// (include/kernels/attention.h:7-41, include/kernels/kvcache.h:7-12,
// include/kernels/split_qkv.h:22-33) so that tests and the benchmark's reference arm can run
// the reference's unmodified CUDA kernels, compiled for sm_100a, on raw device pointers.
// Compiled together with the reference sources by oracle/Makefile into oracle/_ref/; this
// file contains no arithmetic of its own.
#include "kernels/attention.h"
#include "kernels/kvcache.h"
#include "kernels/split_qkv.h"
#include "utils/tensor.h"

#include <cuda_runtime_api.h>

#include <cstdint>
#include <exception>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

thread_local std::string g_error;

nano_vllm::Tensor borrow(const void* ptr, const std::vector<int64_t>& sizes, int dtype) {
    using namespace nano_vllm;
    const ScalarType st = static_cast<ScalarType>(dtype);
    int device = 0;
    cudaGetDevice(&device);
    const size_t bytes = compute_numel(sizes) * scalar_type_size(st);
    Memory::Ptr mem = Memory::make_borrowed(const_cast<void*>(ptr), bytes, Device{DeviceType::kCUDA, device});
    return Tensor::from_memory(mem, sizes, st);
}

template <typename Fn>
int guarded(Fn&& fn) {
    try {
        fn();
        return 0;
    } catch (const std::invalid_argument& e) {
        g_error = e.what();
        return 1;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 2;
    }
}

}  // namespace

extern "C" {

const char* nvkref_last_error() { return g_error.c_str(); }

// dtype codes follow the reference's ScalarType order (include/utils/tensor.h:21-28):
// 0 fp16, 1 bf16, 2 fp32, 3 int32, 4 int64.
int nvkref_store_kvcache(const void* key, const void* value, void* k_cache, void* v_cache,
                         const void* slot_mapping, int slot_dtype, int64_t num_tokens,
                         int64_t row_elems, int64_t cache_rows, int dtype, void* stream) {
    return guarded([&] {
        auto k = borrow(key, {num_tokens, row_elems}, dtype);
        auto v = borrow(value, {num_tokens, row_elems}, dtype);
        auto kc = borrow(k_cache, {cache_rows, row_elems}, dtype);
        auto vc = borrow(v_cache, {cache_rows, row_elems}, dtype);
        auto sm = borrow(slot_mapping, {num_tokens}, slot_dtype);
        nano_vllm::store_kvcache(k, v, kc, vc, sm, static_cast<cudaStream_t>(stream));
    });
}

int nvkref_decode_attention_paged(const void* query, const void* k_cache, const void* v_cache,
                                  const void* context_lens, const void* block_tables,
                                  int64_t batch, int64_t max_blocks, int64_t num_cache_blocks,
                                  int num_heads, int num_kv_heads, int head_dim, int block_size,
                                  float scale, void* output, int dtype, void* stream) {
    return guarded([&] {
        auto q = borrow(query, {batch, num_heads, head_dim}, dtype);
        auto o = borrow(output, {batch, num_heads, head_dim}, dtype);
        auto kc = borrow(k_cache, {num_cache_blocks, block_size, num_kv_heads, head_dim}, dtype);
        auto vc = borrow(v_cache, {num_cache_blocks, block_size, num_kv_heads, head_dim}, dtype);
        auto cl = borrow(context_lens, {batch}, 3);
        auto bt = borrow(block_tables, {batch, max_blocks}, 3);
        nano_vllm::launch_decode_attention_paged(q, kc, vc, cl, bt, num_kv_heads, head_dim,
                                                 block_size, scale, o,
                                                 static_cast<cudaStream_t>(stream));
    });
}

/* int8 KV cache: caches are int8 (dtype code 5), scales fp16 (code 0), both per the reference's headers
 * (include/kernels/kvcache.h:14-24, include/kernels/attention.h:43-56). */
int nvkref_store_kvcache_int8(const void* key, const void* value, void* k_cache, void* v_cache, void* k_scale,
                              void* v_scale, const void* slot_mapping, int64_t num_tokens, int num_kv_heads,
                              int head_dim, int64_t num_cache_blocks, int block_size, int dtype, void* stream) {
    return guarded([&] {
        auto k = borrow(key, {num_tokens, num_kv_heads, head_dim}, dtype);
        auto v = borrow(value, {num_tokens, num_kv_heads, head_dim}, dtype);
        auto kc = borrow(k_cache, {num_cache_blocks, block_size, num_kv_heads, head_dim}, 5);
        auto vc = borrow(v_cache, {num_cache_blocks, block_size, num_kv_heads, head_dim}, 5);
        auto ks = borrow(k_scale, {num_cache_blocks, block_size, num_kv_heads}, 0);
        auto vs = borrow(v_scale, {num_cache_blocks, block_size, num_kv_heads}, 0);
        auto sm = borrow(slot_mapping, {num_tokens}, 3);
        nano_vllm::store_kvcache_int8(k, v, kc, vc, ks, vs, sm, static_cast<cudaStream_t>(stream));
    });
}

int nvkref_decode_attention_paged_int8(const void* query, const void* k_cache, const void* v_cache,
                                       const void* k_scale, const void* v_scale, const void* context_lens,
                                       const void* block_tables, int64_t batch, int64_t max_blocks,
                                       int64_t num_cache_blocks, int num_heads, int num_kv_heads, int head_dim,
                                       int block_size, float scale, void* output, int dtype, void* stream) {
    return guarded([&] {
        auto q = borrow(query, {batch, num_heads, head_dim}, dtype);
        auto o = borrow(output, {batch, num_heads, head_dim}, dtype);
        auto kc = borrow(k_cache, {num_cache_blocks, block_size, num_kv_heads, head_dim}, 5);
        auto vc = borrow(v_cache, {num_cache_blocks, block_size, num_kv_heads, head_dim}, 5);
        auto ks = borrow(k_scale, {num_cache_blocks, block_size, num_kv_heads}, 0);
        auto vs = borrow(v_scale, {num_cache_blocks, block_size, num_kv_heads}, 0);
        auto cl = borrow(context_lens, {batch}, 3);
        auto bt = borrow(block_tables, {batch, max_blocks}, 3);
        nano_vllm::launch_decode_attention_paged_int8(q, kc, vc, ks, vs, cl, bt, num_kv_heads, head_dim,
                                                      block_size, scale, o, static_cast<cudaStream_t>(stream));
    });
}

int nvkref_prefill_attention_dense(const void* query, const void* key, const void* value,
                                   const void* cu_seqlens_q, const void* cu_seqlens_k,
                                   int64_t num_seqs, int64_t total_q, int64_t total_k,
                                   int num_heads, int num_kv_heads, int head_dim, float scale,
                                   void* output, int dtype, void* stream) {
    return guarded([&] {
        auto q = borrow(query, {total_q, num_heads, head_dim}, dtype);
        auto o = borrow(output, {total_q, num_heads, head_dim}, dtype);
        auto k = borrow(key, {total_k, num_kv_heads, head_dim}, dtype);
        auto v = borrow(value, {total_k, num_kv_heads, head_dim}, dtype);
        if (cu_seqlens_q != nullptr && cu_seqlens_k != nullptr) {
            auto cq = borrow(cu_seqlens_q, {num_seqs + 1}, 3);
            auto ck = borrow(cu_seqlens_k, {num_seqs + 1}, 3);
            nano_vllm::launch_prefill_attention_dense(q, &cq, k, v, &ck, num_kv_heads, head_dim,
                                                      scale, o, static_cast<cudaStream_t>(stream));
        } else {
            nano_vllm::launch_prefill_attention_dense(q, nullptr, k, v, nullptr, num_kv_heads,
                                                      head_dim, scale, o,
                                                      static_cast<cudaStream_t>(stream));
        }
    });
}

int nvkref_prefill_attention_paged(const void* query, const void* k_cache, const void* v_cache,
                                   const void* cu_seqlens_q, const void* cu_seqlens_k,
                                   const void* block_tables, int64_t num_seqs, int64_t total_q,
                                   int64_t max_blocks, int64_t num_cache_blocks, int num_heads,
                                   int num_kv_heads, int head_dim, int block_size, float scale,
                                   void* output, int dtype, void* stream) {
    return guarded([&] {
        auto q = borrow(query, {total_q, num_heads, head_dim}, dtype);
        auto o = borrow(output, {total_q, num_heads, head_dim}, dtype);
        auto kc = borrow(k_cache, {num_cache_blocks, block_size, num_kv_heads, head_dim}, dtype);
        auto vc = borrow(v_cache, {num_cache_blocks, block_size, num_kv_heads, head_dim}, dtype);
        auto cq = borrow(cu_seqlens_q, {num_seqs + 1}, 3);
        auto ck = borrow(cu_seqlens_k, {num_seqs + 1}, 3);
        auto bt = borrow(block_tables, {num_seqs, max_blocks}, 3);
        nano_vllm::launch_prefill_attention_paged(q, &cq, kc, vc, &ck, bt, num_kv_heads, head_dim,
                                                  block_size, scale, o,
                                                  static_cast<cudaStream_t>(stream));
    });
}

int nvkref_fused_split_norm_rope_store(const void* qkv, const void* positions,
                                       const void* q_norm_weight, const void* k_norm_weight,
                                       float norm_eps, const void* cos_sin_cache,
                                       int64_t max_positions, const void* slot_mapping,
                                       void* k_cache, void* v_cache, int64_t cache_rows,
                                       int64_t rows, int num_q_heads, int num_kv_heads,
                                       int head_dim, void* q_out, int dtype, void* stream) {
    return guarded([&] {
        const int64_t cols = static_cast<int64_t>(num_q_heads + 2 * num_kv_heads) * head_dim;
        auto x = borrow(qkv, {rows, cols}, dtype);
        auto pos = borrow(positions, {rows}, 3);
        auto qw = borrow(q_norm_weight, {head_dim}, dtype);
        auto kw = borrow(k_norm_weight, {head_dim}, dtype);
        auto cs = borrow(cos_sin_cache, {max_positions, head_dim}, 2);
        auto sm = borrow(slot_mapping, {rows}, 3);
        auto kc = borrow(k_cache, {cache_rows, num_kv_heads, head_dim}, dtype);
        auto vc = borrow(v_cache, {cache_rows, num_kv_heads, head_dim}, dtype);
        auto qo = borrow(q_out, {rows, num_q_heads, head_dim}, dtype);
        nano_vllm::fused_split_norm_rope_store(x, pos, qw, kw, norm_eps, cs, sm, kc, vc,
                                               num_q_heads, num_kv_heads, head_dim, qo,
                                               static_cast<cudaStream_t>(stream));
    });
}

}  // extern "C"
