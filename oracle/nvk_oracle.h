/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the attention / paged-KV hot path of
 * nano-vllm-cpp, used as the checker in tests, in the smoke run and as the timed CPU
 * baseline of the benchmark.  Nothing in the product library links or calls this file.
 *
 * Each function follows one CUDA kernel of the reference (cited per function) in plain
 * fp32 C: same head mapping, same bottom-right causal limit, same online-softmax update
 * order (key 0 -> n-1), same lane-strided dot product and xor-butterfly summation.
 *
 * Parity pin: the closed-form known-answer cases of the reference's own tests
 * (tests/test_tensor.cpp:411-450, tests/test_layers.cpp:82-191) and fixtures produced by
 * the reference's own CUDA kernels compiled for sm_100a (tests/golden/).
 */
#ifndef NVK_ORACLE_H
#define NVK_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Output rounding emulation for kernels whose reference instantiation stores T != float. */
enum { ORACLE_ROUND_NONE = 0, ORACLE_ROUND_BF16 = 1, ORACLE_ROUND_FP16 = 2 };

/* src/kernels/kvcache.cu:19-47 (store_kvcache_kernel): byte copy of one row per token into
 * cache row slot_mapping[token]; rows with slot < 0 or slot >= cache_rows are skipped. */
void oracle_store_kvcache(const void* key, const void* value, void* k_cache, void* v_cache,
                          const void* slot_mapping, int slot_is_i64, int64_t num_tokens,
                          int64_t row_bytes, int64_t cache_rows);

/* src/kernels/attention.cu:313-405 (decode_paged_attention_kernel). */
void oracle_decode_attention_paged(const float* query, const float* k_cache, const float* v_cache,
                                   const int32_t* context_lens, const int32_t* block_tables,
                                   int64_t batch, int64_t max_blocks, int num_heads,
                                   int num_kv_heads, int head_dim, int block_size, float scale,
                                   float* output, int num_threads);

/* src/kernels/kvcache.cu:222-296 (store_kvcache_int8_kernel).  key / value are [tokens, Hkv, D] floats already
 * representable in the model dtype; caches are int8 [cache_rows, Hkv, D]; scales are [cache_rows, Hkv], returned as
 * floats that hold the fp16-rounded value the reference stores. */
void oracle_store_kvcache_int8(const float* key, const float* value, int8_t* k_cache, int8_t* v_cache,
                               float* k_scale, float* v_scale, const int32_t* slot_mapping,
                               int64_t num_tokens, int num_kv_heads, int head_dim, int64_t cache_rows);

/* src/kernels/attention.cu:746-842 (decode_paged_attention_int8_kernel). */
void oracle_decode_attention_paged_int8(const float* query, const int8_t* k_cache, const int8_t* v_cache,
                                        const float* k_scale, const float* v_scale,
                                        const int32_t* context_lens, const int32_t* block_tables,
                                        int64_t batch, int64_t max_blocks, int num_heads, int num_kv_heads,
                                        int head_dim, int block_size, float scale, float* output, int num_threads);

/* fp8 (e4m3) KV cache: no counterpart in the reference (PARITY UNPINNED for this format); the layout and the arithmetic
 * follow its int8 cache with the range of the type: scale = max(absmax / 448, 1e-10) as fp16 per (cache row, KV head),
 * elements = e4m3(x * 448 / max(absmax, 1e-10)), round to nearest even, saturating. */
void oracle_store_kvcache_fp8(const float* key, const float* value, uint8_t* k_cache, uint8_t* v_cache,
                              float* k_scale, float* v_scale, const int32_t* slot_mapping, int64_t num_tokens,
                              int num_kv_heads, int head_dim, int64_t cache_rows);
void oracle_decode_attention_paged_fp8(const float* query, const uint8_t* k_cache, const uint8_t* v_cache,
                                       const float* k_scale, const float* v_scale, const int32_t* context_lens,
                                       const int32_t* block_tables, int64_t batch, int64_t max_blocks, int num_heads,
                                       int num_kv_heads, int head_dim, int block_size, float scale, float* output);

/* src/kernels/attention.cu:114-202 (prefill_dense_attention_kernel) with
 * locate_prefill_sequence (:27-54).  cu_seqlens_* may both be NULL: one sequence. */
void oracle_prefill_attention_dense(const float* query, const float* key, const float* value,
                                    const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                    int64_t num_seqs, int64_t query_rows, int64_t key_rows,
                                    int num_heads, int num_kv_heads, int head_dim, float scale,
                                    float* output, int num_threads);

/* src/kernels/attention.cu:205-302 (prefill_paged_attention_kernel). */
void oracle_prefill_attention_paged(const float* query, const float* k_cache, const float* v_cache,
                                    const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                    const int32_t* block_tables, int64_t num_seqs,
                                    int64_t query_rows, int64_t max_blocks, int num_heads,
                                    int num_kv_heads, int head_dim, int block_size, float scale,
                                    float* output, int num_threads);

/* src/kernels/split_qkv.cu:62-154 (fused_split_norm_rope_store_kernel).  All float arrays hold
 * values already representable in the model dtype; `round_mode` applies the store rounding
 * the reference's from_float<T> performs.  cos_sin_cache is [max_positions, head_dim] fp32. */
void oracle_fused_split_norm_rope_store(const float* qkv, const int32_t* positions,
                                        const float* q_norm_weight, const float* k_norm_weight,
                                        float norm_eps, const float* cos_sin_cache,
                                        int max_positions, const int32_t* slot_mapping,
                                        float* k_cache, float* v_cache, int64_t rows,
                                        int num_q_heads, int num_kv_heads, int head_dim,
                                        float* q_out, int round_mode);

/* src/layers/rotary_embedding.cpp:35-47: fp32 table [max_position, rotary_dim] =
 * [cos(pos*inv_freq_i) | sin(pos*inv_freq_i)], inv_freq_i = base^(-2i/rotary_dim). */
void oracle_build_cos_sin_cache(float* table, int max_position, int rotary_dim, float base);

/* Round-to-nearest-even conversions used for the emulated stores. */
float oracle_round_bf16(float x);
float oracle_round_fp16(float x);

#ifdef __cplusplus
}
#endif
#endif
