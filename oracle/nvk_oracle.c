/*
 * TEST INFRASTRUCTURE ONLY -- see nvk_oracle.h.  Plain C (C99 + optional OpenMP) fp32
 * restatement of the reference's attention / KV-store kernels.  Never linked into the
 * product library; imported only by the tests, the smoke run and the benchmark's CPU
 * baseline leg.
 */
#include "nvk_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_WARP 32

/* ---- rounding helpers ------------------------------------------------------------- */

float oracle_round_bf16(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) { /* NaN: keep quiet NaN */
        u = (u | 0x00400000u) & 0xffff0000u;
    } else {
        const uint32_t lsb = (u >> 16) & 1u;
        u += 0x7fffu + lsb;
        u &= 0xffff0000u;
    }
    memcpy(&x, &u, 4);
    return x;
}

float oracle_round_fp16(float x) {
    /* round-to-nearest-even to IEEE binary16, returned as float */
    uint32_t u;
    memcpy(&u, &x, 4);
    const uint32_t sign = u & 0x80000000u;
    const uint32_t a = u & 0x7fffffffu;
    float r;
    if (a >= 0x7f800000u) { /* inf / nan */
        return x;
    }
    if (a >= 0x477ff000u) { /* >= 65520 -> inf */
        const uint32_t inf = sign | 0x7f800000u;
        memcpy(&r, &inf, 4);
        return r;
    }
    if (a < 0x38800000u) { /* subnormal half: quantum 2^-24 */
        float ax;
        memcpy(&ax, &a, 4);
        const float q = 5.9604644775390625e-08f; /* 2^-24 */
        float n = nearbyintf(ax / q) * q;         /* default rounding mode = RNE */
        uint32_t nu;
        memcpy(&nu, &n, 4);
        nu |= sign;
        memcpy(&r, &nu, 4);
        return r;
    }
    {
        uint32_t m = a;
        const uint32_t lsb = (m >> 13) & 1u;
        m += 0xfffu + lsb;
        m &= 0xffffe000u;
        m |= sign;
        memcpy(&r, &m, 4);
        return r;
    }
}

static float round_store(float x, int mode) {
    if (mode == ORACLE_ROUND_BF16) return oracle_round_bf16(x);
    if (mode == ORACLE_ROUND_FP16) return oracle_round_fp16(x);
    return x;
}

/* ---- summation trees of the reference ------------------------------------------------ */

/* include/kernels/device_helpers.cuh:57-63 and src/kernels/attention.cu:68-74:
 * xor-butterfly over 32 lanes (offsets 16, 8, 4, 2, 1); every lane ends with the same value. */
static float butterfly_sum(float* lanes) {
    for (int offset = ORACLE_WARP / 2; offset >= 1; offset >>= 1) {
        float next[ORACLE_WARP];
        for (int l = 0; l < ORACLE_WARP; ++l) next[l] = lanes[l] + lanes[l ^ offset];
        memcpy(lanes, next, sizeof(next));
    }
    return lanes[0];
}

/* src/kernels/attention.cu:363-379: lane l accumulates d = l, l+32, l+64, l+96 with
 * `partial += q*k` (fused multiply-add on the GPU), then warp_reduce_sum. */
static float warp_strided_dot(const float* q, const float* k, int head_dim) {
    float lanes[ORACLE_WARP];
    for (int l = 0; l < ORACLE_WARP; ++l) {
        float partial = 0.0f;
        for (int i = 0; i < 4; ++i) {
            const int d = l + i * ORACLE_WARP;
            if (d < head_dim) partial = fmaf(q[d], k[d], partial);
        }
        lanes[l] = partial;
    }
    return butterfly_sum(lanes);
}

/* src/kernels/attention.cu:87-98 (block_reduce_sum) as used by the prefill kernels:
 * nthreads = ceil32(head_dim) capped at 256, thread t sums d = t, t+nthreads, ...;
 * per-warp butterfly, then warp 0 butterflies the per-warp totals. */
static float block_strided_dot(const float* q, const float* k, int head_dim) {
    int nthreads = ((head_dim + 31) / 32) * 32;
    if (nthreads > 256) nthreads = 256;
    const int nwarps = nthreads / ORACLE_WARP;
    float warp_tot[ORACLE_WARP];
    for (int w = 0; w < ORACLE_WARP; ++w) warp_tot[w] = 0.0f;
    for (int w = 0; w < nwarps; ++w) {
        float lanes[ORACLE_WARP];
        for (int l = 0; l < ORACLE_WARP; ++l) {
            const int tid = w * ORACLE_WARP + l;
            float partial = 0.0f;
            for (int d = tid; d < head_dim; d += nthreads) partial = fmaf(q[d], k[d], partial);
            lanes[l] = partial;
        }
        warp_tot[w] = butterfly_sum(lanes);
    }
    return butterfly_sum(warp_tot);
}

/* src/kernels/attention.cu:56-58 */
static int kv_head_for_query_head(int query_head, int num_heads, int num_kv_heads) {
    return query_head * num_kv_heads / num_heads;
}

/* ---- store_kvcache --------------------------------------------------------------------- */

void oracle_store_kvcache(const void* key, const void* value, void* k_cache, void* v_cache,
                          const void* slot_mapping, int slot_is_i64, int64_t num_tokens,
                          int64_t row_bytes, int64_t cache_rows) {
    const char* kp = (const char*)key;
    const char* vp = (const char*)value;
    char* kc = (char*)k_cache;
    char* vc = (char*)v_cache;
    for (int64_t token = 0; token < num_tokens; ++token) {
        const int64_t slot = slot_is_i64 ? ((const int64_t*)slot_mapping)[token]
                                         : (int64_t)((const int32_t*)slot_mapping)[token];
        if (slot < 0 || slot >= cache_rows) continue; /* kvcache.cu:33-36 */
        memcpy(kc + slot * row_bytes, kp + token * row_bytes, (size_t)row_bytes);
        memcpy(vc + slot * row_bytes, vp + token * row_bytes, (size_t)row_bytes);
    }
}

/* ---- decode -------------------------------------------------------------------------------- */

void oracle_decode_attention_paged(const float* query, const float* k_cache, const float* v_cache,
                                   const int32_t* context_lens, const int32_t* block_tables,
                                   int64_t batch, int64_t max_blocks, int num_heads,
                                   int num_kv_heads, int head_dim, int block_size, float scale,
                                   float* output, int num_threads) {
    const int64_t total = batch * num_heads;
    (void)num_threads;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1) num_threads(num_threads > 0 ? num_threads : 1)
#endif
    for (int64_t work = 0; work < total; ++work) {
        const int64_t seq = work / num_heads;
        const int head = (int)(work % num_heads);
        const int kv_head = kv_head_for_query_head(head, num_heads, num_kv_heads);
        const float* q = query + (seq * num_heads + head) * head_dim;
        float* out = output + (seq * num_heads + head) * head_dim;
        const int64_t k_len = context_lens[seq];
        if (k_len <= 0) { /* attention.cu:349-355 */
            for (int d = 0; d < head_dim; ++d) out[d] = 0.0f;
            continue;
        }
        float running_max = -INFINITY;
        float running_sum = 0.0f;
        float* v_acc = (float*)calloc((size_t)head_dim, sizeof(float));
        const int32_t* table = block_tables + seq * max_blocks;
        for (int64_t k_index = 0; k_index < k_len; ++k_index) {
            const int64_t block_id = table[k_index / block_size];
            const int64_t cache_row = block_id * block_size + k_index % block_size;
            const float* k_ptr = k_cache + (cache_row * num_kv_heads + kv_head) * head_dim;
            const float* v_ptr = v_cache + (cache_row * num_kv_heads + kv_head) * head_dim;
            const float qk = warp_strided_dot(q, k_ptr, head_dim) * scale;
            const float old_max = running_max;
            running_max = fmaxf(running_max, qk);
            const float correction = expf(old_max - running_max);
            const float exp_qk = expf(qk - running_max);
            running_sum = running_sum * correction + exp_qk;
            for (int d = 0; d < head_dim; ++d) {
                v_acc[d] = v_acc[d] * correction + exp_qk * v_ptr[d];
            }
        }
        {
            const float inv = (running_sum > 0.0f) ? (1.0f / running_sum) : 0.0f;
            for (int d = 0; d < head_dim; ++d) out[d] = v_acc[d] * inv;
        }
        free(v_acc);
    }
}

/* ---- int8 KV cache --------------------------------------------------------------------- */

/* src/kernels/kvcache.cu:222-296 (store_kvcache_int8_kernel): per (token, KV head) the absolute maximum of the head
 * vector gives scale = max(absmax / 127, 1e-10) (stored as fp16) and q = clamp(rint(x * (127 / max(absmax, 1e-10)))). */
void oracle_store_kvcache_int8(const float* key, const float* value, int8_t* k_cache, int8_t* v_cache,
                               float* k_scale, float* v_scale, const int32_t* slot_mapping,
                               int64_t num_tokens, int num_kv_heads, int head_dim, int64_t cache_rows) {
    for (int64_t token = 0; token < num_tokens; ++token) {
        const int64_t slot = slot_mapping[token];
        if (slot < 0 || slot >= cache_rows) continue;
        for (int h = 0; h < num_kv_heads; ++h) {
            for (int which = 0; which < 2; ++which) {
                const float* src = (which ? value : key) + (token * num_kv_heads + h) * head_dim;
                int8_t* dst = (which ? v_cache : k_cache) + (slot * num_kv_heads + h) * head_dim;
                float absmax = 0.0f;
                for (int d = 0; d < head_dim; ++d) {
                    const float a = fabsf(src[d]);
                    if (a > absmax) absmax = a;
                }
                float sc = absmax / 127.0f;
                sc = fmaxf(sc, 1e-10f);
                const float inv_sc = 127.0f / fmaxf(absmax, 1e-10f);
                for (int d = 0; d < head_dim; ++d) {
                    int q = (int)nearbyintf(src[d] * inv_sc);   /* __float2int_rn */
                    if (q > 127) q = 127;
                    if (q < -127) q = -127;
                    dst[d] = (int8_t)q;
                }
                (which ? v_scale : k_scale)[slot * num_kv_heads + h] = oracle_round_fp16(sc);   /* __float2half */
            }
        }
    }
}

/* src/kernels/attention.cu:746-842 (decode_paged_attention_int8_kernel): as the decode kernel above with
 * k = int8 * k_scale and v = int8 * v_scale (scales per cache row and KV head, fp16 widened to float). */
void oracle_decode_attention_paged_int8(const float* query, const int8_t* k_cache, const int8_t* v_cache,
                                        const float* k_scale, const float* v_scale,
                                        const int32_t* context_lens, const int32_t* block_tables,
                                        int64_t batch, int64_t max_blocks, int num_heads, int num_kv_heads,
                                        int head_dim, int block_size, float scale, float* output, int num_threads) {
    const int64_t total = batch * num_heads;
    (void)num_threads;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1) num_threads(num_threads > 0 ? num_threads : 1)
#endif
    for (int64_t work = 0; work < total; ++work) {
        const int64_t seq = work / num_heads;
        const int head = (int)(work % num_heads);
        const int kv_head = kv_head_for_query_head(head, num_heads, num_kv_heads);
        const float* q = query + (seq * num_heads + head) * head_dim;
        float* out = output + (seq * num_heads + head) * head_dim;
        const int64_t k_len = context_lens[seq];
        if (k_len <= 0) {
            for (int d = 0; d < head_dim; ++d) out[d] = 0.0f;
            continue;
        }
        float running_max = -INFINITY;
        float running_sum = 0.0f;
        float* v_acc = (float*)calloc((size_t)head_dim, sizeof(float));
        float* k_row = (float*)malloc((size_t)head_dim * sizeof(float));
        const int32_t* table = block_tables + seq * max_blocks;
        for (int64_t k_index = 0; k_index < k_len; ++k_index) {
            const int64_t block_id = table[k_index / block_size];
            const int64_t cache_row = block_id * block_size + k_index % block_size;
            const float ks = k_scale[cache_row * num_kv_heads + kv_head];
            const float vs = v_scale[cache_row * num_kv_heads + kv_head];
            const int8_t* k_ptr = k_cache + (cache_row * num_kv_heads + kv_head) * head_dim;
            const int8_t* v_ptr = v_cache + (cache_row * num_kv_heads + kv_head) * head_dim;
            for (int d = 0; d < head_dim; ++d) k_row[d] = (float)k_ptr[d] * ks;
            const float qk = warp_strided_dot(q, k_row, head_dim) * scale;
            const float old_max = running_max;
            running_max = fmaxf(running_max, qk);
            const float correction = expf(old_max - running_max);
            const float exp_qk = expf(qk - running_max);
            running_sum = running_sum * correction + exp_qk;
            for (int d = 0; d < head_dim; ++d) {
                const float v_val = (float)v_ptr[d] * vs;
                v_acc[d] = v_acc[d] * correction + exp_qk * v_val;
            }
        }
        {
            const float inv = (running_sum > 0.0f) ? (1.0f / running_sum) : 0.0f;
            for (int d = 0; d < head_dim; ++d) out[d] = v_acc[d] * inv;
        }
        free(k_row);
        free(v_acc);
    }
}

/* ---- prefill ----------------------------------------------------------------------------- */

/* One query row against keys addressed by `row_of_key`; shared by dense and paged prefill. */
static void prefill_row(const float* q, const float* k_base, const float* v_base,
                        int64_t allowed_k, int64_t k_begin, const int32_t* table, int block_size,
                        int num_kv_heads, int kv_head, int head_dim, float scale, float* out) {
    float running_max = -INFINITY;
    float running_sum = 0.0f;
    float* v_acc = (float*)calloc((size_t)head_dim, sizeof(float));
    for (int64_t k_index = 0; k_index < allowed_k; ++k_index) {
        int64_t row;
        if (table != NULL) { /* attention.cu:269-273 */
            row = (int64_t)table[k_index / block_size] * block_size + k_index % block_size;
        } else {             /* attention.cu:172-173 */
            row = k_begin + k_index;
        }
        const float* k_ptr = k_base + (row * num_kv_heads + kv_head) * head_dim;
        const float* v_ptr = v_base + (row * num_kv_heads + kv_head) * head_dim;
        const float qk = block_strided_dot(q, k_ptr, head_dim) * scale;
        const float old_max = running_max;
        running_max = fmaxf(running_max, qk);
        const float exp_correction = expf(old_max - running_max);
        const float exp_qk = expf(qk - running_max);
        running_sum = running_sum * exp_correction + exp_qk;
        for (int d = 0; d < head_dim; ++d) {
            v_acc[d] = v_acc[d] * exp_correction;
            v_acc[d] += exp_qk * v_ptr[d];
        }
    }
    {
        const float inv_sum = (running_sum > 0.0f) ? (1.0f / running_sum) : 0.0f;
        for (int d = 0; d < head_dim; ++d) out[d] = v_acc[d] * inv_sum;
    }
    free(v_acc);
}

void oracle_prefill_attention_dense(const float* query, const float* key, const float* value,
                                    const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                    int64_t num_seqs, int64_t query_rows, int64_t key_rows,
                                    int num_heads, int num_kv_heads, int head_dim, float scale,
                                    float* output, int num_threads) {
    (void)num_threads;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 4) num_threads(num_threads > 0 ? num_threads : 1)
#endif
    for (int64_t q_row = 0; q_row < query_rows; ++q_row) {
        int64_t q_begin, q_end, k_begin, k_end;
        if (cu_seqlens_q == NULL || cu_seqlens_k == NULL || num_seqs <= 0) { /* attention.cu:37-43 */
            q_begin = 0; q_end = query_rows; k_begin = 0; k_end = key_rows;
        } else {                                                            /* attention.cu:45-53 */
            int64_t seq = 0;
            while (seq + 1 < num_seqs && q_row >= cu_seqlens_q[seq + 1]) ++seq;
            q_begin = cu_seqlens_q[seq]; q_end = cu_seqlens_q[seq + 1];
            k_begin = cu_seqlens_k[seq]; k_end = cu_seqlens_k[seq + 1];
        }
        const int64_t allowed_k = (k_end - k_begin) - (q_end - q_begin) + (q_row - q_begin) + 1;
        for (int head = 0; head < num_heads; ++head) {
            float* out = output + (q_row * num_heads + head) * head_dim;
            if (allowed_k <= 0) { /* attention.cu:153-158 */
                for (int d = 0; d < head_dim; ++d) out[d] = 0.0f;
                continue;
            }
            const int kv_head = kv_head_for_query_head(head, num_heads, num_kv_heads);
            prefill_row(query + (q_row * num_heads + head) * head_dim, key, value, allowed_k,
                        k_begin, NULL, 1, num_kv_heads, kv_head, head_dim, scale, out);
        }
    }
}

void oracle_prefill_attention_paged(const float* query, const float* k_cache, const float* v_cache,
                                    const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                    const int32_t* block_tables, int64_t num_seqs,
                                    int64_t query_rows, int64_t max_blocks, int num_heads,
                                    int num_kv_heads, int head_dim, int block_size, float scale,
                                    float* output, int num_threads) {
    (void)num_threads;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 4) num_threads(num_threads > 0 ? num_threads : 1)
#endif
    for (int64_t q_row = 0; q_row < query_rows; ++q_row) {
        int64_t seq = 0; /* attention.cu:231-243 */
        while (seq + 1 < num_seqs && q_row >= cu_seqlens_q[seq + 1]) ++seq;
        const int64_t qb = cu_seqlens_q[seq], qe = cu_seqlens_q[seq + 1];
        const int64_t kb = cu_seqlens_k[seq], ke = cu_seqlens_k[seq + 1];
        const int64_t allowed_k = (ke - kb) - (qe - qb) + (q_row - qb) + 1;
        for (int head = 0; head < num_heads; ++head) {
            float* out = output + (q_row * num_heads + head) * head_dim;
            if (allowed_k <= 0) {
                for (int d = 0; d < head_dim; ++d) out[d] = 0.0f;
                continue;
            }
            const int kv_head = kv_head_for_query_head(head, num_heads, num_kv_heads);
            prefill_row(query + (q_row * num_heads + head) * head_dim, k_cache, v_cache, allowed_k,
                        0, block_tables + seq * max_blocks, block_size, num_kv_heads, kv_head,
                        head_dim, scale, out);
        }
    }
}

/* ---- fused decode prologue --------------------------------------------------------------- */

void oracle_build_cos_sin_cache(float* table, int max_position, int rotary_dim, float base) {
    const int half_dim = rotary_dim / 2;
    for (int position = 0; position < max_position; ++position) {
        for (int idx = 0; idx < half_dim; ++idx) {
            const float exponent = (float)(2 * idx) / (float)rotary_dim;
            const float inv_freq = 1.0f / powf(base, exponent);
            const float angle = (float)position * inv_freq;
            table[(size_t)position * rotary_dim + idx] = cosf(angle);
            table[(size_t)position * rotary_dim + idx + half_dim] = sinf(angle);
        }
    }
}

/* include/kernels/device_helpers.cuh:65-87 (block_reduce_sum) for blockDim = head_dim. */
static float block_sum_of_squares(const float* x, int head_dim) {
    const int nwarps = (head_dim + ORACLE_WARP - 1) / ORACLE_WARP;
    float warp_tot[ORACLE_WARP];
    for (int w = 0; w < ORACLE_WARP; ++w) warp_tot[w] = 0.0f;
    for (int w = 0; w < nwarps && w < ORACLE_WARP; ++w) {
        float lanes[ORACLE_WARP];
        for (int l = 0; l < ORACLE_WARP; ++l) {
            const int d = w * ORACLE_WARP + l;
            lanes[l] = (d < head_dim) ? x[d] * x[d] : 0.0f;
        }
        warp_tot[w] = butterfly_sum(lanes);
    }
    return butterfly_sum(warp_tot);
}

void oracle_fused_split_norm_rope_store(const float* qkv, const int32_t* positions,
                                        const float* q_norm_weight, const float* k_norm_weight,
                                        float norm_eps, const float* cos_sin_cache,
                                        int max_positions, const int32_t* slot_mapping,
                                        float* k_cache, float* v_cache, int64_t rows,
                                        int num_q_heads, int num_kv_heads, int head_dim,
                                        float* q_out, int round_mode) {
    const int q_size = num_q_heads * head_dim;
    const int kv_size = num_kv_heads * head_dim;
    const int total_cols = q_size + 2 * kv_size;
    const int total_heads = num_q_heads + 2 * num_kv_heads;
    const int half_dim = head_dim / 2;
    float* normed = (float*)malloc(sizeof(float) * (size_t)head_dim);
    float* rotated = (float*)malloc(sizeof(float) * (size_t)head_dim);
    for (int64_t row = 0; row < rows; ++row) {
        for (int head_idx = 0; head_idx < total_heads; ++head_idx) {
            const int is_q = head_idx < num_q_heads;
            const int is_k = !is_q && head_idx < num_q_heads + num_kv_heads;
            int src_head, src_offset;
            if (is_q) { src_head = head_idx; src_offset = src_head * head_dim; }
            else if (is_k) { src_head = head_idx - num_q_heads; src_offset = q_size + src_head * head_dim; }
            else { src_head = head_idx - num_q_heads - num_kv_heads; src_offset = q_size + kv_size + src_head * head_dim; }
            const float* src = qkv + row * total_cols + src_offset;
            for (int d = 0; d < head_dim; ++d) rotated[d] = src[d];
            if (is_q || is_k) {
                /* split_qkv.cu:113-119 */
                const float sum_sq = block_sum_of_squares(src, head_dim);
                const float inv_rms = 1.0f / sqrtf(sum_sq / (float)head_dim + norm_eps);
                const float* weight = is_q ? q_norm_weight : k_norm_weight;
                for (int d = 0; d < head_dim; ++d) normed[d] = src[d] * inv_rms * weight[d];
                for (int d = 0; d < head_dim; ++d) rotated[d] = normed[d];
                /* split_qkv.cu:121-140 */
                const int pos = positions[row];
                if (pos >= 0 && pos < max_positions) {
                    const float* cache_row = cos_sin_cache + (size_t)pos * head_dim;
                    for (int d = 0; d < head_dim; ++d) {
                        const int cos_idx = (d < half_dim) ? d : (d - half_dim);
                        const float cos_v = cache_row[cos_idx];
                        const float sin_v = cache_row[cos_idx + half_dim];
                        if (d < half_dim) rotated[d] = normed[d] * cos_v - normed[d + half_dim] * sin_v;
                        else rotated[d] = normed[d] * cos_v + normed[d - half_dim] * sin_v;
                    }
                }
            }
            if (is_q) {
                float* dst = q_out + row * (int64_t)q_size + src_head * head_dim;
                for (int d = 0; d < head_dim; ++d) dst[d] = round_store(rotated[d], round_mode);
            } else {
                const int slot = slot_mapping[row];
                if (slot >= 0) { /* split_qkv.cu:147-153 -- only the lower bound is checked */
                    float* cache = is_k ? k_cache : v_cache;
                    float* dst = cache + (int64_t)slot * kv_size + src_head * head_dim;
                    for (int d = 0; d < head_dim; ++d) dst[d] = round_store(rotated[d], round_mode);
                }
            }
        }
    }
    free(normed);
    free(rotated);
}

/* ---- fp8 (e4m3) KV cache ---------------------------------------------------------------
 * The reference has no fp8 cache (its survey of next steps names one after the int8 cache); the format here follows its
 * int8 cache (src/kernels/kvcache.cu:222-296, src/kernels/attention.cu:746-842) with the value range of the type:
 * one fp16 scale per (cache row, KV head) = max(absmax / 448, 1e-10), elements = e4m3(x * 448 / max(absmax, 1e-10)),
 * round to nearest even, saturating at +-448.  No reference output exists for it: parity for this format is this
 * restatement against the CUDA kernels, and the decode against the 16-bit cache. */
static uint8_t e4m3_from_float(float x) {
    if (x != x) return 0x7f;
    const uint8_t sign = signbit(x) ? 0x80 : 0x00;
    const float a = fabsf(x);
    if (a >= 448.0f) return sign | 0x7e;
    if (a < 0.015625f) return sign | (uint8_t)rintf(a * 512.0f);        /* subnormals: units of 2^-9; 8 = the smallest normal */
    int ex;
    (void)frexpf(a, &ex);                                               /* a = f * 2^ex, f in [0.5, 1) */
    int e = ex - 1;
    int m = (int)rintf((ldexpf(a, -e) - 1.0f) * 8.0f);                  /* exact before the rint */
    if (m == 8) { m = 0; ++e; }
    if (e > 8 || (e == 8 && m > 6)) return sign | 0x7e;
    return sign | (uint8_t)(((e + 7) << 3) | m);
}
static float e4m3_to_float(uint8_t v) {
    const int e = (v >> 3) & 15, m = v & 7;
    float a;
    if (e == 15 && m == 7) return NAN;
    if (e == 0) a = ldexpf((float)m, -9);
    else a = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return (v & 0x80) ? -a : a;
}

void oracle_store_kvcache_fp8(const float* key, const float* value, uint8_t* k_cache, uint8_t* v_cache,
                              float* k_scale, float* v_scale, const int32_t* slot_mapping, int64_t num_tokens,
                              int num_kv_heads, int head_dim, int64_t cache_rows) {
    for (int64_t token = 0; token < num_tokens; ++token) {
        const int64_t slot = slot_mapping[token];
        if (slot < 0 || slot >= cache_rows) continue;
        for (int which = 0; which < 2; ++which) {
            for (int h = 0; h < num_kv_heads; ++h) {
                const float* src = (which ? value : key) + (token * num_kv_heads + h) * head_dim;
                uint8_t* dst = (which ? v_cache : k_cache) + (slot * num_kv_heads + h) * head_dim;
                float absmax = 0.0f;
                for (int d = 0; d < head_dim; ++d) absmax = fmaxf(absmax, fabsf(src[d]));
                const float scale = fmaxf(absmax / 448.0f, 1.0e-10f);
                const float inv_scale = 448.0f / fmaxf(absmax, 1.0e-10f);
                for (int d = 0; d < head_dim; ++d) dst[d] = e4m3_from_float(src[d] * inv_scale);
                (which ? v_scale : k_scale)[slot * num_kv_heads + h] = oracle_round_fp16(scale);
            }
        }
    }
}

void oracle_decode_attention_paged_fp8(const float* query, const uint8_t* k_cache, const uint8_t* v_cache,
                                       const float* k_scale, const float* v_scale, const int32_t* context_lens,
                                       const int32_t* block_tables, int64_t batch, int64_t max_blocks, int num_heads,
                                       int num_kv_heads, int head_dim, int block_size, float scale, float* output) {
    for (int64_t seq = 0; seq < batch; ++seq) {
        for (int head = 0; head < num_heads; ++head) {
            float* out = output + (seq * num_heads + head) * head_dim;
            const int32_t k_len = context_lens[seq];
            if (k_len <= 0) { for (int d = 0; d < head_dim; ++d) out[d] = 0.0f; continue; }
            const int kv_head = head * num_kv_heads / num_heads;
            const float* q = query + (seq * num_heads + head) * head_dim;
            float running_max = -INFINITY, running_sum = 0.0f;
            for (int d = 0; d < head_dim; ++d) out[d] = 0.0f;
            for (int32_t k = 0; k < k_len; ++k) {
                const int64_t block = block_tables[seq * max_blocks + k / block_size];
                const int64_t row = (block * block_size + k % block_size) * num_kv_heads + kv_head;
                const uint8_t* k_ptr = k_cache + row * head_dim;
                const uint8_t* v_ptr = v_cache + row * head_dim;
                float dot = 0.0f;
                for (int d = 0; d < head_dim; ++d) dot += q[d] * (e4m3_to_float(k_ptr[d]) * k_scale[row]);
                const float qk = dot * scale;
                const float old_max = running_max;
                running_max = fmaxf(running_max, qk);
                const float correction = expf(old_max - running_max);
                const float e = expf(qk - running_max);
                running_sum = running_sum * correction + e;
                for (int d = 0; d < head_dim; ++d) out[d] = out[d] * correction + e * (e4m3_to_float(v_ptr[d]) * v_scale[row]);
            }
            const float inv = running_sum > 0.0f ? 1.0f / running_sum : 0.0f;
            for (int d = 0; d < head_dim; ++d) out[d] *= inv;
        }
    }
}
