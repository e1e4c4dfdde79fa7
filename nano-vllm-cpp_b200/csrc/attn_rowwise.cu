// General SIMT attention: one warp per (query row, query head), any of F16 / BF16 / F32,
// head_dim <= 256, any block size, dense or paged keys, decode or bottom-right causal prefill.
//
// This is the shape-agnostic path behind nvk_decode_attention_paged and
// nvk_prefill_attention_varlen for inputs the tensor-core kernels do not take (fp32 models,
// the tiny shapes of the reference's own known-answer tests, odd head sizes).  It computes what
// src/kernels/attention.cu:114-405 of the reference computes -- fp32 accumulation, natural
// exponent, online softmax over keys in order -- with one code path instead of three kernels:
// the per-row key range and addressing mode are resolved up front, and four keys are scored
// per trip so that their warp reductions overlap.
#include "nvk_internal.cuh"

#include <cmath>

namespace nvk {
namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxPerLane = 8;   // head_dim <= 256
constexpr int kKeysPerTrip = 4;

struct RowwiseParams {
    const void* q; const void* k; const void* v; void* out;
    IndexArray cu_q, cu_k;                         // prefill (may be null: one sequence)
    IndexArray context_lens;                       // decode
    IndexArray block_tables;                       // null = dense keys
    int64_t num_rows, num_seqs, total_k, max_blocks, cache_rows;
    int num_heads, num_kv_heads, head_dim, block_size;
    float scale;
    int is_decode;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) attn_rowwise_kernel(RowwiseParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t work = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    if (work >= p.num_rows * p.num_heads) return;
    const int64_t row = work / p.num_heads;
    const int head = static_cast<int>(work - row * p.num_heads);
    const int kv_head = head * p.num_kv_heads / p.num_heads;
    const int per_lane = (p.head_dim + 31) / 32;

    // Resolve the key range of this row.
    int64_t seq = 0, allowed = 0, k_begin = 0;
    if (p.is_decode) {
        seq = row;
        allowed = p.context_lens[row];
    } else if (p.cu_q == nullptr || p.cu_k == nullptr) {
        allowed = (p.total_k - p.num_rows) + row + 1;
    } else {
        int64_t lo = 0, hi = p.num_seqs - 1;  // last seq with cu_q[seq] <= row, skipping empty ones
        while (lo < hi) {
            const int64_t mid = (lo + hi + 1) >> 1;
            if (p.cu_q[mid] <= row) lo = mid; else hi = mid - 1;
        }
        seq = lo;
        const int64_t qb = p.cu_q[seq], qe = p.cu_q[seq + 1];
        const int64_t kb = p.cu_k[seq], ke = p.cu_k[seq + 1];
        k_begin = kb;
        allowed = (ke - kb) - (qe - qb) + (row - qb) + 1;
    }

    T* out = static_cast<T*>(p.out) + (row * p.num_heads + head) * p.head_dim;
    if (allowed <= 0) {
        for (int d = lane; d < p.head_dim; d += 32) out[d] = ElemTraits<T>::from_float(0.0f);
        return;
    }

    const T* q = static_cast<const T*>(p.q) + (row * p.num_heads + head) * p.head_dim;
    float qr[kMaxPerLane], acc[kMaxPerLane];
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int d = lane + 32 * i;
        qr[i] = (i < per_lane && d < p.head_dim) ? ElemTraits<T>::to_float(q[d]) * p.scale : 0.0f;
        acc[i] = 0.0f;
    }
    const T* kbase = static_cast<const T*>(p.k);
    const T* vbase = static_cast<const T*>(p.v);
    const IndexArray table = p.block_tables ? p.block_tables + seq * p.max_blocks : IndexArray();
    const int64_t row_stride = static_cast<int64_t>(p.num_kv_heads) * p.head_dim;
    const int64_t head_off = static_cast<int64_t>(kv_head) * p.head_dim;

    float m = -INFINITY, l = 0.0f;
    for (int64_t k0 = 0; k0 < allowed; k0 += kKeysPerTrip) {
        int64_t src_row[kKeysPerTrip];
        float s[kKeysPerTrip];
#pragma unroll
        for (int j = 0; j < kKeysPerTrip; ++j) {
            const int64_t k = k0 + j;
            src_row[j] = -1;
            if (k < allowed) {
                int64_t r;
                if (table) {
                    const int64_t blk = table[k / p.block_size];
                    r = blk * p.block_size + k % p.block_size;
                } else {
                    r = k_begin + k;
                }
                if (r >= 0 && r < p.cache_rows) src_row[j] = r;
            }
            float part = 0.0f;
            if (src_row[j] >= 0) {
                const T* kp = kbase + src_row[j] * row_stride + head_off;
#pragma unroll
                for (int i = 0; i < kMaxPerLane; ++i) {
                    const int d = lane + 32 * i;
                    if (i < per_lane && d < p.head_dim) part = fmaf(qr[i], ElemTraits<T>::to_float(kp[d]), part);
                }
            }
            s[j] = part;
        }
#pragma unroll
        for (int j = 0; j < kKeysPerTrip; ++j) s[j] = warp_sum(s[j]);
        float m_new = m;
#pragma unroll
        for (int j = 0; j < kKeysPerTrip; ++j) {
            if (k0 + j < allowed) m_new = fmaxf(m_new, s[j]);
        }
        const float corr = expf(m - m_new);
        float pj[kKeysPerTrip];
        float psum = 0.0f;
#pragma unroll
        for (int j = 0; j < kKeysPerTrip; ++j) {
            pj[j] = (k0 + j < allowed) ? expf(s[j] - m_new) : 0.0f;
            psum += pj[j];
        }
        l = l * corr + psum;
        m = m_new;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) acc[i] *= corr;
#pragma unroll
        for (int j = 0; j < kKeysPerTrip; ++j) {
            if (src_row[j] >= 0) {
                const T* vp = vbase + src_row[j] * row_stride + head_off;
#pragma unroll
                for (int i = 0; i < kMaxPerLane; ++i) {
                    const int d = lane + 32 * i;
                    if (i < per_lane && d < p.head_dim) acc[i] = fmaf(pj[j], ElemTraits<T>::to_float(vp[d]), acc[i]);
                }
            }
        }
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int d = lane + 32 * i;
        if (i < per_lane && d < p.head_dim) out[d] = ElemTraits<T>::from_float(acc[i] * inv);
    }
}

int launch(const RowwiseParams& p, int dtype, cudaStream_t stream) {
    if (p.head_dim > 32 * kMaxPerLane) return fail(NVK_ERR_UNSUPPORTED, "attention: head_dim %d > 256 is unsupported", p.head_dim);
    const int64_t work = p.num_rows * p.num_heads;
    if (work <= 0) return NVK_OK;
    const int64_t blocks = (work + kWarpsPerBlock - 1) / kWarpsPerBlock;
    if (blocks > 0x7fffffffLL) return fail(NVK_ERR_INVALID_ARGUMENT, "attention: too many rows");
    const dim3 grid(static_cast<unsigned>(blocks));
    switch (dtype) {
        case NVK_F32: attn_rowwise_kernel<float><<<grid, kWarpsPerBlock * 32, 0, stream>>>(p); break;
        case NVK_F16: attn_rowwise_kernel<__half><<<grid, kWarpsPerBlock * 32, 0, stream>>>(p); break;
        case NVK_BF16: attn_rowwise_kernel<__nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, stream>>>(p); break;
        default: return fail(NVK_ERR_INVALID_ARGUMENT, "attention: query must be float16, bfloat16 or float32");
    }
    return check_launch("attn_rowwise_kernel launch");
}

}  // namespace

int launch_rowwise_decode(const DecodeArgs& a) {
    RowwiseParams p{};
    p.q = a.q; p.k = a.k_cache; p.v = a.v_cache; p.out = a.out;
    p.context_lens = a.context_lens; p.block_tables = a.block_tables;
    p.num_rows = a.batch; p.num_seqs = a.batch; p.max_blocks = a.max_blocks;
    p.cache_rows = a.num_cache_blocks * a.block_size;
    p.num_heads = a.num_heads; p.num_kv_heads = a.num_kv_heads; p.head_dim = a.head_dim;
    p.block_size = a.block_size; p.scale = a.scale; p.is_decode = 1;
    return launch(p, a.dtype, a.stream);
}

int launch_rowwise_prefill(const PrefillArgs& a) {
    RowwiseParams p{};
    p.q = a.q; p.out = a.out; p.cu_q = a.cu_q; p.cu_k = a.cu_k;
    p.num_rows = a.total_q; p.num_seqs = a.num_seqs; p.total_k = a.total_k;
    p.num_heads = a.num_heads; p.num_kv_heads = a.num_kv_heads; p.head_dim = a.head_dim;
    p.scale = a.scale; p.is_decode = 0;
    if (a.block_tables != nullptr) {
        p.k = a.k_cache; p.v = a.v_cache; p.block_tables = a.block_tables;
        p.max_blocks = a.max_blocks; p.block_size = a.block_size;
        p.cache_rows = a.num_cache_blocks * a.block_size;
    } else {
        p.k = a.k; p.v = a.v; p.block_size = 1; p.cache_rows = a.total_k;
    }
    return launch(p, a.dtype, a.stream);
}

}  // namespace nvk
