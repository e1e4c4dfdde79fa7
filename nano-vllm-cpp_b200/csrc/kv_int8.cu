// int8 paged KV cache for sm_100a: quantising store and the general decode path.
//
// Replaces store_kvcache_int8_kernel (src/kernels/kvcache.cu:222-296 of the reference: one 32-thread block per
// (token, KV head), lane-strided element loops) and, for shapes the tensor-core kernel in decode_attn.cu does not
// take, decode_paged_attention_int8_kernel (src/kernels/attention.cu:746-842).
//
// Format (the reference's): K and V as int8 [cache_rows, Hkv, D]; one fp16 scale per (cache row, KV head) in
// k_scale / v_scale [cache_rows, Hkv]; scale = max(absmax / 127, 1e-10), q = clamp(rint(x * 127 / max(absmax, 1e-10)), +-127).
// The store is HBM-bound (reads 2 * tokens * Hkv * D elements, writes half as many bytes plus the scales): a head
// vector is spread over head_dim / 8 lanes (16-byte loads of K and of V per lane, two vectors per warp at head_dim 128), the
// absolute maximum is a shuffle reduction inside that lane group, the quantised bytes leave as one packed store per lane.  The arithmetic is
// the reference's operation for operation (IEEE division, round-to-nearest-even conversion), so caches and scales are
// bit-identical to the reference's.
#include "nvk_internal.cuh"

#include <cuda_fp16.h>

namespace nvk {
namespace {

constexpr int kStoreWarps = 8;

template <int V> struct PackOf;
template <> struct PackOf<2> { using in16 = uint32_t; using in32 = uint2; using out = uint16_t; };
template <> struct PackOf<4> { using in16 = uint2; using in32 = uint4; using out = uint32_t; };
template <> struct PackOf<8> { using in16 = uint4; using in32 = uint4; using out = uint2; };

template <typename T, int V>
__device__ __forceinline__ void load_elems(const T* src, float (&x)[V]) {
    if constexpr (sizeof(T) == 2) {
        union { typename PackOf<V>::in16 v; T e[V]; } u;
        u.v = *reinterpret_cast<const typename PackOf<V>::in16*>(src);
#pragma unroll
        for (int i = 0; i < V; ++i) x[i] = ElemTraits<T>::to_float(u.e[i]);
    } else {
#pragma unroll
        for (int i = 0; i < V; ++i) x[i] = src[i];
    }
}

// One warp quantises 32 / LANES (token, KV head) vectors at a time: 16-bit inputs are read as 16-byte pieces (V = 8,
// LANES = head_dim / 8), fp32 inputs as V = 4.
template <typename T, int V, int LANES>
__global__ void __launch_bounds__(kStoreWarps * 32)
store_int8_kernel(const T* __restrict__ key, const T* __restrict__ value, int8_t* __restrict__ k_cache,
                  int8_t* __restrict__ v_cache, __half* __restrict__ k_scale, __half* __restrict__ v_scale,
                  const int32_t* __restrict__ slot_mapping, int64_t num_tokens, int num_kv_heads, int64_t cache_rows) {
    constexpr int D = V * LANES;
    constexpr int kPerWarp = 32 / LANES;
    const int lane = threadIdx.x & 31;
    const int sub = lane % LANES;
    const int64_t total = num_tokens * num_kv_heads;
    int64_t work = (static_cast<int64_t>(blockIdx.x) * kStoreWarps + (threadIdx.x >> 5)) * kPerWarp + lane / LANES;   // (token, head)
    // lanes past the end repeat the last vector (same values, same destination) so that the shuffles stay full-warp
    if (work >= total) work = total - 1;
    const int64_t token = work / num_kv_heads;
    const int head = static_cast<int>(work % num_kv_heads);
    const int64_t slot = slot_mapping[token];
    const bool live = slot >= 0 && slot < cache_rows;
    float kx[V], vx[V];
    load_elems<T, V>(key + work * D + sub * V, kx);
    load_elems<T, V>(value + work * D + sub * V, vx);
    const int64_t dst_row = (live ? slot : 0) * num_kv_heads + head;
    // the reductions run for every lane; only live vectors are written
    float kmax = 0.0f, vmax = 0.0f;
#pragma unroll
    for (int i = 0; i < V; ++i) { kmax = fmaxf(kmax, fabsf(kx[i])); vmax = fmaxf(vmax, fabsf(vx[i])); }
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) {
        kmax = fmaxf(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
        vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
    }
    if (!live) return;
    const float k_sc = fmaxf(__fdiv_rn(kmax, 127.0f), 1e-10f), k_inv = __fdiv_rn(127.0f, fmaxf(kmax, 1e-10f));
    const float v_sc = fmaxf(__fdiv_rn(vmax, 127.0f), 1e-10f), v_inv = __fdiv_rn(127.0f, fmaxf(vmax, 1e-10f));
    union { typename PackOf<V>::out v; int8_t e[V]; } kq, vq;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        kq.e[i] = static_cast<int8_t>(max(-127, min(127, __float2int_rn(__fmul_rn(kx[i], k_inv)))));
        vq.e[i] = static_cast<int8_t>(max(-127, min(127, __float2int_rn(__fmul_rn(vx[i], v_inv)))));
    }
    *reinterpret_cast<typename PackOf<V>::out*>(k_cache + dst_row * D + sub * V) = kq.v;
    *reinterpret_cast<typename PackOf<V>::out*>(v_cache + dst_row * D + sub * V) = vq.v;
    if (sub == 0) { k_scale[dst_row] = __float2half(k_sc); v_scale[dst_row] = __float2half(v_sc); }
}

// ---- 16-bit inputs: the same arithmetic in about half the instructions (the kernel above is bound by issue slots, not
// by HBM).  Absolute maxima are taken on packed pairs in the 16-bit type (abs and max do not round, and max drops NaNs
// as fmaxf does), K's and V's maxima travel through the shuffles as one packed register, the IEEE divisions run once
// per lane for the two inverse scales and once for the scale the lane may store, products are converted with one F2I
// each and packed with saturating byte packs (|x * inv| <= 127.00002, so the +-127 clamp of the reference cannot
// bind), and the (token, head) split is 32-bit arithmetic.
template <typename T> struct Pair16;
template <> struct Pair16<__nv_bfloat16> {
    using type = __nv_bfloat162;
    static __device__ __forceinline__ float lo(uint32_t w) { return __uint_as_float(w << 16); }
    static __device__ __forceinline__ float hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
    static __device__ __forceinline__ float first(type v) { return __bfloat162float(v.x); }
    static __device__ __forceinline__ float second(type v) { return __bfloat162float(v.y); }
    static __device__ __forceinline__ type join(type a, type b) { return __halves2bfloat162(a.x, b.x); }
};
template <> struct Pair16<__half> {
    using type = __half2;
    static __device__ __forceinline__ float lo(uint32_t w) { return __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xffffu))); }
    static __device__ __forceinline__ float hi(uint32_t w) { return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16))); }
    static __device__ __forceinline__ float first(type v) { return __half2float(v.x); }
    static __device__ __forceinline__ float second(type v) { return __half2float(v.y); }
    static __device__ __forceinline__ type join(type a, type b) { return __halves2half2(a.x, b.x); }
};

// maximum of |x| over the eight elements of a 16-byte piece (in the low half of the result)
template <typename T>
__device__ __forceinline__ typename Pair16<T>::type absmax8(const uint4& v) {
    using P = typename Pair16<T>::type;
    const P a = __habs2(*reinterpret_cast<const P*>(&v.x)), b = __habs2(*reinterpret_cast<const P*>(&v.y));
    const P c = __habs2(*reinterpret_cast<const P*>(&v.z)), d = __habs2(*reinterpret_cast<const P*>(&v.w));
    const P m = __hmax2(__hmax2(a, b), __hmax2(c, d));
    return __hmax2(m, __lowhigh2highlow(m));
}

// bytes {e0, e1, e2, e3} (e0 lowest) of four integers, each saturated to int8
__device__ __forceinline__ uint32_t pack_s8x4(int e0, int e1, int e2, int e3) {
    uint32_t hi, out;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;\n" : "=r"(hi) : "r"(e3), "r"(e2), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;\n" : "=r"(out) : "r"(e1), "r"(e0), "r"(hi));
    return out;
}

template <typename T>
__device__ __forceinline__ uint2 quantise8(const uint4& v, float inv) {
    using P = Pair16<T>;
    uint2 q;
    q.x = pack_s8x4(__float2int_rn(__fmul_rn(P::lo(v.x), inv)), __float2int_rn(__fmul_rn(P::hi(v.x), inv)),
                    __float2int_rn(__fmul_rn(P::lo(v.y), inv)), __float2int_rn(__fmul_rn(P::hi(v.y), inv)));
    q.y = pack_s8x4(__float2int_rn(__fmul_rn(P::lo(v.z), inv)), __float2int_rn(__fmul_rn(P::hi(v.z), inv)),
                    __float2int_rn(__fmul_rn(P::lo(v.w), inv)), __float2int_rn(__fmul_rn(P::hi(v.w), inv)));
    return q;
}

template <typename T, int LANES>
__global__ void __launch_bounds__(kStoreWarps * 32)
store_int8_packed_kernel(const T* __restrict__ key, const T* __restrict__ value, int8_t* __restrict__ k_cache,
                         int8_t* __restrict__ v_cache, __half* __restrict__ k_scale, __half* __restrict__ v_scale,
                         const int32_t* __restrict__ slot_mapping, uint32_t total, uint32_t num_kv_heads, int64_t cache_rows) {
    using P = typename Pair16<T>::type;
    constexpr int D = 8 * LANES;
    constexpr int kPerWarp = 32 / LANES;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t sub = lane % LANES;
    uint32_t work = (blockIdx.x * kStoreWarps + (threadIdx.x >> 5)) * kPerWarp + lane / LANES;   // (token, head)
    if (work >= total) work = total - 1;   // lanes past the end repeat the last vector: the shuffles stay full-warp
    const uint32_t token = work / num_kv_heads;
    const uint32_t head = work - token * num_kv_heads;
    const size_t src = static_cast<size_t>(work) * D + sub * 8;
    const uint4 kv = __ldcs(reinterpret_cast<const uint4*>(key + src));
    const uint4 vv = __ldcs(reinterpret_cast<const uint4*>(value + src));
    const int64_t slot = slot_mapping[token];
    P m = Pair16<T>::join(absmax8<T>(kv), absmax8<T>(vv));   // K's maximum in the low half, V's in the high half
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) {
        const uint32_t other = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<const uint32_t*>(&m), o);
        m = __hmax2(m, *reinterpret_cast<const P*>(&other));
    }
    if (slot < 0 || slot >= cache_rows) return;
    const float kmax = Pair16<T>::first(m), vmax = Pair16<T>::second(m);
    const float k_inv = __fdiv_rn(127.0f, fmaxf(kmax, 1e-10f)), v_inv = __fdiv_rn(127.0f, fmaxf(vmax, 1e-10f));
    const size_t dst_row = static_cast<size_t>(slot) * num_kv_heads + head;
    *reinterpret_cast<uint2*>(k_cache + dst_row * D + sub * 8) = quantise8<T>(kv, k_inv);
    *reinterpret_cast<uint2*>(v_cache + dst_row * D + sub * 8) = quantise8<T>(vv, v_inv);
    if (sub < 2) {   // lane 0 of the group stores K's scale, lane 1 V's
        const float sc = fmaxf(__fdiv_rn(sub == 0 ? kmax : vmax, 127.0f), 1e-10f);
        (sub == 0 ? k_scale : v_scale)[dst_row] = __float2half(sc);
    }
}

// ---- fp8 (e4m3) cache: the packed kernel with the other element type.  No counterpart in the reference; the format follows
// its int8 cache: one fp16 scale per (cache row, KV head) = max(absmax / 448, 1e-10), elements = e4m3(x * 448 / max(absmax,
// 1e-10)) rounded to nearest even from the fp32 product, saturating at +-448.
__device__ __forceinline__ uint32_t pack_e4m3x4(float e0, float e1, float e2, float e3) {   // bytes {e0, e1, e2, e3}, e0 lowest
    unsigned short lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(lo) : "f"(e1), "f"(e0));   // first source -> upper byte
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(hi) : "f"(e3), "f"(e2));
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}
template <typename T>
__device__ __forceinline__ uint2 quantise8_e4m3(const uint4& v, float inv) {
    using P = Pair16<T>;
    uint2 q;
    q.x = pack_e4m3x4(__fmul_rn(P::lo(v.x), inv), __fmul_rn(P::hi(v.x), inv), __fmul_rn(P::lo(v.y), inv), __fmul_rn(P::hi(v.y), inv));
    q.y = pack_e4m3x4(__fmul_rn(P::lo(v.z), inv), __fmul_rn(P::hi(v.z), inv), __fmul_rn(P::lo(v.w), inv), __fmul_rn(P::hi(v.w), inv));
    return q;
}

template <typename T, int LANES>
__global__ void __launch_bounds__(kStoreWarps * 32)
store_fp8_packed_kernel(const T* __restrict__ key, const T* __restrict__ value, uint8_t* __restrict__ k_cache,
                        uint8_t* __restrict__ v_cache, __half* __restrict__ k_scale, __half* __restrict__ v_scale,
                        const int32_t* __restrict__ slot_mapping, uint32_t total, uint32_t num_kv_heads, int64_t cache_rows) {
    using P = typename Pair16<T>::type;
    constexpr int D = 8 * LANES;
    constexpr int kPerWarp = 32 / LANES;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t sub = lane % LANES;
    uint32_t work = (blockIdx.x * kStoreWarps + (threadIdx.x >> 5)) * kPerWarp + lane / LANES;   // (token, head)
    if (work >= total) work = total - 1;   // lanes past the end repeat the last vector: the shuffles stay full-warp
    const uint32_t token = work / num_kv_heads;
    const uint32_t head = work - token * num_kv_heads;
    const size_t src = static_cast<size_t>(work) * D + sub * 8;
    const uint4 kv = __ldcs(reinterpret_cast<const uint4*>(key + src));
    const uint4 vv = __ldcs(reinterpret_cast<const uint4*>(value + src));
    const int64_t slot = slot_mapping[token];
    P m = Pair16<T>::join(absmax8<T>(kv), absmax8<T>(vv));   // K's maximum in the low half, V's in the high half
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) {
        const uint32_t other = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<const uint32_t*>(&m), o);
        m = __hmax2(m, *reinterpret_cast<const P*>(&other));
    }
    if (slot < 0 || slot >= cache_rows) return;
    const float kmax = Pair16<T>::first(m), vmax = Pair16<T>::second(m);
    const float k_inv = __fdiv_rn(448.0f, fmaxf(kmax, 1e-10f)), v_inv = __fdiv_rn(448.0f, fmaxf(vmax, 1e-10f));
    const size_t dst_row = static_cast<size_t>(slot) * num_kv_heads + head;
    *reinterpret_cast<uint2*>(k_cache + dst_row * D + sub * 8) = quantise8_e4m3<T>(kv, k_inv);
    *reinterpret_cast<uint2*>(v_cache + dst_row * D + sub * 8) = quantise8_e4m3<T>(vv, v_inv);
    if (sub < 2) {   // lane 0 of the group stores K's scale, lane 1 V's
        const float sc = fmaxf(__fdiv_rn(sub == 0 ? kmax : vmax, 448.0f), 1e-10f);
        (sub == 0 ? k_scale : v_scale)[dst_row] = __float2half(sc);
    }
}

template <typename T>
int launch_store_fp8_typed(const void* key, const void* value, void* k_cache, void* v_cache, void* k_scale, void* v_scale,
                           const int32_t* slot_mapping, int64_t num_tokens, int num_kv_heads, int head_dim, int64_t cache_rows,
                           cudaStream_t stream) {
    const int lanes = head_dim / 8;
    if (head_dim % 8 != 0 || (lanes != 8 && lanes != 16 && lanes != 32))
        return fail(NVK_ERR_UNSUPPORTED, "store_kvcache_fp8: head_dim must be 64, 128 or 256 (got %d)", head_dim);
    const int64_t work = num_tokens * num_kv_heads;
    if (work <= 0) return NVK_OK;
    if (work >= 0x7fffffffLL) return fail(NVK_ERR_INVALID_ARGUMENT, "store_kvcache_fp8: too many tokens");
    const int64_t per_block = static_cast<int64_t>(kStoreWarps) * (32 / lanes);
    const int64_t blocks = (work + per_block - 1) / per_block;
#define NVK_LAUNCH_FP8(L)                                                                                           \
    store_fp8_packed_kernel<T, L><<<static_cast<unsigned>(blocks), kStoreWarps * 32, 0, stream>>>(                   \
        static_cast<const T*>(key), static_cast<const T*>(value), static_cast<uint8_t*>(k_cache),                  \
        static_cast<uint8_t*>(v_cache), static_cast<__half*>(k_scale), static_cast<__half*>(v_scale), slot_mapping, \
        static_cast<uint32_t>(work), static_cast<uint32_t>(num_kv_heads), cache_rows)
    switch (lanes) {
        case 8: NVK_LAUNCH_FP8(8); break;
        case 16: NVK_LAUNCH_FP8(16); break;
        default: NVK_LAUNCH_FP8(32); break;
    }
#undef NVK_LAUNCH_FP8
    return check_launch("store_kvcache_fp8 kernel launch");
}

// General decode path: one warp per (sequence, query head), lane owns D / 32 contiguous elements; serial online
// softmax over the keys as in the reference.  Used for fp32 queries and head dims other than 128.
template <typename T, int V>
__global__ void __launch_bounds__(128)
decode_int8_rowwise_kernel(const T* __restrict__ query, const int8_t* __restrict__ k_cache, const int8_t* __restrict__ v_cache,
                           const __half* __restrict__ k_scale, const __half* __restrict__ v_scale,
                           const IndexArray context_lens, const IndexArray block_tables,
                           int64_t batch, int64_t max_blocks, int64_t num_cache_blocks, int num_heads, int num_kv_heads,
                           int block_size, float scale, T* __restrict__ output) {
    constexpr int D = V * 32;
    const int lane = threadIdx.x & 31;
    const int64_t work = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    if (work >= batch * num_heads) return;
    const int64_t seq = work / num_heads;
    const int head = static_cast<int>(work % num_heads);
    const int kv_head = head * num_kv_heads / num_heads;
    float q[V], acc[V];
    load_elems<T, V>(query + work * D + lane * V, q);
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.0f;
    const int64_t k_len = context_lens[seq];
    float running_max = -INFINITY, running_sum = 0.0f;
    const IndexArray table = block_tables + seq * max_blocks;
    for (int64_t k = 0; k < k_len; ++k) {
        const int64_t block = table[k / block_size];
        const bool inside = block >= 0 && block < num_cache_blocks;   // ids outside the cache read as zeros
        const int64_t row = inside ? (block * block_size + k % block_size) * num_kv_heads + kv_head : 0;
        const float ks = inside ? __half2float(k_scale[row]) : 0.0f, vs = inside ? __half2float(v_scale[row]) : 0.0f;
        union { typename PackOf<V>::out v; int8_t e[V]; } kq, vq;
        kq.v = *reinterpret_cast<const typename PackOf<V>::out*>(k_cache + row * D + lane * V);
        vq.v = *reinterpret_cast<const typename PackOf<V>::out*>(v_cache + row * D + lane * V);
        float partial = 0.0f;
#pragma unroll
        for (int i = 0; i < V; ++i) partial += q[i] * (static_cast<float>(kq.e[i]) * ks);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, o);
        const float qk = partial * scale;
        const float old_max = running_max;
        running_max = fmaxf(running_max, qk);
        const float correction = expf(old_max - running_max);
        const float e = expf(qk - running_max);
        running_sum = running_sum * correction + e;
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = acc[i] * correction + e * (static_cast<float>(vq.e[i]) * vs);
    }
    const float inv = running_sum > 0.0f ? 1.0f / running_sum : 0.0f;
    T* dst = output + work * D + lane * V;
#pragma unroll
    for (int i = 0; i < V; ++i) dst[i] = ElemTraits<T>::from_float(acc[i] * inv);
}

template <typename T>
int launch_store_typed(const void* key, const void* value, void* k_cache, void* v_cache, void* k_scale, void* v_scale,
                       const int32_t* slot_mapping, int64_t num_tokens, int num_kv_heads, int head_dim, int64_t cache_rows,
                       cudaStream_t stream) {
    constexpr int V = sizeof(T) == 2 ? 8 : 4;   // 16 bytes per lane
    const int lanes = head_dim / V;
    if (head_dim % V != 0 || (lanes != 8 && lanes != 16 && lanes != 32))
        return fail(NVK_ERR_UNSUPPORTED, "store_kvcache_int8: head_dim must be 64, 128 or 256 (fp32: 32, 64 or 128); got %d", head_dim);
    const int64_t work = num_tokens * num_kv_heads;
    const int64_t per_block = static_cast<int64_t>(kStoreWarps) * (32 / lanes);
    const int64_t blocks = (work + per_block - 1) / per_block;
    if (blocks > 0x7fffffffLL) return fail(NVK_ERR_INVALID_ARGUMENT, "store_kvcache_int8: too many tokens");
    if constexpr (sizeof(T) == 2) {
        if (work > 0 && work < 0x7fffffffLL) {
#define NVK_LAUNCH_PACKED(L)                                                                                        \
    store_int8_packed_kernel<T, L><<<static_cast<unsigned>(blocks), kStoreWarps * 32, 0, stream>>>(                  \
        static_cast<const T*>(key), static_cast<const T*>(value), static_cast<int8_t*>(k_cache),                   \
        static_cast<int8_t*>(v_cache), static_cast<__half*>(k_scale), static_cast<__half*>(v_scale), slot_mapping, \
        static_cast<uint32_t>(work), static_cast<uint32_t>(num_kv_heads), cache_rows)
            switch (lanes) {
                case 8: NVK_LAUNCH_PACKED(8); break;
                case 16: NVK_LAUNCH_PACKED(16); break;
                default: NVK_LAUNCH_PACKED(32); break;
            }
#undef NVK_LAUNCH_PACKED
            return check_launch("store_kvcache_int8 kernel launch");
        }
    }
#define NVK_LAUNCH(L)                                                                                               \
    store_int8_kernel<T, V, L><<<static_cast<unsigned>(blocks), kStoreWarps * 32, 0, stream>>>(                      \
        static_cast<const T*>(key), static_cast<const T*>(value), static_cast<int8_t*>(k_cache),                   \
        static_cast<int8_t*>(v_cache), static_cast<__half*>(k_scale), static_cast<__half*>(v_scale), slot_mapping, \
        num_tokens, num_kv_heads, cache_rows)
    switch (lanes) {
        case 8: NVK_LAUNCH(8); break;
        case 16: NVK_LAUNCH(16); break;
        default: NVK_LAUNCH(32); break;
    }
#undef NVK_LAUNCH
    return check_launch("store_kvcache_int8 kernel launch");
}

template <typename T>
int launch_rowwise_typed(const DecodeInt8Args& a) {
    const int64_t work = a.base.batch * a.base.num_heads;
    const int64_t blocks = (work + 3) / 4;
    if (blocks > 0x7fffffffLL) return fail(NVK_ERR_INVALID_ARGUMENT, "decode attention (int8): too many rows");
#define NVK_LAUNCH(V)                                                                                                        \
    decode_int8_rowwise_kernel<T, V><<<static_cast<unsigned>(blocks), 128, 0, a.base.stream>>>(                               \
        static_cast<const T*>(a.base.q), static_cast<const int8_t*>(a.base.k_cache), static_cast<const int8_t*>(a.base.v_cache), \
        static_cast<const __half*>(a.k_scale), static_cast<const __half*>(a.v_scale), a.base.context_lens, a.base.block_tables, \
        a.base.batch, a.base.max_blocks, a.base.num_cache_blocks, a.base.num_heads, a.base.num_kv_heads, a.base.block_size,   \
        a.base.scale, static_cast<T*>(a.base.out))
    switch (a.base.head_dim) {
        case 64: NVK_LAUNCH(2); break;
        case 128: NVK_LAUNCH(4); break;
        case 256: NVK_LAUNCH(8); break;
        default: return fail(NVK_ERR_UNSUPPORTED, "decode attention (int8): head_dim must be 64, 128 or 256 (got %d)", a.base.head_dim);
    }
#undef NVK_LAUNCH
    return check_launch("decode_int8_rowwise_kernel launch");
}

}  // namespace

int launch_store_int8(const void* key, const void* value, void* k_cache, void* v_cache, void* k_scale, void* v_scale,
                      const int32_t* slot_mapping, int64_t num_tokens, int num_kv_heads, int head_dim, int64_t cache_rows,
                      int dtype, cudaStream_t stream) {
    switch (dtype) {
        case NVK_BF16: return launch_store_typed<__nv_bfloat16>(key, value, k_cache, v_cache, k_scale, v_scale, slot_mapping, num_tokens, num_kv_heads, head_dim, cache_rows, stream);
        case NVK_F16: return launch_store_typed<__half>(key, value, k_cache, v_cache, k_scale, v_scale, slot_mapping, num_tokens, num_kv_heads, head_dim, cache_rows, stream);
        default: return launch_store_typed<float>(key, value, k_cache, v_cache, k_scale, v_scale, slot_mapping, num_tokens, num_kv_heads, head_dim, cache_rows, stream);
    }
}

int launch_store_fp8(const void* key, const void* value, void* k_cache, void* v_cache, void* k_scale, void* v_scale,
                     const int32_t* slot_mapping, int64_t num_tokens, int num_kv_heads, int head_dim, int64_t cache_rows,
                     int dtype, cudaStream_t stream) {
    switch (dtype) {
        case NVK_BF16: return launch_store_fp8_typed<__nv_bfloat16>(key, value, k_cache, v_cache, k_scale, v_scale, slot_mapping, num_tokens, num_kv_heads, head_dim, cache_rows, stream);
        case NVK_F16: return launch_store_fp8_typed<__half>(key, value, k_cache, v_cache, k_scale, v_scale, slot_mapping, num_tokens, num_kv_heads, head_dim, cache_rows, stream);
        default: return fail(NVK_ERR_UNSUPPORTED, "store_kvcache_fp8: key / value must be F16 or BF16");
    }
}

int launch_rowwise_decode_int8(const DecodeInt8Args& a) {
    switch (a.base.dtype) {
        case NVK_BF16: return launch_rowwise_typed<__nv_bfloat16>(a);
        case NVK_F16: return launch_rowwise_typed<__half>(a);
        default: return launch_rowwise_typed<float>(a);
    }
}

}  // namespace nvk
