// Decode prologue for sm_100a: split packed qkv rows, RMSNorm + neox RoPE on the q and k heads,
// q -> q_out, k / v -> paged cache rows.
//
// Replaces fused_split_norm_rope_store_kernel (src/kernels/split_qkv.cu:62-154 of the reference:
// a 128-thread block per (row, head), one element per thread, a block reduction and a
// shared-memory exchange per head).  Here one 8-warp block owns one ROW: position, slot, the row
// of the cos/sin table and the norm weights are fetched once per row instead of once per head, a
// warp takes every 8th head, each lane holds D/32 contiguous elements of a head (one 4/8/16-byte
// load), and all of a warp's head vectors are requested before the first one is used.  The sum
// of squares is a shuffle reduction and the rotation partner (d +- D/2) lives in lane ^ 16, so
// there is no shared memory and no barrier.  HBM-bound in the limit of many rows (rows * (Hq + 2 Hkv)
// * D elements read, the same number written); at decode batch sizes it is latency-bound.
#include "nvk_internal.cuh"

namespace nvk {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kHeadsInFlight = 8;   // head vectors a warp keeps in registers at once

template <int V> struct VecOf;
template <> struct VecOf<2> { using type = uint32_t; };
template <> struct VecOf<4> { using type = uint2; };
template <> struct VecOf<8> { using type = uint4; };

template <typename T, int V>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
fused_prologue_kernel(const T* __restrict__ qkv, const int32_t* __restrict__ positions,
                      const T* __restrict__ q_weight, const T* __restrict__ k_weight, float eps,
                      const float* __restrict__ cos_sin, int max_positions,
                      const int32_t* __restrict__ slot_mapping, T* __restrict__ k_cache,
                      T* __restrict__ v_cache, int64_t cache_rows, int64_t rows, int hq, int hkv,
                      T* __restrict__ q_out) {
    constexpr int D = V * 32;
    using Vec = typename VecOf<V>::type;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int heads = hq + 2 * hkv;
    const int64_t row = blockIdx.x;
    if (row >= rows) return;

    const int pos = positions[row];
    const int64_t slot = slot_mapping[row];
    const bool rotate = pos >= 0 && pos < max_positions;
    const bool store_kv = slot >= 0 && slot < cache_rows;
    const T* src_row = qkv + row * static_cast<int64_t>(heads) * D + lane * V;

    // per-row constants of this lane: cos / sin of its V rotation pairs, q and k norm weights
    float cs[V], sn[V], wq[V], wk[V];
    {
        const float* table = cos_sin + static_cast<int64_t>(rotate ? pos : 0) * D + (lane & 15) * V;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            cs[i] = rotate ? table[i] : 1.0f;
            sn[i] = rotate ? table[i + D / 2] : 0.0f;
            wq[i] = ElemTraits<T>::to_float(q_weight[lane * V + i]);
            wk[i] = ElemTraits<T>::to_float(k_weight[lane * V + i]);
        }
    }

    for (int base = warp; base < heads; base += kWarpsPerBlock * kHeadsInFlight) {
        union Pack { Vec v; T e[V]; };
        Pack in[kHeadsInFlight];
#pragma unroll
        for (int u = 0; u < kHeadsInFlight; ++u) {   // all loads first
            const int head = base + u * kWarpsPerBlock;
            if (head < heads) in[u].v = *reinterpret_cast<const Vec*>(src_row + static_cast<int64_t>(head) * D);
        }
#pragma unroll
        for (int u = 0; u < kHeadsInFlight; ++u) {
            const int head = base + u * kWarpsPerBlock;
            if (head >= heads) break;
            const bool is_q = head < hq;
            const bool is_k = !is_q && head < hq + hkv;
            T* dst;
            if (is_q) {
                dst = q_out + (row * hq + head) * D;
            } else {
                if (!store_kv) continue;   // warp-uniform
                const int kv = is_k ? head - hq : head - hq - hkv;
                dst = (is_k ? k_cache : v_cache) + (slot * hkv + kv) * D;
            }
            Pack out;
            if (is_q || is_k) {
                float x[V];
                float ss = 0.0f;
#pragma unroll
                for (int i = 0; i < V; ++i) { x[i] = ElemTraits<T>::to_float(in[u].e[i]); ss += x[i] * x[i]; }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                const float inv_rms = rsqrtf(ss / static_cast<float>(D) + eps);
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    x[i] = x[i] * inv_rms * (is_q ? wq[i] : wk[i]);
                    const float partner = __shfl_xor_sync(0xffffffffu, x[i], 16);
                    // positions outside the table keep cs = 1, sn = 0: the value passes through un-rotated
                    const float rot = lane < 16 ? x[i] * cs[i] - partner * sn[i] : x[i] * cs[i] + partner * sn[i];
                    out.e[i] = ElemTraits<T>::from_float(rotate ? rot : x[i]);
                }
            } else {
                out.v = in[u].v;   // v heads: plain copy
            }
            *reinterpret_cast<Vec*>(dst + lane * V) = out.v;
        }
    }
}

template <typename T>
int launch_typed(const void* qkv, const int32_t* positions, const void* qw, const void* kw, float eps,
                 const float* cos_sin, int64_t max_positions, const int32_t* slot_mapping, void* k_cache,
                 void* v_cache, int64_t cache_rows, int64_t rows, int hq, int hkv, int d, void* q_out,
                 cudaStream_t stream) {
    const int64_t blocks = rows;
    if (blocks > 0x7fffffffLL) return fail(NVK_ERR_INVALID_ARGUMENT, "fused_split_norm_rope_store: too many rows");
    const dim3 grid(static_cast<unsigned>(blocks));
#define NVK_LAUNCH(V)                                                                                          \
    fused_prologue_kernel<T, V><<<grid, kWarpsPerBlock * 32, 0, stream>>>(                                     \
        static_cast<const T*>(qkv), positions, static_cast<const T*>(qw), static_cast<const T*>(kw), eps,     \
        cos_sin, static_cast<int>(max_positions), slot_mapping, static_cast<T*>(k_cache),                      \
        static_cast<T*>(v_cache), cache_rows, rows, hq, hkv, static_cast<T*>(q_out))
    switch (d) {
        case 64: NVK_LAUNCH(2); break;
        case 128: NVK_LAUNCH(4); break;
        case 256: NVK_LAUNCH(8); break;
        default: return fail(NVK_ERR_UNSUPPORTED, "fused_split_norm_rope_store: head_dim must be 64, 128 or 256 (got %d)", d);
    }
#undef NVK_LAUNCH
    return check_launch("fused_split_norm_rope_store kernel launch");
}

}  // namespace

int launch_fused_prologue(const void* qkv, const int32_t* positions, const void* qw, const void* kw, float eps,
                          const float* cos_sin, int64_t max_positions, const int32_t* slot_mapping,
                          void* k_cache, void* v_cache, int64_t cache_rows, int64_t rows, int hq, int hkv,
                          int d, void* q_out, int dtype, cudaStream_t stream) {
    if (dtype == NVK_BF16)
        return launch_typed<__nv_bfloat16>(qkv, positions, qw, kw, eps, cos_sin, max_positions, slot_mapping,
                                           k_cache, v_cache, cache_rows, rows, hq, hkv, d, q_out, stream);
    return launch_typed<__half>(qkv, positions, qw, kw, eps, cos_sin, max_positions, slot_mapping, k_cache,
                                v_cache, cache_rows, rows, hq, hkv, d, q_out, stream);
}

}  // namespace nvk
