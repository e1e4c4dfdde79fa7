// Prologue of an attention layer for sm_100a: split packed qkv rows, RMSNorm + neox RoPE on the q and k
// heads, q -> q_out, k / v -> paged cache rows.
//
// Replaces fused_split_norm_rope_store_kernel (src/kernels/split_qkv.cu:62-154 of the reference:
// a 128-thread block per (row, head), one element per thread, a block reduction and a
// shared-memory exchange per head).  Here an 8-warp block owns whole ROWS: position, slot, the row
// of the cos/sin table and the norm weights are fetched once per row instead of once per head.
// A head vector is spread over D/8 lanes; a lane holds four whole rotation pairs (d, d + D/2): elements
// [4s, 4s+4) of both halves of the head (two 8-byte loads and stores), so RoPE needs no exchange and a
// warp works on 32 / (D/8) heads at a time.  The sum of squares is a shuffle reduction inside the lane
// group; there is no shared memory and no barrier.  Arithmetic runs on packed fp32 pairs (mul / fma
// .f32x2): the kernel was issue-bound, not byte-bound, with scalar arithmetic and a shuffle per element.
// The grid is persistent (about two blocks per SM) and software-pipelined over rows: the pieces,
// position and slot of the block's next row are requested before the current row is computed.
// HBM-bound in the limit of many rows (rows * (Hq + 2 Hkv) * D elements read, the same number
// written); at decode batch sizes it is latency-bound.
#include "nvk_internal.cuh"

namespace nvk {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kMaxPieces = 8;

// Packed fp32 pairs (one 64-bit register pair per two values; Blackwell executes f32x2 mul / fma at one issue slot).
using F2 = unsigned long long;
__device__ __forceinline__ F2 f2_make(float lo, float hi) {
    F2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_split(F2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ F2 f2_mul(F2 a, F2 b) {
    F2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ F2 f2_fma(F2 a, F2 b, F2 c) {
    F2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
template <typename T> __device__ __forceinline__ F2 f2_unpack(uint32_t w);   // two 16-bit elements -> two floats
template <> __device__ __forceinline__ F2 f2_unpack<__nv_bfloat16>(uint32_t w) {
    return f2_make(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ F2 f2_unpack<__half>(uint32_t w) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    return f2_make(f.x, f.y);
}
template <typename T> __device__ __forceinline__ uint32_t f2_pack(F2 v) {
    float lo, hi;
    f2_split(v, lo, hi);
    return ElemTraits<T>::pack2(lo, hi);
}

template <typename T, int LANES, int PIECES>   // LANES = D / 8 lanes per head: 8, 16 or 32
__global__ void __launch_bounds__(kWarpsPerBlock * 32, PIECES <= 3 ? 2 : 1)
fused_prologue_kernel(const T* __restrict__ qkv, const int32_t* __restrict__ positions,
                      const T* __restrict__ q_weight, const T* __restrict__ k_weight, float eps,
                      const float* __restrict__ cos_sin, int max_positions,
                      const int32_t* __restrict__ slot_mapping, T* __restrict__ k_cache,
                      T* __restrict__ v_cache, int64_t cache_rows, int64_t rows, int hq, int hkv,
                      T* __restrict__ q_out) {
    constexpr int D = LANES * 8;
    constexpr int GROUPS = 32 / LANES;                      // heads a warp handles at once
    constexpr int STRIDE = kWarpsPerBlock * GROUPS;         // heads the block handles at once
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane % LANES, group = lane / LANES;
    const int heads = hq + 2 * hkv;                         // <= STRIDE * PIECES (the launcher picks PIECES)
    const int first_head = warp * GROUPS + group;
    // this lane's 8 elements of a head: [sub*4, sub*4+4) of the first half and the same of the second half, i.e. four
    // whole rotation pairs (d, d + D/2)
    const int lo_off = sub * 4, hi_off = D / 2 + sub * 4;

    struct Piece { uint2 lo, hi; };
    Piece wq, wk;                                           // norm weights of this lane's elements, kept packed
    wq.lo = *reinterpret_cast<const uint2*>(q_weight + lo_off); wq.hi = *reinterpret_cast<const uint2*>(q_weight + hi_off);
    wk.lo = *reinterpret_cast<const uint2*>(k_weight + lo_off); wk.hi = *reinterpret_cast<const uint2*>(k_weight + hi_off);

    int64_t row = blockIdx.x;
    if (row >= rows) return;
    Piece in[PIECES];
    int pos = positions[row];
    int64_t slot = slot_mapping[row];
    auto request = [&](Piece (&dst)[PIECES], int64_t r) {
#pragma unroll
        for (int u = 0; u < PIECES; ++u) {
            const int head = first_head + u * STRIDE;
            if (head < heads) {
                const T* src = qkv + (r * heads + head) * D;
                dst[u].lo = *reinterpret_cast<const uint2*>(src + lo_off);
                dst[u].hi = *reinterpret_cast<const uint2*>(src + hi_off);
            } else {
                dst[u].lo = make_uint2(0u, 0u);
                dst[u].hi = make_uint2(0u, 0u);
            }
        }
    };
    request(in, row);
    for (; row < rows; row += gridDim.x) {
        const bool rotate = pos >= 0 && pos < max_positions;
        const bool store_kv = slot >= 0 && slot < cache_rows;
        // cos / sin of this lane's four rotation pairs
        F2 c01, c23, s01, s23, n01, n23;
        {
            const float* table = cos_sin + static_cast<int64_t>(rotate ? pos : 0) * D + lo_off;
            const float4 c = *reinterpret_cast<const float4*>(table), sn = *reinterpret_cast<const float4*>(table + D / 2);
            c01 = f2_make(c.x, c.y); c23 = f2_make(c.z, c.w);
            s01 = f2_make(sn.x, sn.y); s23 = f2_make(sn.z, sn.w);
            n01 = f2_make(-sn.x, -sn.y); n23 = f2_make(-sn.z, -sn.w);
        }
        // the block's next row: requested now, used in the next iteration
        const int64_t next = row + gridDim.x;
        Piece nxt[PIECES];
        int pos_next = 0;
        int64_t slot_next = -1;
        if (next < rows) {
            pos_next = positions[next];
            slot_next = slot_mapping[next];
            request(nxt, next);
        }
#pragma unroll
        for (int u = 0; u < PIECES; ++u) {
            const int head = first_head + u * STRIDE;
            if (head - group >= heads) break;         // warp-uniform: no lane group of this warp has a head left
            const bool valid = head < heads;          // lanes without a head still take part in the shuffles
            const bool is_q = head < hq;
            const bool is_k = !is_q && head < hq + hkv;
            F2 a01 = f2_unpack<T>(in[u].lo.x), a23 = f2_unpack<T>(in[u].lo.y);   // first half
            F2 b01 = f2_unpack<T>(in[u].hi.x), b23 = f2_unpack<T>(in[u].hi.y);   // second half
            float ss;
            {
                F2 sq = f2_mul(a01, a01);
                sq = f2_fma(a23, a23, sq);
                sq = f2_fma(b01, b01, sq);
                sq = f2_fma(b23, b23, sq);
                float s0, s1;
                f2_split(sq, s0, s1);
                ss = s0 + s1;
            }
#pragma unroll
            for (int o = LANES / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float inv_rms = rsqrtf(ss / static_cast<float>(D) + eps);
            const F2 inv2 = f2_make(inv_rms, inv_rms);
            const Piece& w = is_q ? wq : wk;
            a01 = f2_mul(f2_mul(a01, inv2), f2_unpack<T>(w.lo.x));
            a23 = f2_mul(f2_mul(a23, inv2), f2_unpack<T>(w.lo.y));
            b01 = f2_mul(f2_mul(b01, inv2), f2_unpack<T>(w.hi.x));
            b23 = f2_mul(f2_mul(b23, inv2), f2_unpack<T>(w.hi.y));
            Piece out;
            if (rotate) {   // first half: x cos - partner sin; second half: x cos + partner sin
                out.lo.x = f2_pack<T>(f2_fma(a01, c01, f2_mul(b01, n01)));
                out.lo.y = f2_pack<T>(f2_fma(a23, c23, f2_mul(b23, n23)));
                out.hi.x = f2_pack<T>(f2_fma(b01, c01, f2_mul(a01, s01)));
                out.hi.y = f2_pack<T>(f2_fma(b23, c23, f2_mul(a23, s23)));
            } else {        // positions outside the table leave the value un-rotated
                out.lo.x = f2_pack<T>(a01); out.lo.y = f2_pack<T>(a23);
                out.hi.x = f2_pack<T>(b01); out.hi.y = f2_pack<T>(b23);
            }
            if (!valid) continue;
            T* dst;
            if (is_q) {
                dst = q_out + (row * hq + head) * D;
            } else {
                if (!store_kv) continue;
                const int kv = is_k ? head - hq : head - hq - hkv;
                dst = (is_k ? k_cache : v_cache) + (slot * hkv + kv) * D;
                if (!is_k) out = in[u];               // v heads: plain copy
            }
            *reinterpret_cast<uint2*>(dst + lo_off) = out.lo;
            *reinterpret_cast<uint2*>(dst + hi_off) = out.hi;
        }
#pragma unroll
        for (int u = 0; u < PIECES; ++u) in[u] = nxt[u];
        pos = pos_next;
        slot = slot_next;
    }
}

int prologue_sm_count() {
    static int sms[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
    if (sms[device] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
        sms[device] = n;
    }
    return sms[device];
}

template <typename T, int LANES>
int launch_lanes(const void* qkv, const int32_t* positions, const void* qw, const void* kw, float eps,
                 const float* cos_sin, int64_t max_positions, const int32_t* slot_mapping, void* k_cache,
                 void* v_cache, int64_t cache_rows, int64_t rows, int hq, int hkv, void* q_out, cudaStream_t stream) {
    constexpr int STRIDE = kWarpsPerBlock * (32 / LANES);
    const int heads = hq + 2 * hkv;
    const int pieces = (heads + STRIDE - 1) / STRIDE;
    if (pieces > kMaxPieces)
        return fail(NVK_ERR_UNSUPPORTED, "fused_split_norm_rope_store: at most %d heads (q + 2 kv) at head_dim %d", STRIDE * kMaxPieces, LANES * 8);
    const int64_t resident = static_cast<int64_t>(prologue_sm_count()) * (pieces <= 3 ? 2 : 1);
    const unsigned grid = static_cast<unsigned>(rows < resident ? rows : resident);
#define NVK_LAUNCH(PIECES)                                                                                     \
    fused_prologue_kernel<T, LANES, PIECES><<<grid, kWarpsPerBlock * 32, 0, stream>>>(                         \
        static_cast<const T*>(qkv), positions, static_cast<const T*>(qw), static_cast<const T*>(kw), eps,     \
        cos_sin, static_cast<int>(max_positions), slot_mapping, static_cast<T*>(k_cache),                      \
        static_cast<T*>(v_cache), cache_rows, rows, hq, hkv, static_cast<T*>(q_out))
    switch (pieces) {
        case 1: NVK_LAUNCH(1); break;
        case 2: NVK_LAUNCH(2); break;
        case 3: NVK_LAUNCH(3); break;
        case 4: NVK_LAUNCH(4); break;
        case 5: case 6: NVK_LAUNCH(6); break;
        default: NVK_LAUNCH(8); break;
    }
#undef NVK_LAUNCH
    return check_launch("fused_split_norm_rope_store kernel launch");
}

template <typename T>
int launch_typed(const void* qkv, const int32_t* positions, const void* qw, const void* kw, float eps,
                 const float* cos_sin, int64_t max_positions, const int32_t* slot_mapping, void* k_cache,
                 void* v_cache, int64_t cache_rows, int64_t rows, int hq, int hkv, int d, void* q_out,
                 cudaStream_t stream) {
    switch (d) {
        case 64: return launch_lanes<T, 8>(qkv, positions, qw, kw, eps, cos_sin, max_positions, slot_mapping, k_cache, v_cache, cache_rows, rows, hq, hkv, q_out, stream);
        case 128: return launch_lanes<T, 16>(qkv, positions, qw, kw, eps, cos_sin, max_positions, slot_mapping, k_cache, v_cache, cache_rows, rows, hq, hkv, q_out, stream);
        case 256: return launch_lanes<T, 32>(qkv, positions, qw, kw, eps, cos_sin, max_positions, slot_mapping, k_cache, v_cache, cache_rows, rows, hq, hkv, q_out, stream);
        default: return fail(NVK_ERR_UNSUPPORTED, "fused_split_norm_rope_store: head_dim must be 64, 128 or 256 (got %d)", d);
    }
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
