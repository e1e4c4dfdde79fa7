// Prologue of an attention layer for sm_100a: split packed qkv rows, RMSNorm + neox RoPE on the q and k
// heads, q -> q_out, k / v -> paged cache rows.
//
// Replaces fused_split_norm_rope_store_kernel (src/kernels/split_qkv.cu:62-154 of the reference:
// a 128-thread block per (row, head), one element per thread, a block reduction and a
// shared-memory exchange per head).  Here an 8-warp block owns whole ROWS: position, slot, the row
// of the cos/sin table and the norm weights are fetched once per row instead of once per head.
// A head vector is spread over D/8 lanes, 8 contiguous elements (one 16-byte load and store) per
// lane, so a warp works on 32 / (D/8) heads at a time and a lane holds PIECES 16-byte pieces of
// the row.  The sum of squares is a shuffle reduction inside the lane group and the rotation
// partner (d +- D/2) lives in lane ^ (D/16), so there is no shared memory and no barrier.  The grid
// is persistent (about two blocks per SM) and software-pipelined over rows: the pieces, position and
// slot of the block's next row are requested before the current row is computed.  HBM-bound in the
// limit of many rows (rows * (Hq + 2 Hkv) * D elements read, the same number written); at decode
// batch sizes it is latency-bound.
#include "nvk_internal.cuh"

namespace nvk {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kMaxPieces = 8;

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
    const bool low_half = sub < LANES / 2;
    const int heads = hq + 2 * hkv;                         // <= STRIDE * PIECES (the launcher picks PIECES)
    const int first_head = warp * GROUPS + group;

    union Pack { uint4 v; T e[8]; };
    Pack wq, wk;                                            // norm weights of this lane's 8 elements, kept packed
    wq.v = *reinterpret_cast<const uint4*>(q_weight + sub * 8);
    wk.v = *reinterpret_cast<const uint4*>(k_weight + sub * 8);

    int64_t row = blockIdx.x;
    if (row >= rows) return;
    Pack in[PIECES];
    int pos = positions[row];
    int64_t slot = slot_mapping[row];
#pragma unroll
    for (int u = 0; u < PIECES; ++u) {
        const int head = first_head + u * STRIDE;
        in[u].v = head < heads ? *reinterpret_cast<const uint4*>(qkv + (row * heads + head) * D + sub * 8) : make_uint4(0u, 0u, 0u, 0u);
    }
    for (; row < rows; row += gridDim.x) {
        const bool rotate = pos >= 0 && pos < max_positions;
        const bool store_kv = slot >= 0 && slot < cache_rows;
        // cos / sin of this lane's 8 rotation pairs; the second half of a head uses x * cos + partner * sin
        float cs[8], sn[8];
        {
            const float* table = cos_sin + static_cast<int64_t>(rotate ? pos : 0) * D + (sub % (LANES / 2)) * 8;
            const float4 c0 = *reinterpret_cast<const float4*>(table), c1 = *reinterpret_cast<const float4*>(table + 4);
            const float4 s0 = *reinterpret_cast<const float4*>(table + D / 2), s1 = *reinterpret_cast<const float4*>(table + D / 2 + 4);
            cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
            sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
            if (!low_half) {
#pragma unroll
                for (int i = 0; i < 8; ++i) sn[i] = -sn[i];
            }
        }
        // the block's next row: requested now, used in the next iteration
        const int64_t next = row + gridDim.x;
        Pack nxt[PIECES];
        int pos_next = 0;
        int64_t slot_next = -1;
        if (next < rows) {
            pos_next = positions[next];
            slot_next = slot_mapping[next];
#pragma unroll
            for (int u = 0; u < PIECES; ++u) {
                const int head = first_head + u * STRIDE;
                nxt[u].v = head < heads ? *reinterpret_cast<const uint4*>(qkv + (next * heads + head) * D + sub * 8) : make_uint4(0u, 0u, 0u, 0u);
            }
        }
#pragma unroll
        for (int u = 0; u < PIECES; ++u) {
            const int head = first_head + u * STRIDE;
            if (head - group >= heads) break;         // warp-uniform: no lane group of this warp has a head left
            const bool valid = head < heads;          // lanes without a head still take part in the shuffles
            const bool is_q = head < hq;
            const bool is_k = !is_q && head < hq + hkv;
            float x[8];
            float ss = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) { x[i] = ElemTraits<T>::to_float(in[u].e[i]); ss += x[i] * x[i]; }
#pragma unroll
            for (int o = LANES / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float inv_rms = rsqrtf(ss / static_cast<float>(D) + eps);
            const Pack& w = is_q ? wq : wk;
            Pack out;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                x[i] = x[i] * inv_rms * ElemTraits<T>::to_float(w.e[i]);
                const float partner = __shfl_xor_sync(0xffffffffu, x[i], LANES / 2);
                // positions outside the table leave the value un-rotated; sn carries the sign of this half
                const float rot = x[i] * cs[i] - partner * sn[i];
                out.e[i] = ElemTraits<T>::from_float(rotate ? rot : x[i]);
            }
            if (!valid) continue;
            T* dst;
            if (is_q) {
                dst = q_out + (row * hq + head) * D;
            } else {
                if (!store_kv) continue;
                const int kv = is_k ? head - hq : head - hq - hkv;
                dst = (is_k ? k_cache : v_cache) + (slot * hkv + kv) * D;
                if (!is_k) out.v = in[u].v;           // v heads: plain copy
            }
            *reinterpret_cast<uint4*>(dst + sub * 8) = out.v;
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
