// Prologue of an attention layer for sm_100a: split packed qkv rows, RMSNorm + neox RoPE on the q and k
// heads, q -> q_out, k / v -> paged cache rows.
//
// Replaces fused_split_norm_rope_store_kernel (src/kernels/split_qkv.cu:62-154 of the reference:
// a 128-thread block per (row, head), one element per thread, a block reduction and a
// shared-memory exchange per head).
//
// The op is a streaming copy with a little arithmetic: (Hq + 2 Hkv) * D elements read per row, the same
// number written, one row of the fp32 cos / sin table per row.  It is HBM-bound when there are many rows
// and launch / latency-bound at decode batch sizes, so the kernel is built for many light warps:
//   * a head vector is spread over D / 16 lanes; a lane holds eight whole rotation pairs (d, d + D/2):
//     elements [8s, 8s + 8) of both halves of the head, i.e. two 16-byte loads and two 16-byte stores, so
//     RoPE needs no exchange and a warp works on 32 / (D/16) heads at a time;
//   * a warp takes a unit = (row, kSteps consecutive head groups): all of a unit's loads are issued before
//     any arithmetic; position, slot, the table row and the norm weights are fetched once per unit (the table
//     row and the weights hit L1 / L2);
//   * the sum of squares is a shuffle reduction inside the lane group; no shared memory, no barrier;
//   * arithmetic on packed fp32 pairs (mul / fma .f32x2);
//   * about 64 registers per thread, so four 256-thread blocks (32 warps) are resident per SM -- the first
//     version of this kernel kept three heads and a prefetched row per thread in 122 registers and was
//     latency-bound at 16 warps per SM.
// The launch carries the programmatic-stream-serialization attribute: the kernel waits for its predecessor
// in the stream with griddepcontrol.wait as its first action, so its launch latency overlaps the predecessor's
// tail, and it releases its own dependents at once (they wait the same way).
#include "nvk_internal.cuh"

namespace nvk {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kSteps = 2;   // head groups per unit

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

// Streaming 16-byte load of the packed rows (read once: no L1 allocation).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t word(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

struct PrologueParams {
    const void* qkv; const int32_t* positions; const void* q_weight; const void* k_weight;
    const float* cos_sin; const int32_t* slot_mapping;
    void* k_cache; void* v_cache; void* q_out;
    int64_t cache_rows, rows;
    int max_positions, hq, hkv;
    float eps;
};

template <typename T, int D>   // D = head_dim: 64, 128 or 256
__global__ void __launch_bounds__(kWarpsPerBlock * 32, 4) fused_prologue_kernel(const PrologueParams p) {
    constexpr int LANES = D / 16;                           // lanes per head
    constexpr int GROUPS = 32 / LANES;                      // heads a warp handles at once
    asm volatile("griddepcontrol.wait;\n" ::: "memory");    // the packed rows come from the kernel before this one
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane % LANES, group = lane / LANES;
    const int heads = p.hq + 2 * p.hkv;
    const int units_per_row = (heads + GROUPS * kSteps - 1) / (GROUPS * kSteps);
    const int64_t units = p.rows * units_per_row;
    // this lane's 16 elements of a head: [8 sub, 8 sub + 8) of the first half and the same of the second half, i.e. eight
    // whole rotation pairs (d, d + D/2)
    const int lo_off = sub * 8, hi_off = D / 2 + sub * 8;
    const T* qkv = static_cast<const T*>(p.qkv);
    const bool normed = p.q_weight != nullptr;

    for (int64_t u = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp; u < units;
         u += static_cast<int64_t>(gridDim.x) * kWarpsPerBlock) {
        const int64_t row = u / units_per_row;
        const int head0 = static_cast<int>(u - row * units_per_row) * (GROUPS * kSteps) + group;
        uint4 lo[kSteps], hi[kSteps];
#pragma unroll
        for (int s = 0; s < kSteps; ++s) {                  // every load of the unit first
            const int head = head0 + s * GROUPS;
            if (head < heads) {
                const T* src = qkv + (row * heads + head) * D;
                lo[s] = ld_stream16(src + lo_off);
                hi[s] = ld_stream16(src + hi_off);
            } else {
                lo[s] = make_uint4(0u, 0u, 0u, 0u);
                hi[s] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        const int pos = __ldg(p.positions + row);
        const int64_t slot = p.slot_mapping != nullptr ? static_cast<int64_t>(__ldg(p.slot_mapping + row)) : row;
        const bool rotate = pos >= 0 && pos < p.max_positions;
        const bool store_kv = slot >= 0 && slot < p.cache_rows;
        const float* table = p.cos_sin + static_cast<int64_t>(rotate ? pos : 0) * D + lo_off;
#pragma unroll
        for (int s = 0; s < kSteps; ++s) {
            const int head = head0 + s * GROUPS;
            if (head - group >= heads) break;         // warp-uniform: no lane group of this warp has a head left
            const bool valid = head < heads;          // lanes without a head still take part in the shuffles
            const bool is_q = head < p.hq;
            const bool is_k = !is_q && head < p.hq + p.hkv;
            uint4 out_lo = lo[s], out_hi = hi[s];     // v heads (and lanes without a head): the loaded values as they are
            // every lane of a warp that has a q or k head runs the arithmetic (the shuffles need the whole warp); a warp
            // whose heads of this step are all v heads skips it
            if (__any_sync(0xffffffffu, valid && (is_q || is_k))) {
                float inv_rms = 1.0f;
                if (normed) {
                    F2 sq = f2_make(0.0f, 0.0f);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const F2 a = f2_unpack<T>(word(lo[s], i)), b = f2_unpack<T>(word(hi[s], i));
                        sq = f2_fma(a, a, sq);
                        sq = f2_fma(b, b, sq);
                    }
                    float s0, s1;
                    f2_split(sq, s0, s1);
                    float ss = s0 + s1;
#pragma unroll
                    for (int o = LANES / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    inv_rms = rsqrtf(ss / static_cast<float>(D) + p.eps);
                }
                const F2 inv2 = f2_make(inv_rms, inv_rms);
                const T* weight = static_cast<const T*>(is_q ? p.q_weight : p.k_weight);
                uint4 w_lo = make_uint4(0u, 0u, 0u, 0u), w_hi = w_lo;
                if (normed) {
                    w_lo = __ldg(reinterpret_cast<const uint4*>(weight + lo_off));
                    w_hi = __ldg(reinterpret_cast<const uint4*>(weight + hi_off));
                }
                uint32_t r_lo[4], r_hi[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {         // two rotation pairs per trip
                    F2 a = f2_unpack<T>(word(lo[s], i)), b = f2_unpack<T>(word(hi[s], i));
                    if (normed) {
                        a = f2_mul(f2_mul(a, inv2), f2_unpack<T>(word(w_lo, i)));
                        b = f2_mul(f2_mul(b, inv2), f2_unpack<T>(word(w_hi, i)));
                    }
                    if (rotate) {   // first half: x cos - partner sin; second half: x cos + partner sin
                        const float2 c = __ldg(reinterpret_cast<const float2*>(table + 2 * i));
                        const float2 sn = __ldg(reinterpret_cast<const float2*>(table + D / 2 + 2 * i));
                        const F2 c2 = f2_make(c.x, c.y), s2 = f2_make(sn.x, sn.y), n2 = f2_make(-sn.x, -sn.y);
                        r_lo[i] = f2_pack<T>(f2_fma(a, c2, f2_mul(b, n2)));
                        r_hi[i] = f2_pack<T>(f2_fma(b, c2, f2_mul(a, s2)));
                    } else {        // positions outside the table leave the value un-rotated
                        r_lo[i] = f2_pack<T>(a);
                        r_hi[i] = f2_pack<T>(b);
                    }
                }
                if (is_q || is_k) {
                    out_lo = make_uint4(r_lo[0], r_lo[1], r_lo[2], r_lo[3]);
                    out_hi = make_uint4(r_hi[0], r_hi[1], r_hi[2], r_hi[3]);
                }
            }
            if (!valid) continue;
            T* dst;
            if (is_q) {
                dst = static_cast<T*>(p.q_out) + (row * p.hq + head) * D;
            } else {
                if (!store_kv) continue;
                const int kv = is_k ? head - p.hq : head - p.hq - p.hkv;
                dst = static_cast<T*>(is_k ? p.k_cache : p.v_cache) + (slot * p.hkv + kv) * D;
            }
            *reinterpret_cast<uint4*>(dst + lo_off) = out_lo;
            *reinterpret_cast<uint4*>(dst + hi_off) = out_hi;
        }
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

template <typename T, int D>
int launch_dim(const PrologueParams& p, cudaStream_t stream) {
    constexpr int GROUPS = 32 / (D / 16);
    const int heads = p.hq + 2 * p.hkv;
    const int64_t units = p.rows * ((heads + GROUPS * kSteps - 1) / (GROUPS * kSteps));
    const int64_t resident = static_cast<int64_t>(prologue_sm_count()) * 4;   // four blocks per SM
    int64_t blocks = (units + kWarpsPerBlock - 1) / kWarpsPerBlock;
    if (blocks > resident) blocks = resident;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(blocks));
    cfg.blockDim = dim3(kWarpsPerBlock * 32);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, fused_prologue_kernel<T, D>, p);
    if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "fused_split_norm_rope_store kernel launch: %s", cudaGetErrorString(e));
    return check_launch("fused_split_norm_rope_store kernel launch");
}

template <typename T>
int launch_typed(const PrologueParams& p, int d, cudaStream_t stream) {
    switch (d) {
        case 64: return launch_dim<T, 64>(p, stream);
        case 128: return launch_dim<T, 128>(p, stream);
        case 256: return launch_dim<T, 256>(p, stream);
        default: return fail(NVK_ERR_UNSUPPORTED, "fused_split_norm_rope_store: head_dim must be 64, 128 or 256 (got %d)", d);
    }
}

}  // namespace

int launch_fused_prologue(const void* qkv, const int32_t* positions, const void* qw, const void* kw, float eps,
                          const float* cos_sin, int64_t max_positions, const int32_t* slot_mapping,
                          void* k_cache, void* v_cache, int64_t cache_rows, int64_t rows, int hq, int hkv,
                          int d, void* q_out, int dtype, cudaStream_t stream) {
    PrologueParams p{};
    p.qkv = qkv; p.positions = positions; p.q_weight = qw; p.k_weight = kw; p.cos_sin = cos_sin;
    p.slot_mapping = slot_mapping; p.k_cache = k_cache; p.v_cache = v_cache; p.q_out = q_out;
    p.cache_rows = cache_rows; p.rows = rows; p.max_positions = static_cast<int>(max_positions);
    p.hq = hq; p.hkv = hkv; p.eps = eps;
    return dtype == NVK_BF16 ? launch_typed<__nv_bfloat16>(p, d, stream) : launch_typed<__half>(p, d, stream);
}

}  // namespace nvk
