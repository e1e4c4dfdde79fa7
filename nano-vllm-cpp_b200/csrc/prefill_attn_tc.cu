// Varlen causal prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA),
// F16 / BF16, head_dim 128, dense or paged keys (block_size a multiple of 128).
//
// Replaces the same reference code as prefill_attn.cu (src/kernels/attention.cu:114-302,
// src/kernels/flash_attn.cpp:203-300); prefill_attn.cu (mma.sync) remains the path for shapes this
// kernel does not take.
//
// Two kernels live here, chosen by shape: the single-tile kernel described next (odd GQA group sizes) and the
// persistent head-pair kernel further down (even group sizes: the two query heads of a pair share their K / V tiles).
//
// Single-tile kernel: one thread block = 128 query rows of one (sequence, head); 128 threads, thread t owns row t.
//   * Q (128 x 128), K tile (128 keys x 128) and V tile live in shared memory as two 128-byte-wide
//     panels each, written by TMA with the 128-byte swizzle -- exactly the canonical layout the
//     UMMA shared-memory descriptors expect (Q, K: K-major; V: MN-major, so the row-major V tile
//     is consumed as it lies, no transpose).  Paged keys: one TMA box per tile, row coordinate
//     block_tables[seq][tile] * block_size; block ids outside the cache give an out-of-bounds
//     coordinate, which TMA fills with zeros.
//   * S = Q K^T : 8 x tcgen05.mma (M 128, N 128, K 16) issued by one thread, accumulator in TMEM
//     columns [0,128).  Each thread reads its own row of S with tcgen05.ld (no shuffles for the row
//     max / row sum), applies scale + causal mask, and writes P = exp2(s - m) as packed 16-bit pairs
//     back to TMEM columns [0,64) (aliasing S).
//   * O += P V : 8 x tcgen05.mma with A = P from TMEM and B = V from shared memory, accumulator in
//     TMEM columns [128,256).  O is only rescaled when the running maximum grows by more than 8
//     (log2 domain); otherwise the stale maximum keeps being used, which is exact after the final
//     division by the row sum.
//   * 256 TMEM columns and 96 KiB of shared memory per block: two blocks per SM, so one block's
//     softmax overlaps the other's MMAs.  Every mbarrier wait is bounded; on a time-out the block
//     raises an error word, stops waiting, frees its TMEM and returns.
//   * No cluster launch and no multicast anywhere.
#include "decode_body.cuh"

#include <cuda.h>

#include <cmath>
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <utility>

namespace nvk {
namespace {

constexpr int kHeadDim = 128;
constexpr int kBM = 128, kBN = 128, kThreads = 128;
constexpr int kPanelBytes = 128 * 128;          // 128 rows x 64 elements (128 B)
constexpr int kTileBytes = 2 * kPanelBytes;     // 32 KiB
constexpr int kOffQ = 0, kOffK = kTileBytes, kOffV = 2 * kTileBytes, kOffBar = 3 * kTileBytes;
constexpr int kSmemBytes = kOffBar + 128 + 1024;  // + barriers + slack for 1024-byte alignment
constexpr int kTmemCols = 256;
constexpr float kRescaleThreshold = 8.0f;
constexpr long long kWaitCycles = 4000000000LL;  // ~2 s at 2 GHz

__device__ int g_tc_error = 0;

struct TcParams {
    IndexArray cu_q, cu_k, block_tables;
    void* out;
    int64_t num_seqs, total_q, total_k, max_blocks, key_rows, num_cache_blocks;
    int num_heads, num_kv_heads, block_size;
    float scale_log2;
    uint32_t idesc_s, idesc_pv;
};

// ---- PTX wrappers ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// Bounded wait: gives up after kWaitCycles or as soon as another thread of the block gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - start > kWaitCycles) {
            *abort_flag = 1;
            atomicCAS(&g_tc_error, 0, code);
            return false;
        }
    }
}
// Whole-warp wait: lane 0 polls, the result is broadcast (31 fewer spinning threads per warp).
__device__ __forceinline__ bool warp_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_flag, code) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
// D(tmem) (+)= A(smem desc) * B(smem desc)
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
// D(tmem) (+)= A(tmem) * B(smem desc)
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
// SS MMA whose descriptors are a base descriptor plus a compile-time offset of the 14-bit start-address field
// (units of 16 bytes).  The adds sit inside the volatile asm, so the compiler cannot precompute (and then keep in
// registers, or spill) one descriptor pair per MMA of an unrolled loop: the issuing thread stays small.
template <int A_OFF16, int B_OFF16>
__device__ __forceinline__ void umma_ss_off(uint32_t d_tmem, uint64_t a_base, uint64_t b_base, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "add.u64 da, %1, %5;\n\t"
        "add.u64 db, %2, %6;\n\t"
        "setp.ne.u32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}\n"
        :: "r"(d_tmem), "l"(a_base), "l"(b_base), "r"(idesc), "r"(acc), "n"(A_OFF16), "n"(B_OFF16) : "memory");
}
constexpr int kmajor_off16(int step) { return ((step / 4) * kPanelBytes + (step % 4) * 32) / 16; }
// The 8 K-steps of S = Q K^T (both operands K-major: two 64-element panels, 32 bytes per step inside a panel).
template <int... KS>
__device__ __forceinline__ void umma_scores(std::integer_sequence<int, KS...>, uint32_t d_tmem, uint64_t q_base, uint64_t k_base,
                                            uint32_t idesc) {
    (umma_ss_off<kmajor_off16(KS), kmajor_off16(KS)>(d_tmem, q_base, k_base, idesc, KS > 0 ? 1u : 0u), ...);
}
// The 8 K-steps of O += P V (P K-major as above, V MN-major: 2048 bytes per 16 keys).
template <int... KK>
__device__ __forceinline__ void umma_pv(std::integer_sequence<int, KK...>, uint32_t d_tmem, uint64_t p_base, uint64_t v_base,
                                        uint32_t idesc, uint32_t acc_first) {
    (umma_ss_off<kmajor_off16(KK), KK * 2048 / 16>(d_tmem, p_base, v_base, idesc, KK > 0 ? 1u : acc_first), ...);
}

__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}


// The TMEM loads are asynchronous: this pins the use of their results after the preceding
// tcgen05.wait::ld in program order (the compiler may not move register arithmetic across it).
__device__ __forceinline__ void reg_fence32(uint32_t (&r)[32]) {
    asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                      "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]));
    asm volatile("" : "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                      "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]));
}

// sm_100 packed-pair and three-input float instructions: they halve the instruction count of the softmax
// passes, which with two resident warps per scheduler are bound by dependent-issue latency, not by lanes.
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// Maximum of 32 raw scores (keys key_base .. key_base + 31); MASK hides keys >= lim.
template <bool MASK>
__device__ __forceinline__ float chunk_max(const uint32_t (&r)[32], int key_base, int lim) {
    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            v[u] = __uint_as_float(r[i + u]);
            if (MASK && key_base + i + u >= lim) v[u] = -INFINITY;
        }
        m0 = max3(m0, v[0], v[1]); m1 = max3(m1, v[2], v[3]); m2 = max3(m2, v[4], v[5]); m3 = max3(m3, v[6], v[7]);
    }
    return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// 32 scores -> 16 packed probability pairs exp2(s * scale - m); returns their fp32 sum.
template <typename T, bool MASK>
__device__ __forceinline__ float chunk_probs(const uint32_t (&r)[32], uint32_t (&pk)[16], int key_base, int lim,
                                             float scale_log2, float m_use) {
    const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2), neg_m2 = pack_f32x2(-m_use, -m_use);
    uint64_t acc0 = 0ull, acc1 = 0ull;   // two packed pairs of fp32 partial sums
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
        float s0 = __uint_as_float(r[2 * i]), s1 = __uint_as_float(r[2 * i + 1]);
        float s2 = __uint_as_float(r[2 * i + 2]), s3 = __uint_as_float(r[2 * i + 3]);
        if (MASK) {
            if (key_base + 2 * i >= lim) s0 = -INFINITY;
            if (key_base + 2 * i + 1 >= lim) s1 = -INFINITY;
            if (key_base + 2 * i + 2 >= lim) s2 = -INFINITY;
            if (key_base + 2 * i + 3 >= lim) s3 = -INFINITY;
        }
        float x0, x1, x2, x3;
        unpack_f32x2(fma_f32x2(pack_f32x2(s0, s1), scale2, neg_m2), x0, x1);
        unpack_f32x2(fma_f32x2(pack_f32x2(s2, s3), scale2, neg_m2), x2, x3);
        const float p0 = fast_exp2(x0), p1 = fast_exp2(x1), p2 = fast_exp2(x2), p3 = fast_exp2(x3);
        acc0 = add_f32x2(acc0, pack_f32x2(p0, p1));
        acc1 = add_f32x2(acc1, pack_f32x2(p2, p3));
        pk[i] = ElemTraits<T>::pack2(p0, p1);
        pk[i + 1] = ElemTraits<T>::pack2(p2, p3);
    }
    float a0, a1, a2, a3;
    unpack_f32x2(acc0, a0, a1);
    unpack_f32x2(acc1, a2, a3);
    return (a0 + a1) + (a2 + a3);
}
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    const uint32_t lo = ((addr & 0x3FFFFu) >> 4) | ((lbo_bytes >> 4) << 16);
    const uint32_t hi = (sbo_bytes >> 4) | (1u << 14) | (2u << 29);
    return (static_cast<uint64_t>(hi) << 32) | lo;
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 2)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const TcParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ int s_info[4];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5;
    const int head = blockIdx.x;
    const int kvh = head * p.num_kv_heads / p.num_heads;

    // (reversed) tile index -> (sequence, first query row): later tiles of a sequence see more keys
    if (tid == 0) {
        const int64_t want = static_cast<int64_t>(gridDim.y) - 1 - blockIdx.y;
        int64_t acc = 0;
        int found = -1, q0 = 0;
        if (p.cu_q == nullptr) {
            if (want * kBM < p.total_q) { found = 0; q0 = static_cast<int>(want * kBM); }
        } else {
            for (int64_t s = 0; s < p.num_seqs; ++s) {
                const int64_t tiles = (static_cast<int64_t>(p.cu_q[s + 1]) - p.cu_q[s] + kBM - 1) / kBM;
                if (want < acc + tiles) { found = static_cast<int>(s); q0 = static_cast<int>((want - acc) * kBM); break; }
                acc += tiles;
            }
        }
        s_info[0] = found; s_info[1] = q0;
        s_abort = 0;
    }
    __syncthreads();
    const int seq = s_info[0];
    if (seq < 0) return;
    const int q0 = s_info[1];
    int64_t qb, kb;
    int q_len, k_len;
    if (p.cu_q == nullptr) { qb = 0; kb = 0; q_len = static_cast<int>(p.total_q); k_len = static_cast<int>(p.total_k); }
    else {
        qb = p.cu_q[seq]; kb = p.cu_k[seq];
        q_len = p.cu_q[seq + 1] - static_cast<int>(qb); k_len = p.cu_k[seq + 1] - static_cast<int>(kb);
    }
    const int rows_here = min(kBM, q_len - q0);
    const int shift = k_len - q_len;
    int k_hi = shift + q0 + rows_here;
    if (k_hi > k_len) k_hi = k_len;
    const int num_kt = k_hi > 0 ? (k_hi + kBN - 1) / kBN : 0;

    T* out_row0 = static_cast<T*>(p.out) + (static_cast<size_t>(qb + q0) * p.num_heads + head) * kHeadDim;
    const size_t out_stride = static_cast<size_t>(p.num_heads) * kHeadDim;

    if (num_kt == 0) {   // no visible key for any row of this tile
        for (int i = tid; i < rows_here * (kHeadDim / 8); i += kThreads) {
            const int r = i / (kHeadDim / 8), c = i % (kHeadDim / 8);
            *reinterpret_cast<uint4*>(out_row0 + r * out_stride + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
        return;
    }

    // shared memory carve-up (1024-byte aligned panels)
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t sm_q = smem_base + kOffQ, sm_k = smem_base + kOffK, sm_v = smem_base + kOffV;
    const uint32_t bar_q = smem_base + kOffBar, bar_k = bar_q + 8, bar_v = bar_q + 16, bar_s = bar_q + 24, bar_o = bar_q + 32;
    volatile int* abort_flag = &s_abort;

    if (tid == 0) {
        mbar_init(bar_q, 1); mbar_init(bar_k, 1); mbar_init(bar_v, 1); mbar_init(bar_s, 1); mbar_init(bar_o, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncwarp();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    const uint32_t t_s = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);   // this warp's lanes, S / P columns
    const uint32_t t_o = t_s + 128;                                               // O columns

    const IndexArray table = p.block_tables ? p.block_tables + static_cast<int64_t>(seq) * p.max_blocks : IndexArray();
    auto key_row = [&](int key0) -> int {   // row coordinate of a key tile; out-of-range ids -> zero-filled box
        if (table) {
            const int64_t id = table[key0 / p.block_size];
            if (id < 0 || id >= p.num_cache_blocks) return static_cast<int>(p.key_rows);
            return static_cast<int>(id) * p.block_size + key0 % p.block_size;
        }
        return static_cast<int>(kb) + key0;
    };

    if (tid == 0) {
        mbar_expect_tx(bar_q, kTileBytes);
        tma_load_3d(sm_q, &tm_q, 0, head, static_cast<int>(qb) + q0, bar_q);
        tma_load_3d(sm_q + kPanelBytes, &tm_q, 64, head, static_cast<int>(qb) + q0, bar_q);
        const int r0 = key_row(0);
        mbar_expect_tx(bar_k, kTileBytes);
        tma_load_3d(sm_k, &tm_k, 0, kvh, r0, bar_k);
        tma_load_3d(sm_k + kPanelBytes, &tm_k, 64, kvh, r0, bar_k);
        mbar_expect_tx(bar_v, kTileBytes);
        tma_load_3d(sm_v, &tm_v, 0, kvh, r0, bar_v);
        tma_load_3d(sm_v + kPanelBytes, &tm_v, 64, kvh, r0, bar_v);
    }

    const int lim = min(shift + q0 + tid + 1, k_len);   // this row sees keys [0, lim)
    float m_ref = -INFINITY, l_run = 0.0f;
    bool alive = true;

    for (int j = 0; j < num_kt && alive; ++j) {
        const int key0 = j * kBN;
        const uint32_t ph = j & 1;
        // ---- S = Q K^T ------------------------------------------------------------------------------
        if (tid == 0) {
            bool ok = true;
            if (j == 0) ok = mbar_wait(bar_q, 0, abort_flag, 1);
            ok = ok && mbar_wait(bar_k, ph, abort_flag, 2);
            if (ok) {
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (ks >> 2) * kPanelBytes + (ks & 3) * 32;
                    umma_ss(tmem_base, make_smem_desc(sm_q + off, 16, 1024), make_smem_desc(sm_k + off, 16, 1024),
                            p.idesc_s, ks > 0 ? 1u : 0u);
                }
                tc_commit(bar_s);
            }
        }
        __syncwarp();
        alive = warp_mbar_wait(bar_s, ph, abort_flag, 3);
        if (!alive) break;
        tc_fence_after();
        // S_j done => PV_{j-1} done (MMAs retire in order): the K and V buffers are free again.
        if (tid == 0) {
            if (j + 1 < num_kt) {
                const int r = key_row(key0 + kBN);
                mbar_expect_tx(bar_k, kTileBytes);
                tma_load_3d(sm_k, &tm_k, 0, kvh, r, bar_k);
                tma_load_3d(sm_k + kPanelBytes, &tm_k, 64, kvh, r, bar_k);
            }
            if (j > 0) {
                const int r = key_row(key0);
                mbar_expect_tx(bar_v, kTileBytes);
                tma_load_3d(sm_v, &tm_v, 0, kvh, r, bar_v);
                tma_load_3d(sm_v + kPanelBytes, &tm_v, 64, kvh, r, bar_v);
            }
        }

        __syncwarp();   // lane 0 re-joins its warp before the warp-collective TMEM loads
        // ---- softmax: pass 1, row maximum (TMEM loads run one chunk ahead of the arithmetic) -----------
        const bool need_mask = key0 + kBN > min(shift + q0 + 1, k_len);   // block-uniform
        uint32_t ra[32], rb[32];
        float mx;
        tmem_ld32(t_s, ra);
        tc_wait_ld(); reg_fence32(ra);
        tmem_ld32(t_s + 32, rb);
        if (need_mask) {
            mx = chunk_max<true>(ra, key0, lim);
            tc_wait_ld(); reg_fence32(rb);
            tmem_ld32(t_s + 64, ra);
            mx = fmaxf(mx, chunk_max<true>(rb, key0 + 32, lim));
            tc_wait_ld(); reg_fence32(ra);
            tmem_ld32(t_s + 96, rb);
            mx = fmaxf(mx, chunk_max<true>(ra, key0 + 64, lim));
            tc_wait_ld(); reg_fence32(rb);
            mx = fmaxf(mx, chunk_max<true>(rb, key0 + 96, lim));
        } else {
            mx = chunk_max<false>(ra, 0, 0);
            tc_wait_ld(); reg_fence32(rb);
            tmem_ld32(t_s + 64, ra);
            mx = fmaxf(mx, chunk_max<false>(rb, 0, 0));
            tc_wait_ld(); reg_fence32(ra);
            tmem_ld32(t_s + 96, rb);
            mx = fmaxf(mx, chunk_max<false>(ra, 0, 0));
            tc_wait_ld(); reg_fence32(rb);
            mx = fmaxf(mx, chunk_max<false>(rb, 0, 0));
        }
        // start re-reading the scores for pass 2 while the maximum is settled
        tmem_ld32(t_s, ra);
        mx *= p.scale_log2;
        if (__any_sync(0xffffffffu, mx > m_ref + kRescaleThreshold)) {
            const float m_new = fmaxf(m_ref, mx);
            const float f = (m_new == -INFINITY) ? 1.0f : fast_exp2(m_ref - m_new);
            if (j > 0) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    tmem_ld32(t_o + c * 32, r);
                    tc_wait_ld(); reg_fence32(r);
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * f);
                    tmem_st32(t_o + c * 32, r);
                }
            }
            l_run *= f;
            m_ref = m_new;
        }
        const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;

        // ---- softmax: pass 2, P = exp2(s * scale - m) as 16-bit pairs written over S -----------------------
        {
            uint32_t pk[16];
            tc_wait_ld(); reg_fence32(ra);
            tmem_ld32(t_s + 32, rb);
            l_run += need_mask ? chunk_probs<T, true>(ra, pk, key0, lim, p.scale_log2, m_use)
                               : chunk_probs<T, false>(ra, pk, 0, 0, p.scale_log2, m_use);
            tc_wait_ld(); reg_fence32(rb);        // chunk 1 is in registers: columns [0,16) may be overwritten
            tmem_st16(t_s, pk);
            tmem_ld32(t_s + 64, ra);
            l_run += need_mask ? chunk_probs<T, true>(rb, pk, key0 + 32, lim, p.scale_log2, m_use)
                               : chunk_probs<T, false>(rb, pk, 0, 0, p.scale_log2, m_use);
            tc_wait_ld(); reg_fence32(ra);
            tmem_st16(t_s + 16, pk);
            tmem_ld32(t_s + 96, rb);
            l_run += need_mask ? chunk_probs<T, true>(ra, pk, key0 + 64, lim, p.scale_log2, m_use)
                               : chunk_probs<T, false>(ra, pk, 0, 0, p.scale_log2, m_use);
            tc_wait_ld(); reg_fence32(rb);
            tmem_st16(t_s + 32, pk);
            l_run += need_mask ? chunk_probs<T, true>(rb, pk, key0 + 96, lim, p.scale_log2, m_use)
                               : chunk_probs<T, false>(rb, pk, 0, 0, p.scale_log2, m_use);
            tmem_st16(t_s + 48, pk);
        }
        tc_wait_st();

        // ---- last tile: rows of V past the sequence may hold anything; zero them (0 * NaN = NaN) ---------
        if (key0 + kBN > k_len) {
            alive = warp_mbar_wait(bar_v, ph, abort_flag, 4);
            if (alive) {
                const int first_bad = k_len - key0;   // in (0, 128)
                for (int i = tid; i < (kBN - first_bad) * 16; i += kThreads) {
                    const int r = first_bad + i / 16, c16 = i % 16;
                    *reinterpret_cast<uint4*>(smem_gen + kOffV + (c16 >> 3) * kPanelBytes + r * 128 + (c16 & 7) * 16) =
                        make_uint4(0u, 0u, 0u, 0u);
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            }
        }
        tc_fence_before();
        __syncthreads();

        // ---- O += P V ---------------------------------------------------------------------------------
        if (tid == 0 && !*abort_flag) {
            if (mbar_wait(bar_v, ph, abort_flag, 5)) {
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    umma_ts(tmem_base + 128, tmem_base + kk * 8, make_smem_desc(sm_v + kk * 2048, kPanelBytes, 1024),
                            p.idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                }
                tc_commit(bar_o);
            }
        }
    }

    // ---- epilogue ----------------------------------------------------------------------------------------
    __syncwarp();
    if (alive) alive = warp_mbar_wait(bar_o, (num_kt - 1) & 1, abort_flag, 6);
    tc_fence_after();
    if (alive && !*abort_flag) {
        // every thread owns a full row: the row sum needs no cross-lane reduction
        const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
        unsigned char* stage = smem_gen + kOffQ;   // Q is dead after the last S MMA
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld32(t_o + c * 32, r);
            tc_wait_ld();
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                uint4 v;
                v.x = ElemTraits<T>::pack2(__uint_as_float(r[q4 * 8 + 0]) * inv, __uint_as_float(r[q4 * 8 + 1]) * inv);
                v.y = ElemTraits<T>::pack2(__uint_as_float(r[q4 * 8 + 2]) * inv, __uint_as_float(r[q4 * 8 + 3]) * inv);
                v.z = ElemTraits<T>::pack2(__uint_as_float(r[q4 * 8 + 4]) * inv, __uint_as_float(r[q4 * 8 + 5]) * inv);
                v.w = ElemTraits<T>::pack2(__uint_as_float(r[q4 * 8 + 6]) * inv, __uint_as_float(r[q4 * 8 + 7]) * inv);
                const int chunk = c * 4 + q4;
                *reinterpret_cast<uint4*>(stage + tid * 256 + ((chunk ^ (tid & 15)) << 4)) = v;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (alive && !*abort_flag) {
        unsigned char* stage = smem_gen + kOffQ;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int idx = i * kThreads + tid;
            const int r = idx >> 4, chunk = idx & 15;
            if (r < rows_here) {
                const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 256 + ((chunk ^ (r & 15)) << 4));
                *reinterpret_cast<uint4*>(out_row0 + r * out_stride + chunk * 8) = v;
            }
        }
    }
    if (*abort_flag && tid == 0) {
        // give copies that may still be in flight a bounded chance to land before the block retires
        for (int j = 0; j < 2; ++j) {
            const long long start = clock64();
            while (!mbar_try_wait(bar_k, j) && clock64() - start < 2000000) {}
            while (!mbar_try_wait(bar_v, j) && clock64() - start < 4000000) {}
        }
    }
    __syncwarp();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

constexpr int kTmemCols2 = 512;   // head-pair kernels: S0 S1 O0 O1

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

// =================================================================================================
// Head-pair kernel: shared-memory layout and the softmax step.  A block works on the two query heads of a pair
// that share a KV head (K and V tiles are loaded once for both) with 128-key tiles.  The probabilities go to
// SHARED memory (canonical K-major 128-byte-swizzled panels, consumed as the A operand of an SS MMA) instead of
// overwriting the scores in TMEM.  A softmax thread pulls its whole score row into registers first and releases
// the score columns at once, so S_t(j+1) is computed while softmax_t(j) is still running and a tile's softmax
// steps follow each other back to back; P.V_t(j) runs under softmax_t(j+1).  K is double buffered, V single
// buffered, 224 KiB of shared memory and 512 TMEM columns per block.
// =================================================================================================
constexpr int kOff4Q = 0, kOff4K = 2 * kTileBytes, kOff4V = 4 * kTileBytes, kOff4P = 5 * kTileBytes, kOff4Bar = 7 * kTileBytes;
constexpr int kSmemBytes4 = kOff4Bar + 256 + 1024;

// One 128-key online-softmax step of a row.  Scores are read once into registers; `on_scores_read` runs as
// soon as they are (the caller releases the TMEM columns there); probabilities are written to `p_row`
// (this row of the two swizzled P panels).  Returns false when a bounded wait gave up.
template <typename T, typename OnRead>
__device__ __forceinline__ bool softmax_row_to_smem(uint32_t t_s, uint32_t t_o, unsigned char* p_panels, int row,
                                                    bool need_mask, int key0, int lim, float scale_log2, bool first,
                                                    float& m_ref, float& l_run, uint32_t pv_done_bar, uint32_t pv_done_parity,
                                                    volatile int* abort_flag, OnRead on_scores_read) {
    uint32_t r0[32], r1[32], r2[32], r3[32];
    tmem_ld32(t_s, r0);
    tmem_ld32(t_s + 32, r1);
    tmem_ld32(t_s + 64, r2);
    tmem_ld32(t_s + 96, r3);
    tc_wait_ld();
    reg_fence32(r0); reg_fence32(r1); reg_fence32(r2); reg_fence32(r3);
    on_scores_read();
    uint32_t pk[16], pk2[16];
    auto store_chunk = [&](int c32, const uint32_t (&v)[16]) {   // 32 keys = four 16-byte pieces of this row
        unsigned char* panel = p_panels + (c32 >> 1) * kPanelBytes + row * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
            const int cc = (c32 & 1) * 4 + q4;   // 16-byte column inside the 128-byte panel row
            *reinterpret_cast<uint4*>(panel + ((cc ^ (row & 7)) << 4)) =
                make_uint4(v[q4 * 4], v[q4 * 4 + 1], v[q4 * 4 + 2], v[q4 * 4 + 3]);
        }
    };
    auto probs = [&](const uint32_t (&r)[32], uint32_t (&v)[16], int c32, float m_use) -> float {
        return need_mask ? chunk_probs<T, true>(r, v, key0 + 32 * c32, lim, scale_log2, m_use)
                         : chunk_probs<T, false>(r, v, 0, 0, scale_log2, m_use);
    };
    auto row_max = [&]() -> float {
        float mx;
        if (need_mask) {
            mx = fmaxf(fmaxf(chunk_max<true>(r0, key0, lim), chunk_max<true>(r1, key0 + 32, lim)),
                       fmaxf(chunk_max<true>(r2, key0 + 64, lim), chunk_max<true>(r3, key0 + 96, lim)));
        } else {
            mx = fmaxf(fmaxf(chunk_max<false>(r0, 0, 0), chunk_max<false>(r1, 0, 0)),
                       fmaxf(chunk_max<false>(r2, 0, 0), chunk_max<false>(r3, 0, 0)));
        }
        return mx * scale_log2;
    };
    // P.V of the previous step must be complete before O is rescaled and before its P is overwritten: wait
    // as late as that allows (with no rescale, after the first 64 exponentials).
    bool pv_waited = first;
    const float mx = row_max();
    if (__any_sync(0xffffffffu, mx > m_ref + kRescaleThreshold)) {
        if (!pv_waited && !warp_mbar_wait(pv_done_bar, pv_done_parity, abort_flag, 42)) return false;
        pv_waited = true;
        const float m_new = fmaxf(m_ref, mx);
        const float f = (m_new == -INFINITY) ? 1.0f : fast_exp2(m_ref - m_new);
        if (!first) {
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld32(t_o + c * 32, r);
                tc_wait_ld(); reg_fence32(r);
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * f);
                tmem_st32(t_o + c * 32, r);
            }
            tc_wait_st();
        }
        l_run *= f;
        m_ref = m_new;
    }
    const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;
    // the first 64 probabilities wait in registers: by then the previous P.V has all but always completed
    l_run += probs(r0, pk, 0, m_use);
    l_run += probs(r1, pk2, 1, m_use);
    if (!pv_waited && !warp_mbar_wait(pv_done_bar, pv_done_parity, abort_flag, 43)) return false;
    store_chunk(0, pk);
    store_chunk(1, pk2);
    l_run += probs(r2, pk, 2, m_use);
    store_chunk(2, pk);
    l_run += probs(r3, pk2, 3, m_use);
    store_chunk(3, pk2);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic-proxy stores -> visible to the MMA
    return true;
}



// =================================================================================================
// The persistent head-pair kernel.  One block per SM takes (query tile, head pair) items from a
// ticket counter, heaviest query tiles first, and keeps TMEM, barriers and the three warp roles alive
// across items: while the softmax warps write one item's output (staged in the P buffer, which the
// last P.V has finished with), the producer has already fetched the next item's Q and first K tiles and
// the issuer has its first score MMAs in flight.  A block launched per item pays the fill and drain of
// the chain load -> S -> softmax -> P.V -> store (about 1.5 rounds) every time; here only the first
// and last item of a block do.  All barrier phases are counted cumulatively over items.
// =================================================================================================
constexpr int kTicketSlots = 64;
constexpr int kIssuers5 = 2;        // issuing warps, one per query tile
constexpr int kThreads5 = 384;      // three warpgroups (register reallocation works on whole warpgroups)
constexpr int kRegsLow5 = 56;       // registers per thread of the third warpgroup after setmaxnreg.dec
constexpr int kRegsHigh5 = 224;     // registers per thread of the two softmax warpgroups after setmaxnreg.inc
__device__ unsigned int g_prefill_ticket[kTicketSlots];
__device__ unsigned int g_prefill_done[kTicketSlots];

struct Tc5Params {
    TcParams base;
    int pairs;            // head pairs
    int tiles;            // upper bound of query tiles over all sequences
    unsigned int total;   // pairs * tiles
    int slot;             // ticket counter of this launch
};

struct Tc5Item {          // one (query tile, head pair), published by the producer warp
    int kind;             // 1 = work, 0 = no more work
    int seq, q0, pair;
};

// Geometry of an item, derived identically by every role from (seq, q0).
struct Tc5Geom {
    int64_t qb, kb;
    int q_len, k_len, rows_here, shift, num_kt, last_partial;
};
__device__ __forceinline__ Tc5Geom tc5_geometry(const TcParams& p, int seq, int q0) {
    Tc5Geom g;
    if (p.cu_q == nullptr) { g.qb = 0; g.kb = 0; g.q_len = static_cast<int>(p.total_q); g.k_len = static_cast<int>(p.total_k); }
    else {
        g.qb = p.cu_q[seq]; g.kb = p.cu_k[seq];
        g.q_len = p.cu_q[seq + 1] - static_cast<int>(g.qb); g.k_len = p.cu_k[seq + 1] - static_cast<int>(g.kb);
    }
    g.rows_here = min(kBM, g.q_len - q0);
    g.shift = g.k_len - g.q_len;
    int k_hi = g.shift + q0 + g.rows_here;
    if (k_hi > g.k_len) k_hi = g.k_len;
    g.num_kt = k_hi > 0 ? (k_hi + kBN - 1) / kBN : 0;
    g.last_partial = (g.num_kt * kBN > g.k_len) ? g.num_kt - 1 : -1;
    return g;
}

// Query tile number `want` (0 = first tile of the first sequence) -> (seq, q0); false when past the end.
__device__ __forceinline__ bool tc5_locate(const TcParams& p, int64_t want, int& seq, int& q0) {
    if (p.cu_q == nullptr) {
        if (want * kBM >= p.total_q) return false;
        seq = 0; q0 = static_cast<int>(want * kBM);
        return true;
    }
    int64_t acc = 0;
    for (int64_t s = 0; s < p.num_seqs; ++s) {
        const int64_t tiles = (static_cast<int64_t>(p.cu_q[s + 1]) - p.cu_q[s] + kBM - 1) / kBM;
        if (want < acc + tiles) { seq = static_cast<int>(s); q0 = static_cast<int>((want - acc) * kBM); return true; }
        acc += tiles;
    }
    return false;
}

// The decode half of a mixed step (prefill_tc5_kernel<T, true>): the split-K decode items of decode_split_kernel, taken
// from a second ticket counter by the same persistent blocks.  A block runs the two halves one after the other --
// blocks [0, prefill_blocks) the prefill items first, the others the decode items first -- so while some SMs are busy
// on the tensor pipe the rest stream the KV cache, and no SM idles between the two parts of the step as it does at the
// boundary of two launches.  In the decode half the eight softmax warps form two groups of four warps, each with its
// own 96 KiB of the block's shared memory, i.e. what two resident blocks of decode_split_kernel have per SM.
struct MixedDecode {
    dec::DecodeParams dp;
    unsigned int items;       // KV heads x splits x sequences
    int prefill_blocks;
};
__device__ unsigned int g_decode_ticket[kTicketSlots];

template <typename T, bool MIXED>
__global__ void __launch_bounds__(kThreads5, 1)
prefill_tc5_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const Tc5Params pp, const MixedDecode md) {
    const TcParams& p = pp.base;
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ Tc5Item s_ring[4];
    __shared__ int s_dec_blocks[MIXED ? 2 : 1][MIXED ? dec::kMaxChunkBlocks : 1];
    __shared__ unsigned int s_dec_item[2];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    // decode half: warps 0-3 and 4-7 are two independent groups, each taking (KV head, split, sequence) items
    auto decode_half = [&]() {
        if (MIXED && warp < 8) {
            const int group = warp >> 2, gtid = tid & 127, bar = 1 + group;
            unsigned char* gsmem = smem_gen + group * dec::kSmemBytes;
            const unsigned int hkv = static_cast<unsigned int>(md.dp.num_kv_heads), splits = static_cast<unsigned int>(md.dp.num_splits);
            while (true) {
                if (gtid == 0) s_dec_item[group] = atomicAdd(&g_decode_ticket[pp.slot], 1u);
                dec::group_sync(bar);
                const unsigned int item = s_dec_item[group];
                dec::group_sync(bar);   // everyone holds the item before the next ticket overwrites it
                if (item >= md.items) break;
                dec::decode_split_body<T>(md.dp, static_cast<int>(item % hkv), static_cast<int>((item / hkv) % splits),
                                          static_cast<int64_t>(item / (hkv * splits)), gsmem, s_dec_blocks[MIXED ? group : 0], gtid, bar);
                dec::group_sync(bar);   // the group's shared memory is free for its next item
            }
        }
    };
    const bool decode_first = MIXED && static_cast<int>(blockIdx.x) >= md.prefill_blocks;
    if (decode_first) {
        decode_half();
        __syncthreads();
    }
    const uint32_t sm_q = smem_base + kOff4Q, sm_k = smem_base + kOff4K, sm_v = smem_base + kOff4V, sm_p = smem_base + kOff4P;
    const uint32_t bars = smem_base + kOff4Bar;
    const uint32_t bar_qfull = bars, bar_vfix = bars + 8, bar_vfull = bars + 16, bar_vempty = bars + 24, bar_qempty = bars + 144;
    auto bar_kfull = [&](int s) { return bars + 32 + 8 * s; };
    auto bar_kempty = [&](int s) { return bars + 48 + 8 * s; };
    auto bar_sfull = [&](int t) { return bars + 64 + 8 * t; };
    auto bar_sread = [&](int t) { return bars + 80 + 8 * t; };
    auto bar_pfull = [&](int t) { return bars + 96 + 8 * t; };
    auto bar_odone = [&](int t) { return bars + 112 + 8 * t; };
    auto bar_ofinal = [&](int t) { return bars + 128 + 8 * t; };
    auto bar_item = [&](int s) { return bars + 152 + 8 * s; };   // ring entry s published
    volatile int* abort_flag = &s_abort;

    if (tid == 0) {
        s_abort = 0;
        mbar_init(bar_qfull, 1); mbar_init(bar_qempty, kIssuers5); mbar_init(bar_vfix, 1); mbar_init(bar_vfull, 1); mbar_init(bar_vempty, kIssuers5);
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_kfull(i), 1); mbar_init(bar_kempty(i), kIssuers5);
            mbar_init(bar_sfull(i), 1); mbar_init(bar_sread(i), 4); mbar_init(bar_pfull(i), 4);
            mbar_init(bar_odone(i), 1); mbar_init(bar_ofinal(i), 1);
        }
        for (int i = 0; i < 4; ++i) mbar_init(bar_item(i), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncwarp();
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem_base)), "r"(kTmemCols2) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    const size_t out_stride = static_cast<size_t>(p.num_heads) * kHeadDim;

    // Three warpgroups: 0 and 1 are the softmax warps of tile 0 and 1, 2 holds the issuer, the producer and two idle
    // warps.  The block starts with 168 registers per thread (the cap of 384 threads); the third warpgroup hands
    // most of its registers back and the softmax warpgroups grow to 224, which holds a whole 128-key score row, its
    // probabilities and the step's state without spilling.

    if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(kRegsLow5));
    if (warp == 9) {
        // ------------------------------------------------------------------ ticket taker + TMA producer
        int n = 0;            // items published so far (all of them carry work)
        int gk = 0, gv = 0;   // K / V tiles loaded so far, over all items
        bool ok = true;
        // Next item that carries work (whole warp; lane 0 takes the tickets).  Tiles past the last sequence are
        // skipped, tiles whose rows see no key are zero-filled right here and never published.
        auto take_item = [&](int& kind, int& seq, int& q0, int& pair, Tc5Geom& g) {
            while (true) {
                kind = 0; seq = 0; q0 = 0; pair = 0;
                if (lane == 0) {
                    while (true) {
                        const unsigned int ticket = atomicAdd(&g_prefill_ticket[pp.slot], 1u);
                        if (ticket >= pp.total) break;
                        pair = static_cast<int>(ticket % static_cast<unsigned int>(pp.pairs));
                        const int64_t want = static_cast<int64_t>(pp.tiles) - 1 - static_cast<int64_t>(ticket / static_cast<unsigned int>(pp.pairs));
                        if (tc5_locate(p, want, seq, q0)) { kind = 1; break; }
                    }
                }
                kind = __shfl_sync(0xffffffffu, kind, 0);
                seq = __shfl_sync(0xffffffffu, seq, 0);
                q0 = __shfl_sync(0xffffffffu, q0, 0);
                pair = __shfl_sync(0xffffffffu, pair, 0);
                if (!kind) return;
                g = tc5_geometry(p, seq, q0);
                if (g.num_kt > 0) return;
                for (int t = 0; t < 2; ++t) {
                    T* o0 = static_cast<T*>(p.out) + (static_cast<size_t>(g.qb + q0) * p.num_heads + 2 * pair + t) * kHeadDim;
                    for (int i = lane; i < g.rows_here * (kHeadDim / 8); i += 32) {
                        const int r = i / (kHeadDim / 8), c = i % (kHeadDim / 8);
                        *reinterpret_cast<uint4*>(o0 + r * out_stride + c * 8) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
            }
        };
        int kind = 0, seq = 0, q0 = 0, pair = 0;
        Tc5Geom g{};
        int nkind = 0, nseq = 0, nq0 = 0, npair = 0;
        Tc5Geom ng{};
        take_item(nkind, nseq, nq0, npair, ng);
        while (ok) {
            kind = nkind; seq = nseq; q0 = nq0; pair = npair; g = ng;
            if (lane == 0) {
                Tc5Item it;
                it.kind = kind; it.seq = seq; it.q0 = q0; it.pair = pair;
                s_ring[n & 3] = it;
                mbar_arrive(bar_item(n & 3));   // release: the entry is visible to whoever waits on the barrier
            }
            if (!kind) break;
            const int head0 = 2 * pair;
            const int kvh = head0 * p.num_kv_heads / p.num_heads;
            const IndexArray table = p.block_tables ? p.block_tables + static_cast<int64_t>(seq) * p.max_blocks : IndexArray();
            auto key_row = [&](int key0) -> int {
                if (table) {
                    const int64_t id = table[key0 / p.block_size];
                    if (id < 0 || id >= p.num_cache_blocks) return static_cast<int>(p.key_rows);
                    return static_cast<int>(id) * p.block_size + key0 % p.block_size;
                }
                return static_cast<int>(g.kb) + key0;
            };
            auto load_k = [&](int j) -> bool {   // lane 0 only
                const int c = gk + j, s = c & 1;
                if (c >= 2 && !mbar_wait(bar_kempty(s), ((c >> 1) & 1) ^ 1, abort_flag, 11)) return false;
                const int r = key_row(j * kBN);
                mbar_expect_tx(bar_kfull(s), kTileBytes);
                tma_load_3d(sm_k + s * kTileBytes, &tm_k, 0, kvh, r, bar_kfull(s));
                tma_load_3d(sm_k + s * kTileBytes + kPanelBytes, &tm_k, 64, kvh, r, bar_kfull(s));
                return true;
            };
            if (lane == 0) {
                if (n >= 1) ok = mbar_wait(bar_qempty, (n - 1) & 1, abort_flag, 14);   // previous item's score MMAs are done with Q
                if (ok) {
                    mbar_expect_tx(bar_qfull, 2 * kTileBytes);
                    for (int t = 0; t < 2; ++t) {
                        tma_load_3d(sm_q + t * kTileBytes, &tm_q, 0, head0 + t, static_cast<int>(g.qb) + q0, bar_qfull);
                        tma_load_3d(sm_q + t * kTileBytes + kPanelBytes, &tm_q, 64, head0 + t, static_cast<int>(g.qb) + q0, bar_qfull);
                    }
                    ok = load_k(0);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            // the next ticket, its sequence look-up and geometry are fetched now, under this item's rounds
            if (ok) take_item(nkind, nseq, nq0, npair, ng);
            for (int j = 0; j < g.num_kt && ok; ++j) {
                const int cv = gv + j;
                if (lane == 0) {
                    if (j + 1 < g.num_kt) ok = load_k(j + 1);            // K runs one tile ahead of V
                    if (ok && cv >= 1) ok = mbar_wait(bar_vempty, (cv - 1) & 1, abort_flag, 12);
                    if (ok) {
                        const int r = key_row(j * kBN);
                        mbar_expect_tx(bar_vfull, kTileBytes);
                        tma_load_3d(sm_v, &tm_v, 0, kvh, r, bar_vfull);
                        tma_load_3d(sm_v + kPanelBytes, &tm_v, 64, kvh, r, bar_vfull);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (ok && j == g.last_partial) {
                    // rows of V past the sequence may hold anything (0 * NaN = NaN): zero them once landed
                    ok = warp_mbar_wait(bar_vfull, cv & 1, abort_flag, 13);
                    if (ok) {
                        const int first_bad = g.k_len - j * kBN;   // in (0, 128)
                        for (int i = lane; i < (kBN - first_bad) * 16; i += 32) {
                            const int r = first_bad + i / 16, c16 = i % 16;
                            *reinterpret_cast<uint4*>(smem_gen + kOff4V + (c16 >> 3) * kPanelBytes + r * 128 + (c16 & 7) * 16) =
                                make_uint4(0u, 0u, 0u, 0u);
                        }
                        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_vfix);
                    }
                }
            }
            gk += g.num_kt; gv += g.num_kt; ++n;
        }
    } else if (warp == 8 || warp == 8 + 2 * (kIssuers5 - 1)) {
        // ------------------------------------------------------------------ MMA issuer(s): with two, warp 8 drives
        // tile 0 and warp 10 tile 1 (one thread sustains about one MMA per 100 clocks here, the tensor pipe one per 64)
        if (lane == 0) {
            const int t_lo = (kIssuers5 == 2 && warp != 8) ? 1 : 0;
            const int t_hi = (kIssuers5 == 2 && warp == 8) ? 1 : 2;
            int n = 0, G = 0, gk = 0, gv = 0, nf = 0;   // items, rounds, K tiles, V tiles, partial-tile fixes so far
            bool ok = true;
            // One base descriptor per operand buffer; a tile-internal offset only moves the 14-bit start-address
            // field (units of 16 bytes, never carrying out of it), so each MMA's descriptors are one add away and
            // the issuer needs few registers.
            const uint64_t dq[2] = {make_smem_desc(sm_q, 16, 1024), make_smem_desc(sm_q + kTileBytes, 16, 1024)};
            const uint64_t dk[2] = {make_smem_desc(sm_k, 16, 1024), make_smem_desc(sm_k + kTileBytes, 16, 1024)};
            const uint64_t dp[2] = {make_smem_desc(sm_p, 16, 1024), make_smem_desc(sm_p + kTileBytes, 16, 1024)};
            const uint64_t dv = make_smem_desc(sm_v, kPanelBytes, 1024);
            while (ok) {
                ok = mbar_wait(bar_item(n & 3), (n >> 2) & 1, abort_flag, 28);
                if (!ok) break;
                const Tc5Item it = s_ring[n & 3];
                if (it.kind == 0) break;
                const Tc5Geom g = tc5_geometry(p, it.seq, it.q0);
                auto issue_s = [&](int t, int j) {
                    const int s = (gk + j) & 1;
                    umma_scores(std::make_integer_sequence<int, 8>{}, tmem_base + t * 128, dq[t], dk[s], p.idesc_s);
                    tc_commit(bar_sfull(t));
                };
                // scores of the item's first key tile: Q and K(0) landed, the previous round's scores were read
                ok = mbar_wait(bar_qfull, n & 1, abort_flag, 21) && mbar_wait(bar_kfull(gk & 1), (gk >> 1) & 1, abort_flag, 22);
                for (int t = t_lo; t < t_hi && ok; ++t) {
                    if (G >= 1) ok = mbar_wait(bar_sread(t), (G - 1) & 1, abort_flag, 29);
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(t, 0);
                }
                if (!ok) break;
                tc_commit(bar_kempty(gk & 1));              // (every issuer arrives)
                if (g.num_kt == 1) tc_commit(bar_qempty);   // every score MMA of the item has been issued
                for (int j = 0; j < g.num_kt && ok; ++j) {
                    if (j + 1 < g.num_kt) {   // next scores as soon as this step's scores have been read
                        const int c = gk + j + 1;
                        ok = mbar_wait(bar_kfull(c & 1), (c >> 1) & 1, abort_flag, 26);
                        for (int t = t_lo; t < t_hi && ok; ++t) {
                            ok = mbar_wait(bar_sread(t), (G + j) & 1, abort_flag, 27);
                            if (!ok) break;
                            tc_fence_after();
                            issue_s(t, j + 1);
                        }
                        if (!ok) break;
                        tc_commit(bar_kempty(c & 1));
                        if (j + 2 == g.num_kt) tc_commit(bar_qempty);
                    }
                    ok = mbar_wait(bar_vfull, (gv + j) & 1, abort_flag, 23);
                    if (ok && j == g.last_partial) ok = mbar_wait(bar_vfix, nf & 1, abort_flag, 24);
                    for (int t = t_lo; t < t_hi && ok; ++t) {
                        // p_full of an item's first round also says that the previous item's output has left TMEM
                        ok = mbar_wait(bar_pfull(t), (G + j) & 1, abort_flag, 25);
                        if (!ok) break;
                        tc_fence_after();
                        umma_pv(std::make_integer_sequence<int, 8>{}, tmem_base + 256 + t * 128, dp[t], dv, p.idesc_pv, j > 0 ? 1u : 0u);
                        tc_commit(bar_odone(t));
                        if (j == g.num_kt - 1) tc_commit(bar_ofinal(t));
                    }
                    if (ok) tc_commit(bar_vempty);
                }
                G += g.num_kt; gk += g.num_kt; gv += g.num_kt; ++n;
                if (g.last_partial >= 0) ++nf;
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(kRegsHigh5));
        // ------------------------------------------------------------------ softmax warps (thread = row)
        const int t = warp >> 2;
        const int wq = warp & 3;
        const int row = wq * 32 + lane;
        const uint32_t t_s = tmem_base + (static_cast<uint32_t>(wq * 32) << 16) + t * 128;
        const uint32_t t_o = tmem_base + (static_cast<uint32_t>(wq * 32) << 16) + 256 + t * 128;
        unsigned char* p_panels = smem_gen + kOff4P + t * kTileBytes;
        const uint32_t sread = bar_sread(t);
        int n = 0, G = 0;
        bool alive = true;
        while (alive) {
            alive = warp_mbar_wait(bar_item(n & 3), (n >> 2) & 1, abort_flag, 33);
            if (!alive) break;
            const Tc5Item it = s_ring[n & 3];
            if (it.kind == 0) break;
            const Tc5Geom g = tc5_geometry(p, it.seq, it.q0);
            const int q0 = it.q0;
            const int lim = min(g.shift + q0 + row + 1, g.k_len);
            float m_ref = -INFINITY, l_run = 0.0f;
            for (int j = 0; j < g.num_kt; ++j) {
                alive = warp_mbar_wait(bar_sfull(t), (G + j) & 1, abort_flag, 31);
                if (!alive) break;
                tc_fence_after();
                const int key0 = j * kBN;
                const bool need_mask = key0 + kBN > min(g.shift + q0 + 1, g.k_len);
                alive = softmax_row_to_smem<T>(t_s, t_o, p_panels, row, need_mask, key0, lim, p.scale_log2, j == 0, m_ref, l_run,
                                               bar_odone(t), (G + j - 1) & 1, abort_flag, [&] {
                                                   tc_fence_before();
                                                   __syncwarp();
                                                   if (lane == 0) mbar_arrive(sread);   // the score columns may be overwritten
                                               });
                if (!alive) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_pfull(t));
            }
            if (alive) alive = warp_mbar_wait(bar_ofinal(t), n & 1, abort_flag, 32);
            if (!alive) break;
            tc_fence_after();
            {
                // The last P.V is complete, so the P buffer is free: stage this warp's 32 output rows there (16-byte
                // chunks XOR-swizzled by row) and write them out as whole 256-byte rows.  The next item's Q is
                // already being loaded into the Q buffer meanwhile.
                const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
                unsigned char* stage = p_panels;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    tmem_ld32(t_o + c * 32, r);
                    tc_wait_ld(); reg_fence32(r);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 v;
                        v.x = ElemTraits<T>::pack2(__uint_as_float(r[q4 * 8 + 0]) * inv, __uint_as_float(r[q4 * 8 + 1]) * inv);
                        v.y = ElemTraits<T>::pack2(__uint_as_float(r[q4 * 8 + 2]) * inv, __uint_as_float(r[q4 * 8 + 3]) * inv);
                        v.z = ElemTraits<T>::pack2(__uint_as_float(r[q4 * 8 + 4]) * inv, __uint_as_float(r[q4 * 8 + 5]) * inv);
                        v.w = ElemTraits<T>::pack2(__uint_as_float(r[q4 * 8 + 6]) * inv, __uint_as_float(r[q4 * 8 + 7]) * inv);
                        const int chunk = c * 4 + q4;
                        *reinterpret_cast<uint4*>(stage + row * 256 + ((chunk ^ (row & 15)) << 4)) = v;
                    }
                }
                // O has left TMEM: the arrive on p_full in the next item's first round tells the issuer so
                __syncwarp();
                T* o0 = static_cast<T*>(p.out) + (static_cast<size_t>(g.qb + q0) * p.num_heads + 2 * it.pair + t) * kHeadDim;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int r = wq * 32 + 2 * i + (lane >> 4), chunk = lane & 15;
                    if (r < g.rows_here) {
                        const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 256 + ((chunk ^ (r & 15)) << 4));
                        *reinterpret_cast<uint4*>(o0 + r * out_stride + chunk * 8) = v;
                    }
                }
                __syncwarp();   // the staging rows are read before the next item's probabilities overwrite them
            }
            G += g.num_kt; ++n;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols2) : "memory");
    }
    if (MIXED && !decode_first) decode_half();
    if (MIXED) __syncthreads();
    if (tid == 0) {   // the last block to finish re-arms the ticket counters for the next launch that uses this slot
        __threadfence();
        if (atomicAdd(&g_prefill_done[pp.slot], 1u) == gridDim.x - 1) {
            g_prefill_ticket[pp.slot] = 0u;
            g_decode_ticket[pp.slot] = 0u;
            g_prefill_done[pp.slot] = 0u;
            __threadfence();
        }
    }
}

// ---- host side ------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &ptr, 12000, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(ptr);
    });
    return fn;
}

// [rows, heads, 128] 16-bit tensor -> boxes of `box_rows` rows x 1 head x 64 elements, 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* base, int64_t rows, int heads, bool bf16, int box_rows = 128) {
    EncodeFn fn = encode_fn();
    if (fn == nullptr || rows <= 0) return false;
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(kHeadDim), static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(kHeadDim) * 2, static_cast<cuuint64_t>(heads) * kHeadDim * 2};
    const cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[3] = {1, 1, 1};
    return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base),
              dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// kind::f16 instruction descriptor: D = F32, A / B = F16 or BF16, N 128, M 128 (one block) or 256 (a block pair).
uint32_t make_idesc(bool bf16, bool b_mn_major, int m = kBM) {
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (0u << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           (static_cast<uint32_t>(kBN >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}


// Launches that may run at the same time on one device need different ticket counters; 64 of them rotate.
std::atomic<unsigned int> g_launch_seq{0};

// Tensor maps and kernel parameters of a prefill call.
struct TcLaunch {
    CUtensorMap tq, tk, tv;
    TcParams p;
    int64_t tiles;
};
int prepare_tc_launch(const PrefillArgs& a, bool bf16, TcLaunch* out) {
    const bool paged = a.block_tables != nullptr;
    const int64_t key_rows = paged ? a.num_cache_blocks * a.block_size : a.total_k;
    if (!make_map(&out->tq, a.q, a.total_q, a.num_heads, bf16) ||
        !make_map(&out->tk, paged ? a.k_cache : a.k, key_rows, a.num_kv_heads, bf16) ||
        !make_map(&out->tv, paged ? a.v_cache : a.v, key_rows, a.num_kv_heads, bf16))
        return fail(NVK_ERR_CUDA, "prefill attention (tcgen05): cuTensorMapEncodeTiled failed");
    TcParams p{};
    p.cu_q = a.cu_q; p.cu_k = a.cu_k; p.block_tables = a.block_tables; p.out = a.out;
    p.num_seqs = a.cu_q ? a.num_seqs : 1; p.total_q = a.total_q; p.total_k = a.total_k; p.max_blocks = a.max_blocks;
    p.key_rows = key_rows; p.num_cache_blocks = a.num_cache_blocks;
    p.num_heads = a.num_heads; p.num_kv_heads = a.num_kv_heads; p.block_size = paged ? a.block_size : 1;
    p.scale_log2 = a.scale * kLog2e;
    p.idesc_s = make_idesc(bf16, false);
    p.idesc_pv = make_idesc(bf16, true);
    out->p = p;
    out->tiles = (a.total_q + kBM - 1) / kBM + (a.cu_q ? a.num_seqs : 0);
    if (out->tiles > 65535) return fail(NVK_ERR_UNSUPPORTED, "prefill attention (tcgen05): too many query tiles");
    return NVK_OK;
}

// Shared-memory attribute and SM count of the persistent head-pair kernel, once per device.
template <typename T, bool MIXED>
int prepare_tc5(int* sms_out) {
    static bool done[64] = {};
    static int sm_count[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device < 0 || device >= 64) return fail(NVK_ERR_UNSUPPORTED, "prefill attention: device index %d not supported", device);
    if (!done[device]) {
        const cudaError_t e = cudaFuncSetAttribute(prefill_tc5_kernel<T, MIXED>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes4);
        if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "prefill attention (head pairs): cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        if (cudaDeviceGetAttribute(&sm_count[device], cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sm_count[device] <= 0)
            return fail(NVK_ERR_CUDA, "prefill attention (head pairs): cannot read the SM count");
        done[device] = true;
    }
    *sms_out = sm_count[device];
    return NVK_OK;
}

template <typename T>
int launch_typed(const PrefillArgs& a, bool bf16) {
    static bool attr_done[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 0 && device < 64 && !attr_done[device]) {
        const cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "prefill attention (tcgen05): cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        attr_done[device] = true;
    }
    TcLaunch L;
    const int rc = prepare_tc_launch(a, bf16, &L);
    if (rc != NVK_OK) return rc;
    const CUtensorMap &tq = L.tq, &tk = L.tk, &tv = L.tv;
    const TcParams& p = L.p;
    const int64_t tiles = L.tiles;
    const int group = a.num_heads / a.num_kv_heads;
    if (group % 2 == 0) {   // pairs of query heads that share a KV head: persistent blocks, one per SM, items from a ticket counter
        int sms = 0;
        const int rc5 = prepare_tc5<T, false>(&sms);
        if (rc5 != NVK_OK) return rc5;
        Tc5Params pp{};
        pp.base = p;
        pp.pairs = a.num_heads / 2;
        pp.tiles = static_cast<int>(tiles);
        pp.total = static_cast<unsigned int>(pp.pairs) * static_cast<unsigned int>(tiles);
        pp.slot = static_cast<int>(g_launch_seq.fetch_add(1u) % kTicketSlots);
        const unsigned int blocks = pp.total < static_cast<unsigned int>(sms) ? pp.total : static_cast<unsigned int>(sms);
        prefill_tc5_kernel<T, false><<<blocks, kThreads5, kSmemBytes4, a.stream>>>(tq, tk, tv, pp, MixedDecode{});
        return check_launch("prefill_tc5_kernel launch");
    }
    // odd group sizes: one block per (query tile, head)
    const dim3 grid(a.num_heads, static_cast<unsigned>(tiles));
    prefill_tc_kernel<T><<<grid, kThreads, kSmemBytes, a.stream>>>(tq, tk, tv, p);
    return check_launch("prefill_tc_kernel launch");
}

}  // namespace

bool prefill_tc_supported(const PrefillArgs& a) {
    if (a.dtype != NVK_F16 && a.dtype != NVK_BF16) return false;
    if (a.head_dim != kHeadDim) return false;
    if (!aligned_to(a.q, 16) || !aligned_to(a.out, 16)) return false;
    if (a.total_q >= (1LL << 31) || a.num_heads > 65535) return false;
    if (a.block_tables) {
        if (a.block_size % kBN != 0) return false;
        if (!aligned_to(a.k_cache, 16) || !aligned_to(a.v_cache, 16)) return false;
        if (a.num_cache_blocks * a.block_size >= (1LL << 31)) return false;
    } else {
        if (!aligned_to(a.k, 16) || !aligned_to(a.v, 16)) return false;
        if (a.total_k <= 0 || a.total_k >= (1LL << 31)) return false;
    }
    return encode_fn() != nullptr;
}

int launch_prefill_tc(const PrefillArgs& a) {
    return a.dtype == NVK_BF16 ? launch_typed<__nv_bfloat16>(a, true) : launch_typed<__half>(a, false);
}

namespace {

template <typename T>
int launch_mixed_typed(const PrefillArgs& a, const DecodeArgs& d, int prefill_blocks, bool bf16) {
    TcLaunch L;
    int rc = prepare_tc_launch(a, bf16, &L);
    if (rc != NVK_OK) return rc;
    int sms = 0;
    rc = prepare_tc5<T, true>(&sms);
    if (rc != NVK_OK) return rc;
    MixedDecode md{};
    rc = decode_plan(d, &md.dp);
    if (rc != NVK_OK) return rc;
    md.items = static_cast<unsigned int>(d.num_kv_heads) * static_cast<unsigned int>(md.dp.num_splits) * static_cast<unsigned int>(d.batch);
    Tc5Params pp{};
    pp.base = L.p;
    pp.pairs = a.num_heads / 2;
    pp.tiles = static_cast<int>(L.tiles);
    pp.total = static_cast<unsigned int>(pp.pairs) * static_cast<unsigned int>(L.tiles);
    pp.slot = static_cast<int>(g_launch_seq.fetch_add(1u) % kTicketSlots);
    if (prefill_blocks <= 0) {
        // No hint: split the SMs by a crude estimate from host-known sizes -- prefill flops as if all sequences were equally
        // long and had no prefix, at 0.55 PFLOP/s (what the prefill half sustains on a share of the SMs at a few thousand tokens per
        // sequence); decode bytes as if every block table were half full, at 6.5 TB/s.
        const double mean_q = static_cast<double>(a.total_q) / static_cast<double>(a.cu_q ? a.num_seqs : 1);
        const double t_prefill = 4.0 * a.num_heads * kHeadDim * static_cast<double>(a.total_q) * (mean_q + 1.0) / 2.0 / 0.55e15;
        const double t_decode = 0.5 * static_cast<double>(d.batch) * d.max_blocks * d.block_size * d.num_kv_heads * kHeadDim * 4.0 / 6.5e12;
        prefill_blocks = static_cast<int>(sms * t_prefill / (t_prefill + t_decode) + 0.5);
    }
    if (prefill_blocks < 1) prefill_blocks = 1;
    if (prefill_blocks > sms) prefill_blocks = sms;
    md.prefill_blocks = prefill_blocks;
    prefill_tc5_kernel<T, true><<<static_cast<unsigned int>(sms), kThreads5, kSmemBytes4, a.stream>>>(L.tq, L.tk, L.tv, pp, md);
    rc = check_launch("mixed prefill + decode kernel launch");
    if (rc != NVK_OK) return rc;
    return launch_decode_merge(md.dp, d.batch, d.dtype, d.stream);
}

}  // namespace

// One launch for a step with prefill and decode sequences: the head-pair prefill kernel and the tensor-core decode kernel
// must both take their halves, and the decode half needs its split-K workspace.
bool mixed_step_supported(const PrefillArgs& p, const DecodeArgs& d) {
    if (!prefill_tc_supported(p) || (p.num_heads / p.num_kv_heads) % 2 != 0) return false;
    if (!decode_mma_supported(d) || d.workspace == nullptr) return false;
    if (p.dtype != d.dtype || p.num_heads != d.num_heads || p.num_kv_heads != d.num_kv_heads || p.stream != d.stream) return false;
    if (p.total_q <= 0 || d.batch <= 0) return false;
    return true;
}

int launch_mixed_step(const PrefillArgs& p, const DecodeArgs& d, int prefill_blocks) {
    return p.dtype == NVK_BF16 ? launch_mixed_typed<__nv_bfloat16>(p, d, prefill_blocks, true)
                               : launch_mixed_typed<__half>(p, d, prefill_blocks, false);
}

}  // namespace nvk

extern "C" int nvk_prefill_status(void* stream, int* status) {
    using namespace nvk;
    if (!status) return fail(NVK_ERR_INVALID_ARGUMENT, "prefill status: null argument");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int word = 0;
    cudaError_t e = cudaMemcpyFromSymbolAsync(&word, g_tc_error, sizeof(int), 0, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e == cudaSuccess && word != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbolAsync(g_tc_error, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    }
    if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "prefill status: %s", cudaGetErrorString(e));
    *status = word;
    return NVK_OK;
}
