// Varlen causal prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA),
// F16 / BF16, head_dim 128, dense or paged keys (block_size a multiple of 128).
//
// Replaces the same reference code as prefill_attn.cu (src/kernels/attention.cu:114-302,
// src/kernels/flash_attn.cpp:203-300); prefill_attn.cu (mma.sync) remains the path for shapes this
// kernel does not take.
//
// One thread block = 128 query rows of one (sequence, head); 128 threads, thread t owns row t.
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
#include "nvk_internal.cuh"

#include <cuda.h>

#include <cmath>
#include <cstdlib>
#include <mutex>

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
    const int32_t* cu_q; const int32_t* cu_k; const int32_t* block_tables;
    void* out; float* dbg;
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

// UMMA shared-memory descriptor: start address, leading / stride byte offsets (all >> 4), descriptor
// version 1 (bits 46-47), 128-byte swizzle (layout type 2 in bits 61-63).
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

    const int32_t* table = p.block_tables ? p.block_tables + static_cast<int64_t>(seq) * p.max_blocks : nullptr;
    auto key_row = [&](int key0) -> int {   // row coordinate of a key tile; out-of-range ids -> zero-filled box
        if (table) {
            const int id = table[key0 / p.block_size];
            if (id < 0 || id >= p.num_cache_blocks) return static_cast<int>(p.key_rows);
            return id * p.block_size + key0 % p.block_size;
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
        alive = mbar_wait(bar_s, ph, abort_flag, 3);
        __syncwarp();
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
        // ---- softmax: pass 1, row maximum -------------------------------------------------------------
        const bool need_mask = key0 + kBN > min(shift + q0 + 1, k_len);   // block-uniform
        float mx = -INFINITY;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld32(t_s + c * 32, r);
            tc_wait_ld();
            if (p.dbg != nullptr && blockIdx.x == 0 && blockIdx.y == gridDim.y - 1 && j == 0) {
#pragma unroll
                for (int i = 0; i < 32; ++i) p.dbg[tid * kBN + c * 32 + i] = __uint_as_float(r[i]);
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                float s = __uint_as_float(r[i]);
                if (need_mask && key0 + c * 32 + i >= lim) s = -INFINITY;
                mx = fmaxf(mx, s);
            }
        }
        mx *= p.scale_log2;
        if (__any_sync(0xffffffffu, mx > m_ref + kRescaleThreshold)) {
            const float m_new = fmaxf(m_ref, mx);
            const float f = (m_new == -INFINITY) ? 1.0f : fast_exp2(m_ref - m_new);
            if (j > 0) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    tmem_ld32(t_o + c * 32, r);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * f);
                    tmem_st32(t_o + c * 32, r);
                }
            }
            l_run *= f;
            m_ref = m_new;
        }
        const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;

        // ---- softmax: pass 2, P = exp2(s * scale - m) as 16-bit pairs over S ---------------------------
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld32(t_s + c * 32, r);
            tc_wait_ld();
            uint32_t pk[16];
            float part = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float s0 = __uint_as_float(r[2 * i]), s1 = __uint_as_float(r[2 * i + 1]);
                if (need_mask) {
                    if (key0 + c * 32 + 2 * i >= lim) s0 = -INFINITY;
                    if (key0 + c * 32 + 2 * i + 1 >= lim) s1 = -INFINITY;
                }
                const float p0 = fast_exp2(fmaf(s0, p.scale_log2, -m_use));
                const float p1 = fast_exp2(fmaf(s1, p.scale_log2, -m_use));
                part += p0 + p1;
                pk[i] = ElemTraits<T>::pack2(p0, p1);
            }
            l_run += part;
            tmem_st16(t_s + c * 16, pk);
        }
        tc_wait_st();

        // ---- last tile: rows of V past the sequence may hold anything; zero them (0 * NaN = NaN) ---------
        if (key0 + kBN > k_len) {
            alive = mbar_wait(bar_v, ph, abort_flag, 4);
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
    if (alive) alive = mbar_wait(bar_o, (num_kt - 1) & 1, abort_flag, 6);
    __syncwarp();
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

// [rows, heads, 128] 16-bit tensor -> boxes of 128 rows x 1 head x 64 elements, 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* base, int64_t rows, int heads, bool bf16) {
    EncodeFn fn = encode_fn();
    if (fn == nullptr || rows <= 0) return false;
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(kHeadDim), static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(kHeadDim) * 2, static_cast<cuuint64_t>(heads) * kHeadDim * 2};
    const cuuint32_t box[3] = {64, 1, 128};
    const cuuint32_t elem[3] = {1, 1, 1};
    return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base),
              dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// kind::f16 instruction descriptor: D = F32, A / B = F16 or BF16, M 128, N 128.
uint32_t make_idesc(bool bf16, bool b_mn_major) {
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (0u << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           (static_cast<uint32_t>(kBN >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
}

float* g_debug_dump = nullptr;

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
    const bool paged = a.block_tables != nullptr;
    const int64_t key_rows = paged ? a.num_cache_blocks * a.block_size : a.total_k;
    CUtensorMap tq, tk, tv;
    if (!make_map(&tq, a.q, a.total_q, a.num_heads, bf16) ||
        !make_map(&tk, paged ? a.k_cache : a.k, key_rows, a.num_kv_heads, bf16) ||
        !make_map(&tv, paged ? a.v_cache : a.v, key_rows, a.num_kv_heads, bf16))
        return fail(NVK_ERR_CUDA, "prefill attention (tcgen05): cuTensorMapEncodeTiled failed");
    TcParams p{};
    p.cu_q = a.cu_q; p.cu_k = a.cu_k; p.block_tables = a.block_tables; p.out = a.out; p.dbg = g_debug_dump;
    p.num_seqs = a.cu_q ? a.num_seqs : 1; p.total_q = a.total_q; p.total_k = a.total_k; p.max_blocks = a.max_blocks;
    p.key_rows = key_rows; p.num_cache_blocks = a.num_cache_blocks;
    p.num_heads = a.num_heads; p.num_kv_heads = a.num_kv_heads; p.block_size = paged ? a.block_size : 1;
    p.scale_log2 = a.scale * kLog2e;
    p.idesc_s = make_idesc(bf16, false);
    p.idesc_pv = make_idesc(bf16, true);
    const int64_t tiles = (a.total_q + kBM - 1) / kBM + (a.cu_q ? a.num_seqs : 0);
    if (tiles > 65535) return fail(NVK_ERR_UNSUPPORTED, "prefill attention (tcgen05): too many query tiles");
    const dim3 grid(a.num_heads, static_cast<unsigned>(tiles));
    prefill_tc_kernel<T><<<grid, kThreads, kSmemBytes, a.stream>>>(tq, tk, tv, p);
    return check_launch("prefill_tc_kernel launch");
}

}  // namespace

bool prefill_tc_supported(const PrefillArgs& a) {
    static const int mode = [] {   // NVK_PREFILL_IMPL=mma keeps the mma.sync kernel (A/B comparisons)
        const char* e = std::getenv("NVK_PREFILL_IMPL");
        return (e != nullptr && e[0] == 'm') ? 0 : 1;
    }();
    if (mode == 0) return false;
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

}  // namespace nvk

// Debug hooks (declared in csrc/nvk_debug.h, not part of the product ABI).
extern "C" void nvk_debug_set_prefill_dump(float* device_buffer) { nvk::g_debug_dump = device_buffer; }
extern "C" int nvk_debug_take_device_error(void) {
    int v = 0;
    cudaMemcpyFromSymbol(&v, nvk::g_tc_error, sizeof(int));
    const int zero = 0;
    cudaMemcpyToSymbol(nvk::g_tc_error, &zero, sizeof(int));
    return v;
}
