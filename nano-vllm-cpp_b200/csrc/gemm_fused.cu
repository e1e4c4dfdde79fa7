// The two linears on either side of attention, fused with what follows them (tcgen05 + TMEM + TMA, F16 / BF16):
//
//   * QKV projection + attention prologue.  The reference runs qkv_proj as a cuBLASLt GEMM (src/layers/linear.cpp:348-420),
//     writes the packed [rows, (Hq + 2 Hkv) * D] tensor and reads it back in fused_split_norm_rope_store
//     (src/kernels/split_qkv.cu:62-154, called from src/models/transformer.cpp:132-139).  With head_dim 128 one
//     128-column tile of the GEMM IS one head: the epilogue thread that owns a row of the accumulator holds the whole
//     head vector, so the per-head RMSNorm, the rotation pairs (d, d + 64) and the scatter into the paged cache need no
//     exchange at all.  The packed tensor never exists.
//   * Row-parallel projection + all-reduce.  o_proj / down_proj produce a partial sum that is all-reduced over the
//     tensor-parallel ranks (src/layers/linear.cpp:306-320).  Here the epilogue writes each row of the partial sum
//     straight to the rank that will reduce it: its own rows into its addend buffer, the others as tagged vectors into
//     the owners' staging areas over NVLink -- the first phase of nvk_tp_allreduce_add_rmsnorm (tp_allreduce.cu) done
//     by the GEMM, tile by tile, while the other tiles still compute.  The all-reduce kernel that follows is told to
//     skip its push.
//
// GEMM core: C[M, N] = A[M, K] * B[N, K]^T, both operands K-major as torch linears keep them.  One block per 128 x 128
// tile of C; a TMA warp streams 128 x 64 panels of A and B (128-byte swizzle) through a ring of shared-memory stages,
// one thread issues tcgen05.mma (M 128, N 128, K 16) into a 128-column TMEM accumulator, four warps read it back
// (thread = row) for the epilogue.  At decode sizes (M = a few hundred rows) the GEMM streams the weight once and is
// HBM-bound; what the fusion removes is the round trip of the result and one or two launches per layer.
// Every mbarrier wait is bounded; a wait that runs out raises an error word (nvk_gemm_status) and the block leaves.
#include "nvk_internal.cuh"

#include <cuda.h>

#include <atomic>
#include <mutex>

namespace nvk {
namespace {

constexpr int kBM = 128, kBN = 128, kBK = 64;
constexpr int kPanelBytes = kBM * kBK * 2;            // 16 KiB: 128 rows x 128 bytes
constexpr int kStageBytes = 2 * kPanelBytes;          // A panel + B panel
constexpr int kStages = 6;
constexpr int kBarOffset = kStages * kStageBytes;     // 192 KiB
constexpr int kSmemBytes = kBarOffset + 256 + 1024;
constexpr int kThreads = 192;                         // warp 0 TMA, warp 1 MMA + TMEM, warps 2-5 epilogue
constexpr int kTmemCols = 128;
constexpr long long kWaitCycles = 4000000000LL;       // ~2 s
constexpr int kMaxRanks = NVK_TP_MAX_RANKS;

__device__ int g_gemm_error = 0;

enum Epilogue { kPlain = 0, kQkvPrologue = 1, kAllReducePush = 2 };

struct GemmParams {
    void* out;                 // kPlain: C [M, N]
    int64_t m, n, k;
    uint32_t idesc;
    // kQkvPrologue
    const int32_t* positions; const void* q_weight; const void* k_weight; const float* cos_sin; const int32_t* slot_mapping;
    void* q_out; void* k_cache; void* v_cache;
    int64_t cache_rows;
    int max_positions, hq, hkv;
    float eps;
    // kAllReducePush
    void* addend;              // this rank's addend buffer [M, N]: rows it reduces itself
    uint4* stage[kMaxRanks];   // every rank's staging area (index = rank)
    const uint32_t* flags;     // this rank's flag area: [0] = epoch of the last completed all-reduce
    int rank, world;
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - start > kWaitCycles) {
            *abort_flag = 1;
            atomicCAS(&g_gemm_error, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
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
// pins the use of asynchronously loaded registers after the preceding tcgen05.wait::ld
__device__ __forceinline__ void reg_fence32(uint32_t (&r)[32]) {
    asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                      "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]));
    asm volatile("" : "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                      "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]));
}
// K-major, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr) {
    const uint32_t lo = ((addr & 0x3FFFFu) >> 4) | ((16u >> 4) << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return (static_cast<uint64_t>(hi) << 32) | lo;
}
__device__ __forceinline__ void st_tagged(uint4* slot, const uint4& v, uint32_t ep) {   // the all-reduce's wire format
    // one 32-byte store per payload vector: a warp writes 1 KiB of contiguous, fully covered 128-byte lines (two 16-byte
    // stores per lane left every sector half written per instruction, which costs NVLink packets)
    asm volatile("st.volatile.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n"
                 ::"l"(slot), "r"(v.x), "r"(ep), "r"(v.y), "r"(ep), "r"(v.z), "r"(ep), "r"(v.w), "r"(ep) : "memory");
}

// 32 accumulator columns of this thread's row, rounded to T (what the unfused GEMM would have written)
template <typename T>
__device__ __forceinline__ void load_rounded(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    tmem_ld32(taddr, r);
    tc_wait_ld();
    reg_fence32(r);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = ElemTraits<T>::to_float(ElemTraits<T>::from_float(__uint_as_float(r[i])));
}
template <typename T>
__device__ __forceinline__ void store32(T* dst, const float (&v)[32]) {   // 64 bytes, 16-byte aligned
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        uint4 w;
        w.x = ElemTraits<T>::pack2(v[q * 8 + 0], v[q * 8 + 1]); w.y = ElemTraits<T>::pack2(v[q * 8 + 2], v[q * 8 + 3]);
        w.z = ElemTraits<T>::pack2(v[q * 8 + 4], v[q * 8 + 5]); w.w = ElemTraits<T>::pack2(v[q * 8 + 6], v[q * 8 + 7]);
        reinterpret_cast<uint4*>(dst)[q] = w;
    }
}

template <typename T, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = smem_base + kBarOffset;
    auto bar_full = [&](int s) { return bars + 8 * s; };
    auto bar_empty = [&](int s) { return bars + 64 + 8 * s; };
    const uint32_t bar_acc = bars + 128;
    volatile int* abort_flag = &s_abort;
    const int n0 = blockIdx.x * kBN, m0 = blockIdx.y * kBM;
    const int kb_count = static_cast<int>((p.k + kBK - 1) / kBK);

    asm volatile("griddepcontrol.wait;\n" ::: "memory");             // A comes from the kernel before this one
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
        mbar_init(bar_acc, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncwarp();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            for (int kb = 0; kb < kb_count; ++kb) {
                const int s = kb % kStages;
                if (kb >= kStages && !mbar_wait(bar_empty(s), ((kb / kStages) & 1) ^ 1, abort_flag, 1)) break;
                mbar_expect_tx(bar_full(s), kStageBytes);
                tma_load_2d(smem_base + s * kStageBytes, &tm_a, kb * kBK, m0, bar_full(s));
                tma_load_2d(smem_base + s * kStageBytes + kPanelBytes, &tm_b, kb * kBK, n0, bar_full(s));
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            bool ok = true;
            for (int kb = 0; kb < kb_count && ok; ++kb) {
                const int s = kb % kStages;
                ok = mbar_wait(bar_full(s), (kb / kStages) & 1, abort_flag, 2);
                if (!ok) break;
                tc_fence_after();
                const uint64_t da = make_smem_desc(smem_base + s * kStageBytes), db = make_smem_desc(smem_base + s * kStageBytes + kPanelBytes);
#pragma unroll
                for (int ks = 0; ks < kBK / 16; ++ks)   // 32 bytes further along the 128-byte row per K step: +2 in the address field
                    umma_ss(tmem_base, da + 2 * ks, db + 2 * ks, p.idesc, (kb > 0 || ks > 0) ? 1u : 0u);
                tc_commit(bar_empty(s));
            }
            if (ok) tc_commit(bar_acc);
        }
    } else {
        // ------------------------------------------------------------------ epilogue: thread = row of the tile
        const int wq = warp & 3;                       // TMEM lanes 32 wq .. 32 wq + 31 belong to this warp
        const int row_in_tile = wq * 32 + lane;
        const int64_t row = m0 + row_in_tile;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(wq * 32) << 16);
        bool ok = true;
        if (lane == 0) ok = mbar_wait(bar_acc, 0, abort_flag, 3);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        tc_fence_after();
        if (ok) {
            if (EPI == kPlain) {
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    float v[32];
                    load_rounded<T>(t_row + c * 32, v);
                    if (row < p.m) store32<T>(static_cast<T*>(p.out) + row * p.n + n0 + c * 32, v);
                }
            } else if (EPI == kQkvPrologue) {
                // this tile is head `blockIdx.x` of the packed qkv row: q heads, then k heads, then v heads
                const int head = blockIdx.x;
                const bool is_q = head < p.hq, is_k = !is_q && head < p.hq + p.hkv;
                const bool live = row < p.m;
                const int pos = live ? __ldg(p.positions + row) : 0;
                const int64_t slot = live ? (p.slot_mapping != nullptr ? static_cast<int64_t>(__ldg(p.slot_mapping + row)) : row) : -1;
                T* dst = nullptr;
                if (live) {
                    if (is_q) dst = static_cast<T*>(p.q_out) + (row * p.hq + head) * kBN;
                    else if (slot >= 0 && slot < p.cache_rows)
                        dst = static_cast<T*>(is_k ? p.k_cache : p.v_cache) + (slot * p.hkv + (is_k ? head - p.hq : head - p.hq - p.hkv)) * kBN;
                }
                if (!is_q && !is_k) {                  // v heads: the rounded GEMM output as it is
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        float v[32];
                        load_rounded<T>(t_row + c * 32, v);
                        if (dst != nullptr) store32<T>(dst + c * 32, v);
                    }
                } else {
                    const bool normed = p.q_weight != nullptr;
                    float inv_rms = 1.0f;
                    if (normed) {                      // pass 1 over the accumulator: the head's sum of squares
                        float ss = 0.0f;
#pragma unroll 1
                        for (int c = 0; c < 4; ++c) {
                            float v[32];
                            load_rounded<T>(t_row + c * 32, v);
#pragma unroll
                            for (int i = 0; i < 32; ++i) ss += v[i] * v[i];
                        }
                        inv_rms = rsqrtf(ss / static_cast<float>(kBN) + p.eps);
                    }
                    const bool rotate = pos >= 0 && pos < p.max_positions;
                    const float* table = p.cos_sin + static_cast<int64_t>(rotate ? pos : 0) * kBN;
                    const T* weight = static_cast<const T*>(is_q ? p.q_weight : p.k_weight);
#pragma unroll 1
                    for (int c = 0; c < 2; ++c) {      // pass 2: columns [32 c, 32 c + 32) rotate with [64 + 32 c, 64 + 32 c + 32)
                        float lo[32], hi[32];
                        load_rounded<T>(t_row + c * 32, lo);
                        load_rounded<T>(t_row + 64 + c * 32, hi);
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            float a = lo[i], b = hi[i];
                            if (normed) {
                                a = a * inv_rms * ElemTraits<T>::to_float(weight[c * 32 + i]);
                                b = b * inv_rms * ElemTraits<T>::to_float(weight[64 + c * 32 + i]);
                            }
                            if (rotate) {              // first half: x cos - partner sin; second half: x cos + partner sin
                                const float cs = __ldg(table + c * 32 + i), sn = __ldg(table + 64 + c * 32 + i);
                                lo[i] = fmaf(a, cs, b * -sn);
                                hi[i] = fmaf(b, cs, a * sn);
                            } else {
                                lo[i] = a; hi[i] = b;
                            }
                        }
                        if (dst != nullptr) {
                            store32<T>(dst + c * 32, lo);
                            store32<T>(dst + 64 + c * 32, hi);
                        }
                    }
                }
            } else {   // kAllReducePush: every row of the partial sum goes to the rank that reduces it
                const uint32_t last = *reinterpret_cast<const volatile uint32_t*>(p.flags);
                const uint32_t epoch = last + 1u == 0u ? 1u : last + 1u;      // the epoch the all-reduce launch after this GEMM will use
                const bool poisoned = *reinterpret_cast<const volatile uint32_t*>(p.flags + 2) != 0u;
                const int64_t rows_per_rank = p.m / p.world;
                const int64_t row_vecs = p.n / 8, chunk_vecs = rows_per_rank * row_vecs;
                // (the TMEM loads are warp-collective: every lane runs them, only the stores depend on the row)
                const bool live = row < p.m && !poisoned;
                const int owner = live ? static_cast<int>(row / rows_per_rank) : p.rank;
                {
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        float v[32];
                        load_rounded<T>(t_row + c * 32, v);
                        if (!live) continue;
                        if (owner == p.rank) {
                            store32<T>(static_cast<T*>(p.addend) + row * p.n + n0 + c * 32, v);
                        } else {
                            uint4* slot = p.stage[owner] + 2 * (p.rank * chunk_vecs + (row - owner * rows_per_rank) * row_vecs + (n0 + c * 32) / 8);
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                uint4 w;
                                w.x = ElemTraits<T>::pack2(v[q * 8 + 0], v[q * 8 + 1]); w.y = ElemTraits<T>::pack2(v[q * 8 + 2], v[q * 8 + 3]);
                                w.z = ElemTraits<T>::pack2(v[q * 8 + 4], v[q * 8 + 5]); w.w = ElemTraits<T>::pack2(v[q * 8 + 6], v[q * 8 + 7]);
                                st_tagged(slot + 2 * q, w, epoch);
                            }
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
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
// [rows, k] 16-bit row-major -> boxes of 128 rows x 64 elements, 128-byte swizzle; rows past the end read as zeros
bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, bool bf16) {
    EncodeFn fn = encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
    const cuuint32_t box[2] = {kBK, kBM};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims,
              strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
uint32_t make_idesc(bool bf16) {   // kind::f16: D = F32, A / B = F16 or BF16 (both K-major), M 128, N 128
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(kBN >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
}

template <typename T, int EPI>
int launch(const void* a, const void* b, GemmParams& p, bool bf16, cudaStream_t stream, const char* what) {
    static bool attr_done[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 0 && device < 64 && !attr_done[device]) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<T, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "%s: cudaFuncSetAttribute: %s", what, cudaGetErrorString(e));
        attr_done[device] = true;
    }
    CUtensorMap ta, tb;
    if (!make_map(&ta, a, p.m, p.k, bf16) || !make_map(&tb, b, p.n, p.k, bf16))
        return fail(NVK_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed", what);
    p.idesc = make_idesc(bf16);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(p.n / kBN), static_cast<unsigned>((p.m + kBM - 1) / kBM));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<T, EPI>, ta, tb, p);
    if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
    return check_launch(what);
}

int check_gemm(const char* what, const void* a, const void* b, int64_t m, int64_t n, int64_t k, int dtype) {
    if (!a || !b) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: input and weight must be defined", what);
    if (dtype != NVK_F16 && dtype != NVK_BF16) return fail(NVK_ERR_UNSUPPORTED, "%s: dtype must be F16 or BF16", what);
    if (m <= 0 || n <= 0 || k <= 0) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: sizes must be positive", what);
    if (n % kBN != 0) return fail(NVK_ERR_UNSUPPORTED, "%s: the output width must be a multiple of %d", what, kBN);
    if (k % 8 != 0) return fail(NVK_ERR_UNSUPPORTED, "%s: the inner size must be a multiple of 8 (16-byte rows)", what);
    if (!aligned_to(a, 16) || !aligned_to(b, 16)) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: input and weight must be 16-byte aligned", what);
    if (m >= (1LL << 31) || n >= (1LL << 31) || (m + kBM - 1) / kBM > 65535) return fail(NVK_ERR_UNSUPPORTED, "%s: too large", what);
    if (encode_fn() == nullptr) return fail(NVK_ERR_UNSUPPORTED, "%s: cuTensorMapEncodeTiled is not available", what);
    return NVK_OK;
}

}  // namespace
}  // namespace nvk

using namespace nvk;

extern "C" int nvk_linear(const void* x, const void* weight, void* out, int64_t rows, int64_t out_features, int64_t in_features,
                          int dtype, void* stream) {
    const char* what = "linear";
    const int rc = check_gemm(what, x, weight, rows, out_features, in_features, dtype);
    if (rc != NVK_OK) return rc;
    if (!out || !aligned_to(out, 16)) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: the output must be defined and 16-byte aligned", what);
    GemmParams p{};
    p.out = out; p.m = rows; p.n = out_features; p.k = in_features;
    return dtype == NVK_BF16 ? launch<__nv_bfloat16, kPlain>(x, weight, p, true, static_cast<cudaStream_t>(stream), what)
                             : launch<__half, kPlain>(x, weight, p, false, static_cast<cudaStream_t>(stream), what);
}

extern "C" int nvk_qkv_linear_norm_rope_store(const void* x, const void* qkv_weight, int64_t rows, int64_t in_features,
                                              const int32_t* positions, const void* q_norm_weight, const void* k_norm_weight,
                                              float norm_eps, const float* cos_sin_cache, int64_t max_positions,
                                              const int32_t* slot_mapping, void* k_cache, void* v_cache, int64_t cache_rows,
                                              int num_q_heads, int num_kv_heads, int head_dim, void* q_out, int dtype, void* stream) {
    const char* what = "qkv linear + norm + rope + store";
    if (head_dim != kBN) return fail(NVK_ERR_UNSUPPORTED, "%s: head_dim must be %d (one GEMM tile per head)", what, kBN);
    if (num_q_heads <= 0 || num_kv_heads <= 0 || max_positions <= 0 || cache_rows <= 0)
        return fail(NVK_ERR_INVALID_ARGUMENT, "%s: sizes must be positive", what);
    const int64_t n = static_cast<int64_t>(num_q_heads + 2 * num_kv_heads) * head_dim;
    const int rc = check_gemm(what, x, qkv_weight, rows, n, in_features, dtype);
    if (rc != NVK_OK) return rc;
    if (!positions || !cos_sin_cache || !k_cache || !v_cache || !q_out)
        return fail(NVK_ERR_INVALID_ARGUMENT, "%s: positions, the rotary table, the caches and q_out must be defined", what);
    if ((q_norm_weight == nullptr) != (k_norm_weight == nullptr))
        return fail(NVK_ERR_INVALID_ARGUMENT, "%s: q_norm_weight and k_norm_weight go together", what);
    if (!aligned_to(q_out, 16) || !aligned_to(k_cache, 16) || !aligned_to(v_cache, 16))
        return fail(NVK_ERR_INVALID_ARGUMENT, "%s: q_out and the caches must be 16-byte aligned", what);
    GemmParams p{};
    p.m = rows; p.n = n; p.k = in_features;
    p.positions = positions; p.q_weight = q_norm_weight; p.k_weight = k_norm_weight; p.cos_sin = cos_sin_cache;
    p.slot_mapping = slot_mapping; p.q_out = q_out; p.k_cache = k_cache; p.v_cache = v_cache; p.cache_rows = cache_rows;
    p.max_positions = static_cast<int>(max_positions); p.hq = num_q_heads; p.hkv = num_kv_heads; p.eps = norm_eps;
    return dtype == NVK_BF16 ? launch<__nv_bfloat16, kQkvPrologue>(x, qkv_weight, p, true, static_cast<cudaStream_t>(stream), what)
                             : launch<__half, kQkvPrologue>(x, qkv_weight, p, false, static_cast<cudaStream_t>(stream), what);
}

namespace {
// The GEMM of a row-parallel linear on rank `rank`, its result rows delivered to the ranks that reduce them.
int launch_row_linear_push(const char* what, const void* x, const void* weight, int64_t rows, int64_t out_features, int64_t in_features,
                           void* addend, void* const* stage_ptrs, size_t stage_bytes, const void* flags, int rank, int world, int dtype,
                           cudaStream_t stream) {
    const int rc = check_gemm(what, x, weight, rows, out_features, in_features, dtype);
    if (rc != NVK_OK) return rc;
    if (world < 2 || world > kMaxRanks || rank < 0 || rank >= world)
        return fail(NVK_ERR_INVALID_ARGUMENT, "%s: world must be 2..%d and rank inside it", what, kMaxRanks);
    if (rows % world != 0) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: rows must be a multiple of world", what);
    if (!addend || !stage_ptrs || !flags || !aligned_to(addend, 16))
        return fail(NVK_ERR_INVALID_ARGUMENT, "%s: the addend buffer, the staging table and the flag area must be defined", what);
    if (stage_bytes < nvk_tp_allreduce_stage_bytes(rows * out_features))
        return fail(NVK_ERR_INVALID_ARGUMENT, "%s: staging areas of %zu bytes given, %zu needed", what, stage_bytes,
                    nvk_tp_allreduce_stage_bytes(rows * out_features));
    GemmParams p{};
    p.m = rows; p.n = out_features; p.k = in_features;
    p.addend = addend; p.flags = static_cast<const uint32_t*>(flags); p.rank = rank; p.world = world;
    for (int r = 0; r < world; ++r) {
        if (!stage_ptrs[r] || !aligned_to(stage_ptrs[r], 16)) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: bad staging area of rank %d", what, r);
        p.stage[r] = static_cast<uint4*>(stage_ptrs[r]);
    }
    return dtype == NVK_BF16 ? launch<__nv_bfloat16, kAllReducePush>(x, weight, p, true, stream, what)
                             : launch<__half, kAllReducePush>(x, weight, p, false, stream, what);
}
}  // namespace

extern "C" int nvk_tp_row_linear_allreduce_add_rmsnorm(const void* x, const void* weight, int64_t rows, int64_t out_features,
                                                       int64_t in_features, void* addend, void* out, void* norm,
                                                       void* const* stage_ptrs, size_t stage_bytes, void* flags, const void* residual,
                                                       const void* norm_weight, float eps, int rank, int world, int dtype, void* stream) {
    const char* what = "row-parallel linear + all-reduce + add + rmsnorm";
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (out_features > 8192) return fail(NVK_ERR_UNSUPPORTED, "%s: at most 8192 output features", what);
    int rc = launch_row_linear_push(what, x, weight, rows, out_features, in_features, addend, stage_ptrs, stage_bytes, flags, rank, world, dtype, st);
    if (rc != NVK_OK) return rc;
    return launch_allreduce_add_rmsnorm(addend, out, norm, stage_ptrs, stage_bytes, flags, residual, norm_weight, eps, rank, world,
                                        static_cast<int>(rows), static_cast<int>(out_features), dtype, /*pushed=*/true, st);
}

extern "C" int nvk_tp_row_linear_allreduce_add_rmsnorm_inprocess(const void* const* x_ptrs, const void* const* weight_ptrs, int64_t rows,
                                                                 int64_t out_features, int64_t in_features, void* const* addend_ptrs,
                                                                 void* const* out_ptrs, void* const* norm_ptrs, void* const* stage_ptrs,
                                                                 size_t stage_bytes, void* const* flag_ptrs,
                                                                 const void* const* residual_ptrs, const void* norm_weight, float eps,
                                                                 int world, int dtype, void* stream) {
    const char* what = "row-parallel linear + all-reduce + add + rmsnorm (in-process)";
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!x_ptrs || !weight_ptrs || !addend_ptrs || !flag_ptrs) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: pointer tables must be defined", what);
    if (world < 2 || world > kMaxRanks) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: world must be 2..%d", what, kMaxRanks);
    if (out_features > 8192) return fail(NVK_ERR_UNSUPPORTED, "%s: at most 8192 output features", what);
    for (int r = 0; r < world; ++r) {   // the ranks' GEMMs wait for nobody: one launch after the other
        const int rc = launch_row_linear_push(what, x_ptrs[r], weight_ptrs[r], rows, out_features, in_features, addend_ptrs[r], stage_ptrs,
                                              stage_bytes, flag_ptrs[r], r, world, dtype, st);
        if (rc != NVK_OK) return rc;
    }
    return launch_allreduce_inprocess(const_cast<const void* const*>(reinterpret_cast<void* const*>(addend_ptrs)), out_ptrs, norm_ptrs,
                                      stage_ptrs, stage_bytes, flag_ptrs, residual_ptrs, norm_weight, eps, world, static_cast<int>(rows),
                                      static_cast<int>(out_features), dtype, /*pushed=*/true, st);
}

extern "C" int nvk_gemm_status(void* stream, int* status) {
    if (!status) return fail(NVK_ERR_INVALID_ARGUMENT, "gemm status: null argument");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int word = 0;
    cudaError_t e = cudaMemcpyFromSymbolAsync(&word, g_gemm_error, sizeof(int), 0, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e == cudaSuccess && word != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbolAsync(g_gemm_error, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    }
    if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "gemm status: %s", cudaGetErrorString(e));
    *status = word;
    return NVK_OK;
}
