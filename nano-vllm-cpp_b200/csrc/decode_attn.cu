// Paged-KV decode attention for sm_100a (F16 / BF16, head_dim 128).
//
// Replaces decode_paged_attention_kernel (src/kernels/attention.cu:313-405 of the reference:
// one warp per (sequence, query head), every KV row re-read by each query head of its group,
// 8 dependent shuffles per key) and the FlashAttention-2 call it can dlopen
// (src/kernels/flash_attn.cpp:302-431).
//
// The op is HBM-bound: per sequence it must stream context_len * Hkv * D * 2 elements of K and V
// exactly once.  Design:
//   * one thread block per (KV head, split, sequence); the G = Hq / Hkv query heads of the group
//     are packed into the M dimension of the tensor-core tile, so each K/V row is read once;
//   * split-K with a FIXED grid (splits = ceil(max_blocks * block_size / chunk)) so that nothing
//     depends on host knowledge of context_lens (CUDA-graph safe); blocks whose chunk lies beyond
//     the context exit at once; partial (O, log-sum-exp) go to a workspace and a second small
//     kernel merges them;
//   * inside a block every warp streams its own 16-token tiles through a private ring of
//     cp.async stages (16-byte coalesced copies of the 256-byte head rows, XOR-swizzled in shared
//     memory) -- no block-wide barrier in the main loop, (kStages - 1) * 8 KiB in flight per warp;
//   * S = Q K^T as mma.sync m16n8k16 with the (zero padded) query heads as the 16 rows;
//     O^T = V^T P^T with V^T taken straight from the row-major V tile by ldmatrix.trans, so the
//     probability fragment of S is already in the layout the second MMA wants (no shuffles, no
//     shared-memory round trip); online softmax in the exp2 domain with warp shuffles.
#include "decode_body.cuh"

#include <atomic>
#include <cmath>
#include <utility>

#include <cuda_fp16.h>

namespace nvk {
namespace {

using namespace dec;   // constants, DecodeParams and decode_split_body: decode_body.cuh

// The decode kernels are launched with the programmatic-stream-serialization attribute: a kernel's blocks may be
// scheduled while its predecessor in the stream still runs, wait here until that predecessor has completed and its
// writes are visible (the first thing every block does, so nothing is read early), and at once allow their own
// successor the same head start.  In a decode graph of several hundred short kernels this hides launch latency.
__device__ __forceinline__ void pdl_wait_then_release() {
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}

// <<<grid, block, smem, stream>>> with that attribute.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 2) decode_split_kernel(const DecodeParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_blocks[kMaxChunkBlocks];
    pdl_wait_then_release();
    decode_split_body<T>(p, blockIdx.x, blockIdx.y, blockIdx.z, smem, s_blocks, threadIdx.x, 1);
}

// One warp per (sequence, query head): merges the live splits' (O, lse) pairs.
template <typename T>
__global__ void __launch_bounds__(128) decode_merge_kernel(const DecodeParams p, int64_t num_rows) {
    pdl_wait_then_release();
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    if (row >= num_rows) return;
    const int lane = threadIdx.x & 31;
    const int ctx = clamped_context(p, row / p.num_heads);
    const int live = (ctx + p.chunk_tokens - 1) / p.chunk_tokens;
    if (ctx <= 0 || live <= 1) return;  // already final
    const float* lse = p.ws_lse + row * p.num_splits;
    float mx = -INFINITY;
    for (int s = 0; s < live; ++s) mx = fmaxf(mx, lse[s]);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float wsum = 0.0f;
    for (int s = 0; s < live; ++s) {
        const float w = fast_exp2(lse[s] - mx);
        const float4 v = *reinterpret_cast<const float4*>(p.ws_o + (row * p.num_splits + s) * kHeadDim + lane * 4);
        acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
        wsum += w;
    }
    const float inv = 1.0f / wsum;
    T* dst = static_cast<T*>(p.out) + row * kHeadDim + lane * 4;
    uint2 packed;
    packed.x = ElemTraits<T>::pack2(acc.x * inv, acc.y * inv);
    packed.y = ElemTraits<T>::pack2(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(dst) = packed;
}

// ---------------------------------------------------------------------------------------------
// int8 KV cache (src/kernels/attention.cu:746-842 of the reference: decode_paged_attention_int8_kernel).
//
// Same block / split / merge structure as decode_split_kernel; what streams from HBM is half as wide:
// per token and KV head 128 int8 of K, 128 of V and two fp16 scales.  Each warp's cp.async ring carries
// the int8 tiles (16 tokens x 128 B for K, the same for V) and the MMA fragments are built from them in
// registers -- no widened copy in shared memory, no ldmatrix:
//   * an int8 x becomes the fp16 number 1024 + (x + 128) by gluing the byte (x ^ 0x80) under the exponent
//     byte 0x64 (one PRMT per pair); the constant 1152 is taken out afterwards: q . (k' - 1152) =
//     q . k' - 1152 * sum(q), and P (v' - 1152) = P v' - 1152 * sum(P), where sum(P) comes from one extra
//     MMA per tile against a row of ones, i.e. from exactly the rounded probabilities the other MMAs used;
//   * the MMAs contract over d (scores) and over keys (output); a contraction does not care in which order
//     its index runs, and neither does the output care which accumulator row holds which d, so every lane
//     takes whole 16-byte pieces: for K, piece 4q + t of key row g supplies its k-steps 4q .. 4q + 3 (the
//     query fragment is loaded with the same permutation); for V, piece g of key rows 2t, 2t+1, 2t+8, 2t+9
//     supplies all eight d-tiles after a byte interleave of row pairs (two PRMTs), and accumulator row g /
//     g + 8 of d-tile 2a + e holds d = 16 g + 4 a + 2 e (+ 1);
//   * pieces are XOR-swizzled in the ring so that those 16-byte reads are conflict free.
// The scales never touch the tiles: k_scale multiplies the score of its key after the first MMA, v_scale
// the probability of its key before the second (the row sum uses the unscaled probability).  They are
// fetched two tiles ahead into registers by lanes 0-15 (K) and 16-31 (V).  MMAs run as f16 whatever the
// query type: the query is converted once, probabilities are <= 1.
// ---------------------------------------------------------------------------------------------
constexpr int kRowBytesI8 = kHeadDim;                      // one head row of int8 K or V
constexpr int kTileBytesI8 = kTileTokens * kRowBytesI8;    // 2 KiB
constexpr int kScaleBytesI8 = 2 * kTileTokens * 4;         // one 32-bit word per (K | V, token): the word that holds its fp16 scale
constexpr int kStageBytesI8 = 2 * kTileBytesI8 + kScaleBytesI8;   // K + V + scales
constexpr int kStagesI8 = 4;                               // tiles in flight per warp: kStagesI8 - 1
constexpr int kWarpBytesI8 = kStagesI8 * kStageBytesI8;    // 16.5 KiB
constexpr int kSmemBytesI8 = kWarps * kWarpBytesI8;        // 66 KiB -> three blocks per SM
constexpr float kI8Offset = 1152.0f;                       // 1024 (exponent glue) + 128 (sign flip)

__device__ __forceinline__ uint32_t lds32x4(uint32_t addr, uint32_t (&w)[4]) {
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(addr));
    return 0;
}

__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

struct DecodeInt8Params {
    DecodeParams base;
    const __half* k_scale; const __half* v_scale;
};

// Two 8-bit cache elements -> two f16 (MMA operand halves).  int8: the byte glued under the exponent byte of 1024 (the word has
// had its sign bits flipped: value + 1152, taken out algebraically afterwards); e4m3: the hardware conversion, exact.
template <bool FP8> __device__ __forceinline__ uint32_t widen_pair_lo(uint32_t x) {   // bytes 0, 1
    if constexpr (FP8) {
        uint32_t d;
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(d) : "h"(static_cast<unsigned short>(x & 0xffffu)));
        return d;
    } else {
        return __byte_perm(x, 0x64646464u, 0x4140);
    }
}
template <bool FP8> __device__ __forceinline__ uint32_t widen_pair_hi(uint32_t x) {   // bytes 2, 3
    if constexpr (FP8) {
        uint32_t d;
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(d) : "h"(static_cast<unsigned short>(x >> 16)));
        return d;
    } else {
        return __byte_perm(x, 0x64646464u, 0x4342);
    }
}

// FP8 = false: int8 cache (the reference's format); FP8 = true: e4m3 cache of the same layout.
template <typename T, bool FP8>
__global__ void __launch_bounds__(kThreads, 3) decode_split_int8_kernel(const DecodeInt8Params pp) {
    const DecodeParams& p = pp.base;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_blocks[kMaxChunkBlocks];
    pdl_wait_then_release();

    const int kvh = blockIdx.x;
    const int split = blockIdx.y;
    const int64_t b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int G = p.group;

    const int ctx = clamped_context(p, b);
    const int t0 = split * p.chunk_tokens;
    T* out = static_cast<T*>(p.out);
    if (ctx <= 0) {
        if (split == 0) {
            for (int i = tid; i < G * kHeadDim; i += kThreads)
                out[(b * p.num_heads + kvh * G) * kHeadDim + i] = ElemTraits<T>::from_float(0.0f);
        }
        return;
    }
    if (t0 >= ctx) return;
    const int t1 = min(ctx, t0 + p.chunk_tokens);
    const int live_splits = (ctx + p.chunk_tokens - 1) / p.chunk_tokens;

    const int blk0 = t0 / p.block_size;
    const int nblk = (t1 - 1) / p.block_size - blk0 + 1;
    for (int i = tid; i < nblk; i += kThreads) {
        const int64_t id = p.block_tables[b * p.max_blocks + blk0 + i];
        s_blocks[i] = (id >= 0 && id < p.num_cache_blocks) ? static_cast<int>(id) : -1;
    }
    __syncthreads();

    // Query fragments as f16, rows g < G of the 16-row A tile (rows 8..15 are zero), in the K permutation:
    // k-step ks = 4 q + w, positions {2t, 2t+1 | 2t+8, 2t+9} <- d = 64 q + 16 t + 4 w + {0, 1 | 2, 3}.
    uint32_t qa[8][2];
    float qsum = 0.0f;   // sum over d of the (f16-rounded) query row g
    {
        const T* qrow = static_cast<const T*>(p.q) + (b * p.num_heads + kvh * G + (g < G ? g : 0)) * kHeadDim;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const int d0 = 64 * (ks >> 2) + 16 * t + 4 * (ks & 3);
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
                const __half2 h2 = __floats2half2_rn(ElemTraits<T>::to_float(qrow[d0 + 2 * hlf]), ElemTraits<T>::to_float(qrow[d0 + 2 * hlf + 1]));
                qa[ks][hlf] = g < G ? *reinterpret_cast<const uint32_t*>(&h2) : 0u;
                if (g < G) qsum += __low2float(h2) + __high2float(h2);
            }
        }
        qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
        qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
    }
    const float q_off = FP8 ? 0.0f : kI8Offset * qsum;
    constexpr uint32_t kFlip = FP8 ? 0u : 0x80808080u;   // int8: sign bits flipped before the glue

    const uint32_t ring_u32 = smem_u32(smem + warp * kWarpBytesI8);
    const int num_tiles = (t1 - t0 + kTileTokens - 1) / kTileTokens;
    const int my_tiles = num_tiles > warp ? (num_tiles - warp + kWarps - 1) / kWarps : 0;
    const size_t row_stride = static_cast<size_t>(p.num_kv_heads) * kRowBytesI8;   // bytes between tokens
    const unsigned char* kc = static_cast<const unsigned char*>(p.k_cache) + static_cast<size_t>(kvh) * kRowBytesI8;
    const unsigned char* vc = static_cast<const unsigned char*>(p.v_cache) + static_cast<size_t>(kvh) * kRowBytesI8;

    // Copy pattern: 16-byte piece c of rows r = 4 i + (lane >> 3), i = 0..3.  Ring swizzles: K piece c of row r sits at
    // c ^ ((r & 1) << 2), V piece c of row r at c ^ (r & 6).
    const int c = lane & 7, rq = lane >> 3;

    auto issue = [&](int j) {
        if (j < my_tiles) {
            const int tok0 = t0 + (warp + j * kWarps) * kTileTokens;
            const int blk = tok0 / p.block_size;
            const int phys = s_blocks[blk - blk0];
            const int off = tok0 - blk * p.block_size;
            const size_t base = (static_cast<size_t>(phys < 0 ? 0 : phys) * p.block_size + off) * row_stride + c * 16;
            const uint32_t stage = ring_u32 + (j % kStagesI8) * kStageBytesI8;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = 4 * i + rq;
                const int bytes = (phys >= 0 && tok0 + r < t1) ? 16 : 0;
                const size_t src = base + (bytes ? r * row_stride : 0);
                cp_async16(stage + r * kRowBytesI8 + ((c ^ ((r & 1) << 2)) << 4), kc + src, bytes);
                cp_async16(stage + kTileBytesI8 + r * kRowBytesI8 + ((c ^ (r & 6)) << 4), vc + src, bytes);
            }
            // the scale of token (lane & 15): lanes 0-15 K, lanes 16-31 V; copied as the aligned 32-bit word around it
            const int tr = lane & 15;
            const int sbytes = (phys >= 0 && tok0 + tr < t1) ? 4 : 0;
            const size_t sidx = sbytes ? ((static_cast<size_t>(phys) * p.block_size + off + tr) * p.num_kv_heads + kvh) : 0;
            const __half* sbase = lane < 16 ? pp.k_scale : pp.v_scale;
            cp_async4(stage + 2 * kTileBytesI8 + lane * 4, sbase + (sidx & ~static_cast<size_t>(1)), sbytes);
        }
        cp_async_commit();
    };
    // which half of the copied word is this lane's scale: cache rows of a tile start at an even row, so the parity of
    // row * Hkv + kvh is that of (token & Hkv & 1) + kvh
    const bool scale_hi = (((lane & p.num_kv_heads) ^ kvh) & 1) != 0;
    const float scale_mul = lane < 16 ? p.scale_log2 : 1.0f;   // the softmax scale rides on the K scale

    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float osum[4] = {0.f, 0.f, 0.f, 0.f};   // sum of the (scaled, rounded) probabilities per head, from the ones-row MMA
    float m_run = -INFINITY, l_run = 0.0f;

#pragma unroll
    for (int s = 0; s < kStagesI8 - 1; ++s) issue(s);

    constexpr uint32_t kOnes = 0x3C003C00u;   // {1.0, 1.0}

    for (int j = 0; j < my_tiles; ++j) {
        issue(j + kStagesI8 - 1);
        cp_async_wait<kStagesI8 - 1>();
        __syncwarp();
        const uint32_t stage = ring_u32 + (j % kStagesI8) * kStageBytesI8;
        const int tok0 = t0 + (warp + j * kWarps) * kTileTokens;
        float sc_cur;
        {
            uint32_t word;
            asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(word) : "r"(stage + 2 * kTileBytesI8 + lane * 4));
            const __half2 pair = *reinterpret_cast<const __half2*>(&word);
            sc_cur = (scale_hi ? __high2float(pair) : __low2float(pair)) * scale_mul;
        }

        // ---- scores: keys g (n-tile 0) and g + 8 (n-tile 1)
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            uint32_t w0[4], w1[4];
            lds32x4(stage + g * kRowBytesI8 + (((4 * q + t) ^ ((g & 1) << 2)) << 4), w0);
            lds32x4(stage + (g + 8) * kRowBytesI8 + (((4 * q + t) ^ ((g & 1) << 2)) << 4), w1);
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                const int ks = 4 * q + wi;
                const uint32_t x0 = w0[wi] ^ kFlip, x1 = w1[wi] ^ kFlip;
                mma_16816<__half>(s0, qa[ks][0], 0u, qa[ks][1], 0u, widen_pair_lo<FP8>(x0), widen_pair_hi<FP8>(x0));
                mma_16816<__half>(s1, qa[ks][0], 0u, qa[ks][1], 0u, widen_pair_lo<FP8>(x1), widen_pair_hi<FP8>(x1));
            }
        }
        // scores of head g: tokens tok0 + {2t, 2t+1, 8+2t, 9+2t}; remove the offset, apply each key's K scale
        const float ks0 = __shfl_sync(0xffffffffu, sc_cur, 2 * t), ks1 = __shfl_sync(0xffffffffu, sc_cur, 2 * t + 1);
        const float ks2 = __shfl_sync(0xffffffffu, sc_cur, 8 + 2 * t), ks3 = __shfl_sync(0xffffffffu, sc_cur, 9 + 2 * t);
        const float vs0 = __shfl_sync(0xffffffffu, sc_cur, 16 + 2 * t), vs1 = __shfl_sync(0xffffffffu, sc_cur, 17 + 2 * t);
        const float vs2 = __shfl_sync(0xffffffffu, sc_cur, 24 + 2 * t), vs3 = __shfl_sync(0xffffffffu, sc_cur, 25 + 2 * t);
        float sc[4];
        sc[0] = (s0[0] - q_off) * ks0; sc[1] = (s0[1] - q_off) * ks1;
        sc[2] = (s1[0] - q_off) * ks2; sc[3] = (s1[1] - q_off) * ks3;
        if (tok0 + kTileTokens > t1) {   // only a chunk's last tile can reach past its end (warp-uniform)
            const int tk = tok0 + 2 * t;
            if (tk >= t1) sc[0] = -INFINITY;
            if (tk + 1 >= t1) sc[1] = -INFINITY;
            if (tk + 8 >= t1) sc[2] = -INFINITY;
            if (tk + 9 >= t1) sc[3] = -INFINITY;
        }
        float m_tile = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 1));
        m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 2));
        // The running maximum of a head moves on a handful of tiles only; the 36 accumulator multiplies are skipped
        // on all the others (warp-uniform branch).
        if (__any_sync(0xffffffffu, m_tile > m_run)) {
            const float m_new = fmaxf(m_run, m_tile);   // finite: token tok0 is always valid
            const float corr = fast_exp2(m_run - m_new);
            l_run *= corr;
            m_run = m_new;
            const float c0 = __shfl_sync(0xffffffffu, corr, 8 * t);
            const float c1 = __shfl_sync(0xffffffffu, corr, 8 * t + 4);
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) { o[mt][0] *= c0; o[mt][1] *= c1; o[mt][2] *= c0; o[mt][3] *= c1; }
            osum[0] *= c0; osum[1] *= c1; osum[2] *= c0; osum[3] *= c1;
        }
        const float p0 = fast_exp2(sc[0] - m_run), p1 = fast_exp2(sc[1] - m_run);
        const float p2 = fast_exp2(sc[2] - m_run), p3 = fast_exp2(sc[3] - m_run);
        l_run += (p0 + p1) + (p2 + p3);
        const uint32_t pb0 = ElemTraits<__half>::pack2(p0 * vs0, p1 * vs1);
        const uint32_t pb1 = ElemTraits<__half>::pack2(p2 * vs2, p3 * vs3);

        // ---- output: V rows 2t, 2t+1, 2t+8, 2t+9, piece g (d = 16 g .. 16 g + 15)
        uint32_t v0[4], v1[4], v2[4], v3[4];
        const uint32_t vbase = stage + kTileBytesI8;
        lds32x4(vbase + (2 * t) * kRowBytesI8 + ((g ^ ((2 * t) & 6)) << 4), v0);
        lds32x4(vbase + (2 * t + 1) * kRowBytesI8 + ((g ^ ((2 * t + 1) & 6)) << 4), v1);
        lds32x4(vbase + (2 * t + 8) * kRowBytesI8 + ((g ^ ((2 * t + 8) & 6)) << 4), v2);
        lds32x4(vbase + (2 * t + 9) * kRowBytesI8 + ((g ^ ((2 * t + 9) & 6)) << 4), v3);
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const uint32_t x0 = v0[a] ^ kFlip, x1 = v1[a] ^ kFlip, x2 = v2[a] ^ kFlip, x3 = v3[a] ^ kFlip;
            // bytes of one d from two consecutive keys, side by side
            const uint32_t lo01 = __byte_perm(x0, x1, 0x5140), hi01 = __byte_perm(x0, x1, 0x7362);
            const uint32_t lo23 = __byte_perm(x2, x3, 0x5140), hi23 = __byte_perm(x2, x3, 0x7362);
            float (&oe)[4] = o[2 * a];
            float (&oo)[4] = o[2 * a + 1];
            mma_16816<__half>(oe, widen_pair_lo<FP8>(lo01), widen_pair_hi<FP8>(lo01), widen_pair_lo<FP8>(lo23), widen_pair_hi<FP8>(lo23), pb0, pb1);
            mma_16816<__half>(oo, widen_pair_lo<FP8>(hi01), widen_pair_hi<FP8>(hi01), widen_pair_lo<FP8>(hi23), widen_pair_hi<FP8>(hi23), pb0, pb1);
        }
        if (!FP8) mma_16816<__half>(osum, kOnes, kOnes, kOnes, kOnes, pb0, pb1);
        __syncwarp();   // the stage is refilled two iterations from now by other lanes' copies
    }
    cp_async_wait<0>();
    __syncthreads();  // every ring is idle from here on: reuse the shared memory for the cross-warp merge

    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);

    float* sm_o = reinterpret_cast<float*>(smem);                    // [warp][head][128]
    float* sm_m = sm_o + kWarps * kMaxGroup * kHeadDim;              // [warp][head]
    float* sm_l = sm_m + kWarps * kMaxGroup;
    if (t == 0) { sm_m[warp * kMaxGroup + g] = m_run; sm_l[warp * kMaxGroup + g] = l_run; }
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
        // accumulator rows g / g + 8 of d-tile mt = 2 a + e hold d = 16 g + 4 a + 2 e (+ 1); columns are heads 2t, 2t + 1
        const int d = 16 * g + 4 * (mt >> 1) + 2 * (mt & 1);
        float* dst = sm_o + (warp * kMaxGroup + 2 * t) * kHeadDim + d;
        const float off = FP8 ? 0.0f : kI8Offset;
        dst[0] = o[mt][0] - off * osum[0];
        dst[kHeadDim] = o[mt][1] - off * osum[1];
        dst[1] = o[mt][2] - off * osum[0];
        dst[kHeadDim + 1] = o[mt][3] - off * osum[1];
    }
    __syncthreads();

    const int d = tid;
    for (int h = 0; h < G; ++h) {
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) mx = fmaxf(mx, sm_m[w * kMaxGroup + h]);
        float acc = 0.0f, lsum = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float f = fast_exp2(sm_m[w * kMaxGroup + h] - mx);
            acc += f * sm_o[(w * kMaxGroup + h) * kHeadDim + d];
            lsum += f * sm_l[w * kMaxGroup + h];
        }
        const float val = acc / lsum;
        const int64_t head = b * p.num_heads + kvh * G + h;
        if (live_splits == 1) {
            out[head * kHeadDim + d] = ElemTraits<T>::from_float(val);
        } else {
            p.ws_o[(head * p.num_splits + split) * kHeadDim + d] = val;
            if (d == 0) p.ws_lse[head * p.num_splits + split] = mx + log2f(lsum);
        }
    }
}

// Split policy from host-known sizes only.  Returns chunk length in tokens (multiple of block_size).
int choose_chunk_tokens(int64_t batch, int num_kv_heads, int64_t max_blocks, int block_size, bool have_workspace) {
    const int64_t max_tokens = max_blocks * block_size;
    if (!have_workspace) return static_cast<int>(max_tokens);
    int64_t chunk = 2048;                         // longest chunk we ever use
    // Split only while there is less than one block per SM: a split costs a second pass over its partial results in the merge
    // kernel, and at the per-rank shapes of a tensor-parallel decoder (batch 256, one KV head, 2048-token tables) the unsplit
    // grid measured 29 us per call against 36 us with chunks of 256 tokens.
    const int64_t want_blocks = 148;
    while (chunk > 256 && batch * num_kv_heads * ((max_tokens + chunk - 1) / chunk) < want_blocks) chunk >>= 1;
    // whole cache blocks per chunk
    int64_t per = (chunk + block_size - 1) / block_size;
    if (per < 1) per = 1;
    chunk = per * block_size;
    if (chunk > max_tokens) chunk = max_tokens;
    return static_cast<int>(chunk);
}

}  // namespace

// Kernel parameters of a split-K decode call from host-known sizes only: chunk length, split count, scratch layout.
int decode_plan(const DecodeArgs& a, dec::DecodeParams* out) {
    DecodeParams p{};
    p.q = a.q; p.k_cache = a.k_cache; p.v_cache = a.v_cache;
    p.context_lens = a.context_lens; p.block_tables = a.block_tables; p.out = a.out;
    p.max_blocks = a.max_blocks; p.num_cache_blocks = a.num_cache_blocks;
    p.num_heads = a.num_heads; p.num_kv_heads = a.num_kv_heads; p.group = a.num_heads / a.num_kv_heads;
    p.block_size = a.block_size;
    p.scale_log2 = a.scale * kLog2e;

    const size_t need = decode_mma_workspace_bytes(a.batch, a.num_heads, a.num_kv_heads, a.head_dim, a.max_blocks, a.block_size);
    bool have_ws = a.workspace != nullptr && a.workspace_bytes >= need && aligned_to(a.workspace, 16);
    p.chunk_tokens = choose_chunk_tokens(a.batch, a.num_kv_heads, a.max_blocks, a.block_size, have_ws);
    if (p.chunk_tokens / a.block_size > kMaxChunkBlocks) {
        // a chunk may cover at most kMaxChunkBlocks cache blocks
        if (!have_ws) return fail(NVK_ERR_UNSUPPORTED, "decode attention: max_blocks %lld needs a workspace", (long long)a.max_blocks);
        p.chunk_tokens = kMaxChunkBlocks * a.block_size;
    }
    const int64_t max_tokens = a.max_blocks * a.block_size;
    p.num_splits = static_cast<int>((max_tokens + p.chunk_tokens - 1) / p.chunk_tokens);
    if (p.num_splits > 1) {
        p.ws_lse = static_cast<float*>(a.workspace);
        const size_t lse_bytes = (static_cast<size_t>(a.batch) * a.num_heads * p.num_splits * sizeof(float) + 15) / 16 * 16;
        p.ws_o = reinterpret_cast<float*>(static_cast<unsigned char*>(a.workspace) + lse_bytes);
    }
    if (a.batch > 65535 || p.num_splits > 65535) return fail(NVK_ERR_UNSUPPORTED, "decode attention: batch or split count exceeds grid limits");
    *out = p;
    return NVK_OK;
}

// The merge of the live splits' partial results (nothing to do when the plan has a single split).
int launch_decode_merge(const dec::DecodeParams& p, int64_t batch, int dtype, cudaStream_t stream) {
    if (p.num_splits <= 1) return NVK_OK;
    const int64_t rows = batch * p.num_heads;
    const cudaError_t le = dtype == NVK_BF16
        ? launch_pdl(decode_merge_kernel<__nv_bfloat16>, dim3(static_cast<unsigned>((rows + 3) / 4)), dim3(128), 0, stream, p, rows)
        : launch_pdl(decode_merge_kernel<__half>, dim3(static_cast<unsigned>((rows + 3) / 4)), dim3(128), 0, stream, p, rows);
    if (le != cudaSuccess) return fail(NVK_ERR_CUDA, "decode_merge_kernel launch: %s", cudaGetErrorString(le));
    return check_launch("decode_merge_kernel launch");
}

namespace {

template <typename T>
int launch_typed(const DecodeArgs& a) {
    static bool attr_done[64] = {};  // per device; the attribute call is idempotent
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 0 && device < 64 && !attr_done[device]) {
        const cudaError_t e = cudaFuncSetAttribute(decode_split_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "decode attention: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        attr_done[device] = true;
    }
    DecodeParams p{};
    int rc0 = decode_plan(a, &p);
    if (rc0 != NVK_OK) return rc0;
    const dim3 grid(a.num_kv_heads, p.num_splits, static_cast<unsigned>(a.batch));
    cudaError_t le = launch_pdl(decode_split_kernel<T>, grid, dim3(kThreads), kSmemBytes, a.stream, p);
    if (le != cudaSuccess) return fail(NVK_ERR_CUDA, "decode_split_kernel launch: %s", cudaGetErrorString(le));
    int rc = check_launch("decode_split_kernel launch");
    if (rc != NVK_OK) return rc;
    if (p.num_splits > 1) {
        const int64_t rows = a.batch * a.num_heads;
        le = launch_pdl(decode_merge_kernel<T>, dim3(static_cast<unsigned>((rows + 3) / 4)), dim3(128), 0, a.stream, p, rows);
        if (le != cudaSuccess) return fail(NVK_ERR_CUDA, "decode_merge_kernel launch: %s", cudaGetErrorString(le));
        rc = check_launch("decode_merge_kernel launch");
    }
    return rc;
}

template <typename T, bool FP8>
int launch_int8_typed(const DecodeInt8Args& x) {
    const DecodeArgs& a = x.base;
    static bool attr_done[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 0 && device < 64 && !attr_done[device]) {
        const cudaError_t e = cudaFuncSetAttribute(decode_split_int8_kernel<T, FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytesI8);
        if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "decode attention (int8): cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        attr_done[device] = true;
    }
    DecodeInt8Params pp{};
    DecodeParams& p = pp.base;
    pp.k_scale = static_cast<const __half*>(x.k_scale); pp.v_scale = static_cast<const __half*>(x.v_scale);
    p.q = a.q; p.k_cache = a.k_cache; p.v_cache = a.v_cache;
    p.context_lens = a.context_lens; p.block_tables = a.block_tables; p.out = a.out;
    p.max_blocks = a.max_blocks; p.num_cache_blocks = a.num_cache_blocks;
    p.num_heads = a.num_heads; p.num_kv_heads = a.num_kv_heads; p.group = a.num_heads / a.num_kv_heads;
    p.block_size = a.block_size;
    p.scale_log2 = a.scale * kLog2e;
    const size_t need = decode_mma_workspace_bytes(a.batch, a.num_heads, a.num_kv_heads, a.head_dim, a.max_blocks, a.block_size);
    const bool have_ws = a.workspace != nullptr && a.workspace_bytes >= need && aligned_to(a.workspace, 16);
    p.chunk_tokens = choose_chunk_tokens(a.batch, a.num_kv_heads, a.max_blocks, a.block_size, have_ws);
    if (p.chunk_tokens / a.block_size > kMaxChunkBlocks) {
        if (!have_ws) return fail(NVK_ERR_UNSUPPORTED, "decode attention (int8): max_blocks %lld needs a workspace", (long long)a.max_blocks);
        p.chunk_tokens = kMaxChunkBlocks * a.block_size;
    }
    const int64_t max_tokens = a.max_blocks * a.block_size;
    p.num_splits = static_cast<int>((max_tokens + p.chunk_tokens - 1) / p.chunk_tokens);
    if (p.num_splits > 1) {
        p.ws_lse = static_cast<float*>(a.workspace);
        const size_t lse_bytes = (static_cast<size_t>(a.batch) * a.num_heads * p.num_splits * sizeof(float) + 15) / 16 * 16;
        p.ws_o = reinterpret_cast<float*>(static_cast<unsigned char*>(a.workspace) + lse_bytes);
    }
    if (a.batch > 65535 || p.num_splits > 65535) return fail(NVK_ERR_UNSUPPORTED, "decode attention (int8): batch or split count exceeds grid limits");
    const dim3 grid(a.num_kv_heads, p.num_splits, static_cast<unsigned>(a.batch));
    cudaError_t le = launch_pdl(decode_split_int8_kernel<T, FP8>, grid, dim3(kThreads), kSmemBytesI8, a.stream, pp);
    if (le != cudaSuccess) return fail(NVK_ERR_CUDA, "decode_split_int8_kernel launch: %s", cudaGetErrorString(le));
    int rc = check_launch("decode_split_int8_kernel launch");
    if (rc != NVK_OK) return rc;
    if (p.num_splits > 1) {
        const int64_t rows = a.batch * a.num_heads;
        le = launch_pdl(decode_merge_kernel<T>, dim3(static_cast<unsigned>((rows + 3) / 4)), dim3(128), 0, a.stream, p, rows);
        if (le != cudaSuccess) return fail(NVK_ERR_CUDA, "decode_merge_kernel launch: %s", cudaGetErrorString(le));
        rc = check_launch("decode_merge_kernel launch");
    }
    return rc;
}

}  // namespace

bool decode_mma_supported(const DecodeArgs& a) {
    if (a.dtype != NVK_F16 && a.dtype != NVK_BF16) return false;
    if (a.head_dim != kHeadDim) return false;
    if (a.num_kv_heads <= 0 || a.num_heads % a.num_kv_heads != 0) return false;
    if (a.num_heads / a.num_kv_heads > kMaxGroup) return false;
    if (a.block_size < kTileTokens || a.block_size % kTileTokens != 0) return false;
    if (!aligned_to(a.q, 4) || !aligned_to(a.k_cache, 16) || !aligned_to(a.v_cache, 16) || !aligned_to(a.out, 8)) return false;
    if (a.workspace == nullptr && a.max_blocks > kMaxChunkBlocks) return false;
    return true;
}

size_t decode_mma_workspace_bytes(int64_t batch, int num_heads, int num_kv_heads, int head_dim,
                                  int64_t max_blocks, int block_size) {
    if (batch <= 0 || num_heads <= 0 || num_kv_heads <= 0 || max_blocks <= 0 || block_size <= 0) return 0;
    int chunk = choose_chunk_tokens(batch, num_kv_heads, max_blocks, block_size, true);
    if (chunk / block_size > kMaxChunkBlocks) chunk = kMaxChunkBlocks * block_size;
    const int64_t splits = (max_blocks * block_size + chunk - 1) / chunk;
    if (splits <= 1) return 0;
    const size_t rows = static_cast<size_t>(batch) * num_heads * splits;
    const size_t lse_bytes = (rows * sizeof(float) + 15) / 16 * 16;
    return lse_bytes + rows * static_cast<size_t>(head_dim) * sizeof(float);
}

bool decode_int8_mma_supported(const DecodeInt8Args& x) {
    const DecodeArgs& a = x.base;
    if (a.dtype != NVK_F16 && a.dtype != NVK_BF16) return false;
    if (a.head_dim != kHeadDim) return false;
    if (a.num_kv_heads <= 0 || a.num_heads % a.num_kv_heads != 0) return false;
    if (a.num_heads / a.num_kv_heads > kMaxGroup) return false;
    if (a.block_size < kTileTokens || a.block_size % kTileTokens != 0) return false;
    if (!aligned_to(a.q, 2) || !aligned_to(a.k_cache, 16) || !aligned_to(a.v_cache, 16) || !aligned_to(a.out, 8)) return false;
    if (!aligned_to(x.k_scale, 4) || !aligned_to(x.v_scale, 4)) return false;   // scales are copied as aligned 32-bit words
    if ((a.num_cache_blocks * a.block_size * a.num_kv_heads) % 2 != 0) return false;
    if (a.workspace == nullptr && a.max_blocks > kMaxChunkBlocks) return false;
    return true;
}

int launch_decode_int8_mma(const DecodeInt8Args& x) {
    if (x.fp8) return x.base.dtype == NVK_BF16 ? launch_int8_typed<__nv_bfloat16, true>(x) : launch_int8_typed<__half, true>(x);
    return x.base.dtype == NVK_BF16 ? launch_int8_typed<__nv_bfloat16, false>(x) : launch_int8_typed<__half, false>(x);
}

int launch_decode_mma(const DecodeArgs& a) {
    return a.dtype == NVK_BF16 ? launch_typed<__nv_bfloat16>(a) : launch_typed<__half>(a);
}

}  // namespace nvk

// ---------------------------------------------------------------------------------------------
// Allocation-free variant: split-K scratch in a fixed device array owned by this library.
//
// Some callers of decode attention have no way to hand over a workspace: the reference's own
// launch_decode_attention_paged signature carries no allocator, an engine may already have given
// every free byte of HBM to its KV-cache pool, and code running under a "no device allocation
// after start-up" rule (latency-critical serving loops, plug-ins that are only handed tensors)
// must not call cudaMalloc at all.  For them the split-K partials live in the array below.  It is
// part of the loaded module, so every GPU that uses this library keeps kStaticScratchBytes of HBM
// reserved until the process exits.
// ---------------------------------------------------------------------------------------------
namespace nvk {
namespace {

constexpr size_t kStaticScratchBytes = 32u << 20;  // 32 MiB: batch 256 x 32 heads x 4 splits needs 16.9 MB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_scratch_addr[kMaxDevices];   // null until the first call on that device (static storage: zeroed)

// Resolves the device address of g_static_scratch for the current device (once per device).
// In host code the symbol's name is only a handle; the kernels need the address returned here.
int static_scratch_for_current_device(void** out) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "decode attention (static scratch): cudaGetDevice: %s", cudaGetErrorString(e));
    if (device < 0 || device >= kMaxDevices)
        return fail(NVK_ERR_UNSUPPORTED, "decode attention (static scratch): device index %d not supported", device);
    void* ptr = g_scratch_addr[device].load(std::memory_order_acquire);
    if (ptr == nullptr) {   // two threads racing here both look the same address up; either store is fine
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return fail(NVK_ERR_CUDA, "decode attention (static scratch): cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_scratch_addr[device].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return NVK_OK;
}

}  // namespace
}  // namespace nvk

extern "C" size_t nvk_decode_attention_static_scratch_bytes(void) { return nvk::kStaticScratchBytes; }

extern "C" int nvk_decode_attention_paged_static(const void* query, const void* k_cache, const void* v_cache,
                                                 const void* context_lens, int context_lens_dtype,
                                                 const void* block_tables, int block_tables_dtype,
                                                 int64_t batch, int64_t max_blocks, int64_t num_cache_blocks,
                                                 int num_heads, int num_kv_heads, int head_dim, int block_size,
                                                 float scale, void* output, int dtype, void* stream) {
    using namespace nvk;
    const size_t need = nvk_decode_attention_workspace_bytes(batch, num_heads, num_kv_heads, head_dim, max_blocks, block_size);
    if (need > kStaticScratchBytes)
        return fail(NVK_ERR_INVALID_ARGUMENT,
                    "decode attention (static scratch): this problem needs %zu bytes of split-K scratch but the built-in "
                    "array holds %zu; use nvk_decode_attention_paged with a caller-provided workspace",
                    need, kStaticScratchBytes);
    void* scratch = nullptr;
    const int rc = static_scratch_for_current_device(&scratch);
    if (rc != NVK_OK) return rc;
    // The partials of a split are fully written before the merge kernel reads them, and only live
    // splits are read, so nothing in the array has to start at zero.
    return nvk_decode_attention_paged(query, k_cache, v_cache, context_lens, context_lens_dtype, block_tables,
                                      block_tables_dtype, batch, max_blocks, num_cache_blocks, num_heads, num_kv_heads, head_dim, block_size, scale, output,
                                      dtype, scratch, kStaticScratchBytes, stream);
}
