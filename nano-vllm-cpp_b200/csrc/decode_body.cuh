// Device code of the split-K paged decode step, shared by decode_split_kernel (decode_attn.cu) and the mixed
// prefill + decode kernel (prefill_attn_tc.cu): one group of four warps works on one (KV head, split, sequence) item.
// The group synchronises on a named barrier, so several groups can live in one thread block.
#pragma once

#include "nvk_internal.cuh"

namespace nvk {
namespace dec {

constexpr int kHeadDim = 128;
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kTileTokens = 16;                       // tokens per warp tile
constexpr int kRowBytes = kHeadDim * 2;               // one head row of K or V
constexpr int kTileBytes = kTileTokens * kRowBytes;   // 4 KiB (K) ; V follows
constexpr int kStageBytes = 2 * kTileBytes;           // K + V
constexpr int kStages = 3;
constexpr int kMaxGroup = 8;                          // query heads per KV head
constexpr int kMaxChunkBlocks = 128;                  // block-table entries cached per block
constexpr int kSmemBytes = kWarps * kStages * kStageBytes;  // 96 KiB -> two blocks per SM

struct DecodeParams {
    const void* q; const void* k_cache; const void* v_cache;
    IndexArray context_lens; IndexArray block_tables;
    void* out; float* ws_o; float* ws_lse;
    int64_t max_blocks, num_cache_blocks;
    int num_heads, num_kv_heads, group, block_size, chunk_tokens, num_splits;
    float scale_log2;
};

// context_lens[b], limited to what the block table can address (max_blocks * block_size): a longer value would make
// the split kernels read block_tables past the row and the merge kernel read partial results of the next row.
__device__ __forceinline__ int clamped_context(const DecodeParams& p, int64_t b) {
    const int64_t ctx = p.context_lens[b];
    const int64_t cap = p.max_blocks * p.block_size;
    return static_cast<int>(ctx < cap ? ctx : cap);
}

// Barrier over the 128 threads of one group (id 1..15; a block of exactly one group may as well use __syncthreads()).
__device__ __forceinline__ void group_sync(int bar_id) { asm volatile("bar.sync %0, 128;\n" ::"r"(bar_id) : "memory"); }

// One (KV head, split, sequence) item.  `smem`: kSmemBytes of shared memory owned by this group (128-byte aligned),
// `s_blocks`: kMaxChunkBlocks ints of shared memory, `tid`: 0..127 inside the group.  All 128 threads call it.
template <typename T>
__device__ __forceinline__ void decode_split_body(const DecodeParams& p, int kvh, int split, int64_t b, unsigned char* smem,
                                                  int* s_blocks, int tid, int bar_id) {
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int G = p.group;

    const int ctx = clamped_context(p, b);
    const int t0 = split * p.chunk_tokens;
    T* out = static_cast<T*>(p.out);
    if (ctx <= 0) {
        if (split == 0) {  // empty context: zero rows for the whole group
            for (int i = tid; i < G * kHeadDim; i += kThreads)
                out[(b * p.num_heads + kvh * G) * kHeadDim + i] = ElemTraits<T>::from_float(0.0f);
        }
        return;
    }
    if (t0 >= ctx) return;
    const int t1 = min(ctx, t0 + p.chunk_tokens);
    const int live_splits = (ctx + p.chunk_tokens - 1) / p.chunk_tokens;

    // Physical block ids of this chunk (-1 = outside the cache: reads as zeros).
    const int blk0 = t0 / p.block_size;
    const int nblk = (t1 - 1) / p.block_size - blk0 + 1;
    for (int i = tid; i < nblk; i += kThreads) {
        const int64_t id = p.block_tables[b * p.max_blocks + blk0 + i];
        s_blocks[i] = (id >= 0 && id < p.num_cache_blocks) ? static_cast<int>(id) : -1;
    }
    group_sync(bar_id);

    // Query fragments: rows g < G of the 16-row A tile, rows 8..15 are zero.
    uint32_t qa[8][2];
    {
        const uint32_t* qrow = reinterpret_cast<const uint32_t*>(
            static_cast<const T*>(p.q) + (b * p.num_heads + kvh * G + (g < G ? g : 0)) * kHeadDim);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            qa[ks][0] = g < G ? qrow[ks * 8 + t] : 0u;
            qa[ks][1] = g < G ? qrow[ks * 8 + 4 + t] : 0u;
        }
    }

    unsigned char* ring = smem + warp * (kStages * kStageBytes);
    const uint32_t ring_u32 = smem_u32(ring);
    const int num_tiles = (t1 - t0 + kTileTokens - 1) / kTileTokens;
    const int my_tiles = num_tiles > warp ? (num_tiles - warp + kWarps - 1) / kWarps : 0;
    const size_t row_stride = static_cast<size_t>(p.num_kv_heads) * kRowBytes;  // bytes between tokens
    const unsigned char* kc = static_cast<const unsigned char*>(p.k_cache) + static_cast<size_t>(kvh) * kRowBytes;
    const unsigned char* vc = static_cast<const unsigned char*>(p.v_cache) + static_cast<size_t>(kvh) * kRowBytes;

    // Lane's piece of a tile: 16-byte column c of rows r = 2 * i + (lane >> 4), i = 0..7.
    const int c = lane & 15, rhalf = lane >> 4;

    auto issue = [&](int j) {  // load this warp's j-th tile into stage j % kStages
        if (j < my_tiles) {
            const int tok0 = t0 + (warp + j * kWarps) * kTileTokens;
            const int blk = tok0 / p.block_size;
            const int phys = s_blocks[blk - blk0];
            const int off = tok0 - blk * p.block_size;
            const size_t base = (static_cast<size_t>(phys < 0 ? 0 : phys) * p.block_size + off) * row_stride + c * 16;
            const uint32_t stage = ring_u32 + (j % kStages) * kStageBytes;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = 2 * i + rhalf;
                const int bytes = (phys >= 0 && tok0 + r < t1) ? 16 : 0;
                const size_t src = base + (bytes ? r * row_stride : 0);
                const uint32_t dst = stage + r * kRowBytes + ((c ^ (r & 7)) << 4);
                cp_async16(dst, kc + src, bytes);
                cp_async16(dst + kTileBytes, vc + src, bytes);
            }
        }
        cp_async_commit();
    };

    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m_run = -INFINITY, l_run = 0.0f;  // per head g (replicated over the 4 lanes of a row)

#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) issue(s);

    // ldmatrix lane addressing.  K (non-transposed): matrices (tok 0-7, d lo), (tok 0-7, d hi),
    // (tok 8-15, d lo), (tok 8-15, d hi) of one 16-wide k-step.  V (transposed): matrices
    // (tok 0-7, d lo), (tok 0-7, d hi), (tok 8-15, d lo), (tok 8-15, d hi) of one 16-wide d-tile.
    const int k_row = ((lane >> 4) << 3) + (lane & 7);
    const int k_sel = (lane >> 3) & 1;
    const int v_row = (((lane >> 3) >> 1) << 3) + (lane & 7);
    const int v_sel = (lane >> 3) & 1;

    for (int j = 0; j < my_tiles; ++j) {
        issue(j + kStages - 1);
        cp_async_wait<kStages - 1>();
        __syncwarp();
        const uint32_t stage = ring_u32 + (j % kStages) * kStageBytes;
        const int tok0 = t0 + (warp + j * kWarps) * kTileTokens;

        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t b0, b1, b2, b3;
            const int chunk = 2 * ks + k_sel;
            ldmatrix_x4(b0, b1, b2, b3, stage + k_row * kRowBytes + ((chunk ^ (k_row & 7)) << 4));
            mma_16816<T>(s0, qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
            mma_16816<T>(s1, qa[ks][0], 0u, qa[ks][1], 0u, b2, b3);
        }
        // scores of head g: tokens tok0 + {2t, 2t+1, 8+2t, 9+2t}
        float sc[4];
        sc[0] = s0[0] * p.scale_log2; sc[1] = s0[1] * p.scale_log2;
        sc[2] = s1[0] * p.scale_log2; sc[3] = s1[1] * p.scale_log2;
        const int tk = tok0 + 2 * t;
        if (tk >= t1) sc[0] = -INFINITY;
        if (tk + 1 >= t1) sc[1] = -INFINITY;
        if (tk + 8 >= t1) sc[2] = -INFINITY;
        if (tk + 9 >= t1) sc[3] = -INFINITY;
        float m_tile = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 1));
        m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 2));
        const float m_new = fmaxf(m_run, m_tile);   // finite: token tok0 is always valid
        const float corr = fast_exp2(m_run - m_new);
        const float p0 = fast_exp2(sc[0] - m_new), p1 = fast_exp2(sc[1] - m_new);
        const float p2 = fast_exp2(sc[2] - m_new), p3 = fast_exp2(sc[3] - m_new);
        l_run = l_run * corr + ((p0 + p1) + (p2 + p3));
        m_run = m_new;
        const uint32_t pb0 = ElemTraits<T>::pack2(p0, p1);
        const uint32_t pb1 = ElemTraits<T>::pack2(p2, p3);
        // accumulator columns of this lane are heads 2t and 2t+1
        const float c0 = __shfl_sync(0xffffffffu, corr, 8 * t);
        const float c1 = __shfl_sync(0xffffffffu, corr, 8 * t + 4);
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            uint32_t a0, a1, a2, a3;
            const int chunk = 2 * mt + v_sel;
            ldmatrix_x4_trans(a0, a1, a2, a3, stage + kTileBytes + v_row * kRowBytes + ((chunk ^ (v_row & 7)) << 4));
            o[mt][0] *= c0; o[mt][1] *= c1; o[mt][2] *= c0; o[mt][3] *= c1;
            mma_16816<T>(o[mt], a0, a1, a2, a3, pb0, pb1);
        }
        __syncwarp();
    }
    cp_async_wait<0>();
    group_sync(bar_id);  // every ring is idle from here on: reuse it for the cross-warp merge

    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);

    float* sm_o = reinterpret_cast<float*>(smem);                    // [warp][head][128]
    float* sm_m = sm_o + kWarps * kMaxGroup * kHeadDim;              // [warp][head]
    float* sm_l = sm_m + kWarps * kMaxGroup;
    if (t == 0) { sm_m[warp * kMaxGroup + g] = m_run; sm_l[warp * kMaxGroup + g] = l_run; }
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
        const int d = mt * 16 + g;
        float* dst = sm_o + (warp * kMaxGroup + 2 * t) * kHeadDim + d;
        dst[0] = o[mt][0]; dst[kHeadDim] = o[mt][1]; dst[8] = o[mt][2]; dst[kHeadDim + 8] = o[mt][3];
    }
    group_sync(bar_id);

    // thread d merges column d of every head of the group over the four warps
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

}  // namespace dec
}  // namespace nvk
