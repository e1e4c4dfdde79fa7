// Varlen causal prefill attention for sm_100a (F16 / BF16, head_dim 128), dense or paged keys.
//
// Replaces prefill_dense_attention_kernel / prefill_paged_attention_kernel
// (src/kernels/attention.cu:114-302 of the reference: one block per (query row, head), serial
// over keys with a block reduction and two barriers per key) and the FlashAttention-2 varlen call
// (src/kernels/flash_attn.cpp:203-300).  One kernel serves both key layouts: the reference sends
// a batch with any prefix-cache hit through the scalar paged kernel
// (src/layers/attention.cpp:142-157); here cached prefix blocks and freshly stored tokens are
// read through block_tables by the same tiled kernel.
//
// Tiling: one thread block = 64 query rows of one (sequence, head), 4 warps x 16 rows; keys in
// 64-row tiles staged by 16-byte cp.async into XOR-swizzled shared memory (double buffered);
// S = Q K^T and O += P V as mma.sync m16n8k16 with fp32 accumulation; online softmax in the
// exp2 domain; key tiles above the bottom-right-aligned diagonal are skipped, the diagonal
// tile is masked per element.  Heavier (later) query tiles are scheduled first.
#include "nvk_internal.cuh"

#include <cmath>

namespace nvk {
namespace {

constexpr int kHeadDim = 128;
constexpr int kBM = 64;                 // query rows per block
constexpr int kBN = 64;                 // keys per tile
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kRowBytes = kHeadDim * 2;
constexpr int kQBytes = kBM * kRowBytes;          // 16 KiB
constexpr int kKVTileBytes = kBN * kRowBytes;     // 16 KiB each for K and V
constexpr int kStageBytes = 2 * kKVTileBytes;
constexpr int kStages = 2;
constexpr int kSmemBytes = kQBytes + kStages * kStageBytes;  // 80 KiB

struct PrefillParams {
    const void* q; const void* k; const void* v; void* out;
    IndexArray cu_q, cu_k, block_tables;
    int64_t num_seqs, total_q, total_k, max_blocks, key_rows;   // key_rows: rows addressable in k / v
    int num_heads, num_kv_heads, block_size;
    float scale_log2;
};

__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return static_cast<uint32_t>(row * kRowBytes + ((chunk ^ (row & 7)) << 4));
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 2) prefill_tile_kernel(const PrefillParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_info[4];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int head = blockIdx.y;
    const int kvh = head * p.num_kv_heads / p.num_heads;

    // Map the (reversed) tile index to (sequence, first query row).
    if (tid == 0) {
        const int64_t want = static_cast<int64_t>(gridDim.x) - 1 - blockIdx.x;
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
    const int shift = k_len - q_len;                         // bottom-right alignment
    int k_hi = shift + q0 + rows_here;                       // keys visible to the last row of the tile
    if (k_hi > k_len) k_hi = k_len;
    const int num_kt = k_hi > 0 ? (k_hi + kBN - 1) / kBN : 0;

    unsigned char* q_smem = smem;
    const uint32_t q_u32 = smem_u32(q_smem);
    const uint32_t kv_u32 = q_u32 + kQBytes;
    const IndexArray table = p.block_tables ? p.block_tables + static_cast<int64_t>(seq) * p.max_blocks : IndexArray();
    const size_t kv_row_stride = static_cast<size_t>(p.num_kv_heads) * kRowBytes;
    const unsigned char* kbase = static_cast<const unsigned char*>(p.k) + static_cast<size_t>(kvh) * kRowBytes;
    const unsigned char* vbase = static_cast<const unsigned char*>(p.v) + static_cast<size_t>(kvh) * kRowBytes;

    const int c = tid & 15;        // 16-byte column handled by this thread
    const int r0 = tid >> 4;       // first row; rows r0 + 8 i

    // Q tile -> shared (rows beyond the sequence are zero filled)
    {
        const unsigned char* qsrc = static_cast<const unsigned char*>(p.q) +
                                    (static_cast<size_t>(qb + q0) * p.num_heads + head) * kRowBytes + c * 16;
        const size_t q_row_stride = static_cast<size_t>(p.num_heads) * kRowBytes;
#pragma unroll
        for (int i = 0; i < kBM / 8; ++i) {
            const int r = r0 + 8 * i;
            const int bytes = r < rows_here ? 16 : 0;
            cp_async16(q_u32 + swz(r, c), qsrc + (bytes ? r * q_row_stride : 0), bytes);
        }
    }
    auto issue_kv = [&](int kt) {
        const int key0 = kt * kBN;
        const uint32_t stage = kv_u32 + (kt % kStages) * kStageBytes;
        int64_t tile_row0 = 0;
        bool tile_ok = true;
        if (table) {   // a 64-key tile never straddles a cache block (block_size % 64 == 0)
            const int64_t id = table[key0 / p.block_size];
            tile_row0 = static_cast<int64_t>(id) * p.block_size + key0 % p.block_size;
            tile_ok = id >= 0;
        } else {
            tile_row0 = kb + key0;
        }
#pragma unroll
        for (int i = 0; i < kBN / 8; ++i) {
            const int r = r0 + 8 * i;
            const int64_t src_row = tile_row0 + r;
            const int bytes = (tile_ok && key0 + r < k_len && src_row < p.key_rows) ? 16 : 0;
            const size_t off = (bytes ? static_cast<size_t>(src_row) * kv_row_stride : 0) + c * 16;
            cp_async16(stage + swz(r, c), kbase + off, bytes);
            cp_async16(stage + kKVTileBytes + swz(r, c), vbase + off, bytes);
        }
    };
    if (num_kt > 0) issue_kv(0);
    cp_async_commit();

    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    uint32_t qa[8][4];

    const int qi0 = q0 + warp * 16 + g;                 // query index (within the sequence) of row g
    const int lim0 = min(shift + qi0 + 1, k_len);       // keys [0, lim) are visible
    const int lim1 = min(shift + qi0 + 9, k_len);

    // ldmatrix lane addressing
    const int a_row = warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
    const int a_sel = lane >> 4;
    const int kb_row = ((lane >> 4) << 3) + (lane & 7);
    const int kb_sel = (lane >> 3) & 1;
    const int vb_row = ((lane >> 3) & 1) * 8 + (lane & 7);
    const int vb_sel = lane >> 4;

    for (int kt = 0; kt < num_kt; ++kt) {
        if (kt + 1 < num_kt) issue_kv(kt + 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (kt == 0) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
                ldmatrix_x4(qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], q_u32 + swz(a_row, 2 * ks + a_sel));
        }
        const uint32_t stage = kv_u32 + (kt % kStages) * kStageBytes;
        const int key0 = kt * kBN;
        // a warp whose rows see none of this tile's keys skips the math (still takes the barriers)
        const bool warp_active = key0 < shift + q0 + warp * 16 + 16;
        if (warp_active) {
            float s[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f; }
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, stage + swz(np * 16 + kb_row, 2 * ks + kb_sel));
                    mma_16816<T>(s[2 * np], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
                    mma_16816<T>(s[2 * np + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
                }
            }
            const bool need_mask = key0 + kBN > min(shift + q0 + warp * 16 + 1, k_len);   // warp-uniform
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] *= p.scale_log2;
                if (need_mask) {
                    const int key = key0 + nt * 8 + 2 * t;
                    if (key >= lim0) s[nt][0] = -INFINITY;
                    if (key + 1 >= lim0) s[nt][1] = -INFINITY;
                    if (key >= lim1) s[nt][2] = -INFINITY;
                    if (key + 1 >= lim1) s[nt][3] = -INFINITY;
                }
                mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
                mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
            const float base0 = mn0 == -INFINITY ? 0.0f : mn0;   // fully masked row so far
            const float base1 = mn1 == -INFINITY ? 0.0f : mn1;
            const float corr0 = fast_exp2(m_run[0] - base0), corr1 = fast_exp2(m_run[1] - base1);
            m_run[0] = mn0; m_run[1] = mn1;
            float sum0 = 0.0f, sum1 = 0.0f;
            uint32_t pa[4][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const float p0 = fast_exp2(s[nt][0] - base0), p1 = fast_exp2(s[nt][1] - base0);
                const float p2 = fast_exp2(s[nt][2] - base1), p3 = fast_exp2(s[nt][3] - base1);
                sum0 += p0 + p1; sum1 += p2 + p3;
                pa[nt >> 1][(nt & 1) * 2] = ElemTraits<T>::pack2(p0, p1);
                pa[nt >> 1][(nt & 1) * 2 + 1] = ElemTraits<T>::pack2(p2, p3);
            }
            l_run[0] = l_run[0] * corr0 + sum0;
            l_run[1] = l_run[1] * corr1 + sum1;
#pragma unroll
            for (int nt = 0; nt < 16; ++nt) { o[nt][0] *= corr0; o[nt][1] *= corr0; o[nt][2] *= corr1; o[nt][3] *= corr1; }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                for (int dp = 0; dp < 8; ++dp) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3, stage + kKVTileBytes + swz(kk * 16 + vb_row, 2 * dp + vb_sel));
                    mma_16816<T>(o[2 * dp], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                    mma_16816<T>(o[2 * dp + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    __syncthreads();   // covers num_kt == 0: Q copies landed, shared memory reusable

    // Epilogue: normalise, stage the warp's 16 x 128 tile in shared memory, 16-byte row stores.
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
    const float inv0 = l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f;
    const float inv1 = l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f;
    unsigned char* stage_out = q_smem + warp * 16 * kRowBytes;   // this warp's own Q rows
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
        const int chunk = nt;            // 8 columns = one 16-byte chunk; lane t writes 4 bytes of it
        *reinterpret_cast<uint32_t*>(stage_out + swz(g, chunk) + t * 4) = ElemTraits<T>::pack2(o[nt][0] * inv0, o[nt][1] * inv0);
        *reinterpret_cast<uint32_t*>(stage_out + swz(g + 8, chunk) + t * 4) = ElemTraits<T>::pack2(o[nt][2] * inv1, o[nt][3] * inv1);
    }
    __syncwarp();
    unsigned char* obase = static_cast<unsigned char*>(p.out) +
                           (static_cast<size_t>(qb + q0 + warp * 16) * p.num_heads + head) * kRowBytes;
    const size_t o_row_stride = static_cast<size_t>(p.num_heads) * kRowBytes;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = 2 * i + (lane >> 4);
        const int cc = lane & 15;
        if (warp * 16 + r < rows_here) {
            const uint4 vv = *reinterpret_cast<const uint4*>(stage_out + swz(r, cc));
            *reinterpret_cast<uint4*>(obase + r * o_row_stride + cc * 16) = vv;
        }
    }
}

template <typename T>
int launch_typed(const PrefillArgs& a) {
    static bool attr_done[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 0 && device < 64 && !attr_done[device]) {
        const cudaError_t e = cudaFuncSetAttribute(prefill_tile_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "prefill attention: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        attr_done[device] = true;
    }
    PrefillParams p{};
    p.q = a.q; p.out = a.out; p.cu_q = a.cu_q; p.cu_k = a.cu_k; p.block_tables = a.block_tables;
    p.num_seqs = a.cu_q ? a.num_seqs : 1; p.total_q = a.total_q; p.total_k = a.total_k; p.max_blocks = a.max_blocks;
    p.num_heads = a.num_heads; p.num_kv_heads = a.num_kv_heads; p.block_size = a.block_size;
    p.scale_log2 = a.scale * kLog2e;
    if (a.block_tables) { p.k = a.k_cache; p.v = a.v_cache; p.key_rows = a.num_cache_blocks * a.block_size; }
    else { p.k = a.k; p.v = a.v; p.key_rows = a.total_k; }
    const int64_t tiles = (a.total_q + kBM - 1) / kBM + (a.cu_q ? a.num_seqs : 0);
    if (tiles > 0x7fffffffLL || a.num_heads > 65535) return fail(NVK_ERR_UNSUPPORTED, "prefill attention: grid too large");
    const dim3 grid(static_cast<unsigned>(tiles), a.num_heads);
    prefill_tile_kernel<T><<<grid, kThreads, kSmemBytes, a.stream>>>(p);
    return check_launch("prefill_tile_kernel launch");
}

}  // namespace

bool prefill_mma_supported(const PrefillArgs& a) {
    if (a.dtype != NVK_F16 && a.dtype != NVK_BF16) return false;
    if (a.head_dim != kHeadDim) return false;
    if (!aligned_to(a.q, 16) || !aligned_to(a.out, 16)) return false;
    if (a.block_tables) {
        if (a.block_size % kBN != 0) return false;
        if (!aligned_to(a.k_cache, 16) || !aligned_to(a.v_cache, 16)) return false;
    } else {
        if (!aligned_to(a.k, 16) || !aligned_to(a.v, 16)) return false;
    }
    return true;
}

int launch_prefill_mma(const PrefillArgs& a) {
    return a.dtype == NVK_BF16 ? launch_typed<__nv_bfloat16>(a) : launch_typed<__half>(a);
}

}  // namespace nvk
