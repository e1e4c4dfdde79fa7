// Tensor-parallel all-reduce (sum) over NVLink peer memory for the small, latency-bound messages of a decode step.
//
// Replaces, for that case, NcclTensorParallelCommunicator::all_reduce_sum (src/utils/tensor_parallel.cpp:331-353 of the
// reference), which the row-parallel linears call after o_proj and down_proj (src/layers/linear.cpp:315-318): 72
// all-reduces of [rows, hidden] 16-bit per decode step, 2 MiB each at 256 rows -- far too small to be bandwidth bound.
//
// One process per GPU.  Every rank owns three buffers that all ranks have mapped (plain peer mappings, no multicast):
// `in` (its addend), `out` (the result) and a small flag area.  One launch does a two-shot all-reduce:
//   1. block c of rank r tells every peer "rank r has started" (flag A), i.e. its addend is complete, and waits for the
//      same from every peer;
//   2. it reduces slice c of chunk r (chunk = count / world) over all ranks' `in` buffers in fp32 -- peer loads -- and
//      writes the rounded sums into slice c of chunk r of EVERY rank's `out` buffer -- peer stores;
//   3. after a block barrier it tells every peer, with a system-scope release store, "slice c of chunk r has landed"
//      (flag B) and waits for the same from every peer, so when the kernel ends the whole `out` buffer of this rank is
//      complete.
// Blocks never wait for other blocks of their own GPU, only for the block with the same index on the peers, so the
// ranks' kernels need not be co-scheduled block for block.  Flags carry a launch counter (epoch) kept in device memory,
// so a captured launch can be replayed.  Every wait is bounded (about one second): on a time-out the block raises an
// error word in its own flag area, skips its remaining waits and returns; the host reads the word with
// nvk_tp_allreduce_status.
#include "nvk_internal.cuh"

namespace nvk {
namespace {

constexpr int kArBlocks = 128;           // most blocks a launch uses = flag slots per phase
constexpr int kArUnroll = 2;             // vectors a thread has in flight
constexpr int kArThreads = 256;
constexpr long long kArWaitCycles = 2000000000LL;

struct ArParams {
    const void* in[NVK_TP_MAX_RANKS];    // every rank's addend (index = rank), as mapped in this process
    void* out[NVK_TP_MAX_RANKS];         // every rank's result buffer
    uint32_t* flags[NVK_TP_MAX_RANKS];   // every rank's flag area
    int rank, world;
    int64_t count;                       // elements; a multiple of 8 * world
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Flag area layout (uint32): [0] epoch of the last completed launch, [1] blocks finished in the current launch,
// [2] error word, [3] unused, then phase A slots [block][rank], then phase B slots [block][rank].
__device__ __forceinline__ uint32_t* flag_slot(uint32_t* base, int phase, int block, int rank) {
    return base + 4 + (phase * kArBlocks + block) * NVK_TP_MAX_RANKS + rank;
}

// Thread r < world of the block: publish `epoch` in slot [phase][block][my rank] of rank r's flags, then wait until rank r
// has published it in mine.  Returns false (whole block) when a wait ran out.
//
// Phase 0 publishes with a relaxed store: what it announces (this rank's addend) was written by earlier kernels of the
// stream into this GPU's own memory and is complete at the kernel boundary, and nothing this kernel wrote precedes it.
// A release store there costs about 4 us for nothing.  Phase 1 publishes with a release store after the block's
// __syncthreads(): the barrier orders every thread's peer stores before the publishing thread, and its release makes
// them visible system-wide before the flag (no per-thread system fence, which cost another 7 us).
__device__ __forceinline__ bool exchange(const ArParams& p, int phase, uint32_t epoch, int* timed_out) {
    const int r = threadIdx.x;
    if (r < p.world) {
        if (phase == 0) st_relaxed_sys(flag_slot(p.flags[r], phase, blockIdx.x, p.rank), epoch);
        else st_release_sys(flag_slot(p.flags[r], phase, blockIdx.x, p.rank), epoch);
        const uint32_t* mine = flag_slot(p.flags[p.rank], phase, blockIdx.x, r);
        const long long start = clock64();
        while (ld_acquire_sys(mine) != epoch) {
            if (clock64() - start > kArWaitCycles) {
                atomicExch(reinterpret_cast<unsigned int*>(p.flags[p.rank] + 2), 1u + static_cast<unsigned int>(phase));
                *timed_out = 1;
                break;
            }
        }
    }
    __syncthreads();
    return *timed_out == 0;
}

template <typename T>
__global__ void __launch_bounds__(kArThreads) allreduce_two_shot_kernel(const ArParams p) {
    __shared__ int s_timed_out;
    if (threadIdx.x == 0) s_timed_out = 0;
    __syncthreads();
    uint32_t* my_flags = p.flags[p.rank];
    const uint32_t epoch = my_flags[0] + 1u;   // the same on every rank: all ranks run the same sequence of launches

    bool ok = exchange(p, 0, epoch, &s_timed_out);   // every addend is complete

    if (ok) {
        const int64_t chunk_vecs = p.count / p.world / 8;          // 16-byte vectors in one rank's chunk
        const int64_t per_block = (chunk_vecs + gridDim.x - 1) / gridDim.x;
        const int64_t v0 = static_cast<int64_t>(blockIdx.x) * per_block;
        const int64_t v1 = v0 + per_block < chunk_vecs ? v0 + per_block : chunk_vecs;
        const int64_t base = static_cast<int64_t>(p.rank) * chunk_vecs;   // this rank reduces chunk `rank`
        for (int64_t vb = v0 + threadIdx.x; vb < v1; vb += kArThreads * kArUnroll) {
            uint4 part[kArUnroll][NVK_TP_MAX_RANKS];
#pragma unroll
            for (int u = 0; u < kArUnroll; ++u) {   // every load of this round first: peer latency is paid once
                const int64_t v = vb + u * kArThreads;
#pragma unroll
                for (int r = 0; r < NVK_TP_MAX_RANKS; ++r)
                    if (r < p.world && v < v1) part[u][r] = ld_peer16(static_cast<const uint4*>(p.in[r]) + base + v);
            }
#pragma unroll
            for (int u = 0; u < kArUnroll; ++u) {
                const int64_t v = vb + u * kArThreads;
                if (v >= v1) break;
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int r = 0; r < NVK_TP_MAX_RANKS; ++r) {
                    if (r < p.world) {
                        const T* e = reinterpret_cast<const T*>(&part[u][r]);
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[i] += ElemTraits<T>::to_float(e[i]);
                    }
                }
                uint4 sum;
                sum.x = ElemTraits<T>::pack2(acc[0], acc[1]); sum.y = ElemTraits<T>::pack2(acc[2], acc[3]);
                sum.z = ElemTraits<T>::pack2(acc[4], acc[5]); sum.w = ElemTraits<T>::pack2(acc[6], acc[7]);
#pragma unroll
                for (int r = 0; r < NVK_TP_MAX_RANKS; ++r)
                    if (r < p.world) static_cast<uint4*>(p.out[r])[base + v] = sum;
            }
        }
        __syncthreads();          // every thread's peer stores precede the release store of the publishing threads
        ok = exchange(p, 1, epoch, &s_timed_out);   // every rank's slice of every chunk has landed here
    }

    // the last block of the launch publishes the epoch for the next launch
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(reinterpret_cast<unsigned int*>(my_flags + 1), 1u) == gridDim.x - 1) {
            my_flags[1] = 0u;
            my_flags[0] = epoch;
            __threadfence();
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The same all-reduce with the two element-wise kernels that follow it in a decoder layer folded in:
//     h_new = residual + sum over ranks of addend          (src/layers/linear.cpp:315-318 then the residual add)
//     x     = rmsnorm(h_new) * weight                      (the layer norm that consumes h_new next)
// A rank's chunk of the [rows, cols] message is rows / world whole rows, so the rank that reduces a row also has all of
// it for the mean of squares: it adds its (replicated) residual row, rounds to T, normalises the rounded values as the
// separate kernel would, and pushes both rows into every rank's `out` (h_new) and `norm` (x) buffers.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kNormMaxVecs = 4;   // 16-byte vectors of a row per thread: cols <= 256 * 4 * 8 = 8192

struct ArNormParams {
    ArParams ar;
    void* norm[NVK_TP_MAX_RANKS];     // every rank's buffer for x
    const void* residual;             // [rows, cols], this rank's copy (identical on all ranks)
    const void* weight;               // [cols]
    float eps;
    int rows, cols;
};

template <typename T>
__global__ void __launch_bounds__(kArThreads) allreduce_add_rmsnorm_kernel(const ArNormParams q) {
    const ArParams& p = q.ar;
    __shared__ int s_timed_out;
    __shared__ float s_part[kArThreads / 32];
    if (threadIdx.x == 0) s_timed_out = 0;
    __syncthreads();
    uint32_t* my_flags = p.flags[p.rank];
    const uint32_t epoch = my_flags[0] + 1u;

    bool ok = exchange(p, 0, epoch, &s_timed_out);

    if (ok) {
        const int rows_per_rank = q.rows / p.world;
        const int row_vecs = q.cols / 8;
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        for (int lr = blockIdx.x; lr < rows_per_rank; lr += gridDim.x) {
            const int64_t row = static_cast<int64_t>(p.rank) * rows_per_rank + lr;
            const int64_t base = row * row_vecs;
            uint4 part[kNormMaxVecs][NVK_TP_MAX_RANKS];
            uint4 res[kNormMaxVecs];
#pragma unroll
            for (int u = 0; u < kNormMaxVecs; ++u) {   // every load first
                const int v = threadIdx.x + u * kArThreads;
                if (v < row_vecs) {
                    res[u] = static_cast<const uint4*>(q.residual)[base + v];
#pragma unroll
                    for (int r = 0; r < NVK_TP_MAX_RANKS; ++r)
                        if (r < p.world) part[u][r] = ld_peer16(static_cast<const uint4*>(p.in[r]) + base + v);
                }
            }
            float hn[kNormMaxVecs][8];
            uint4 hpack[kNormMaxVecs];
            float ss = 0.0f;
#pragma unroll
            for (int u = 0; u < kNormMaxVecs; ++u) {
                const int v = threadIdx.x + u * kArThreads;
                if (v < row_vecs) {
                    float acc[8];
                    const T* e0 = reinterpret_cast<const T*>(&res[u]);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
#pragma unroll
                    for (int r = 0; r < NVK_TP_MAX_RANKS; ++r) {
                        if (r < p.world) {
                            const T* e = reinterpret_cast<const T*>(&part[u][r]);
#pragma unroll
                            for (int i = 0; i < 8; ++i) acc[i] += ElemTraits<T>::to_float(e[i]);
                        }
                    }
                    // the sum is rounded to T first (what the all-reduce alone would deliver), then the residual is added in T
                    T* hp = reinterpret_cast<T*>(&hpack[u]);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float s = ElemTraits<T>::to_float(ElemTraits<T>::from_float(acc[i]));
                        hp[i] = ElemTraits<T>::from_float(ElemTraits<T>::to_float(e0[i]) + s);
                        hn[u][i] = ElemTraits<T>::to_float(hp[i]);
                        ss += hn[u][i] * hn[u][i];
                    }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            __syncthreads();   // s_part of the previous row has been read by everyone
            if (lane == 0) s_part[warp] = ss;
            __syncthreads();
            float total = 0.0f;
#pragma unroll
            for (int w = 0; w < kArThreads / 32; ++w) total += s_part[w];
            const float inv_rms = rsqrtf(total / static_cast<float>(q.cols) + q.eps);
#pragma unroll
            for (int u = 0; u < kNormMaxVecs; ++u) {
                const int v = threadIdx.x + u * kArThreads;
                if (v < row_vecs) {
                    const uint4 wv = static_cast<const uint4*>(q.weight)[v];
                    const T* we = reinterpret_cast<const T*>(&wv);
                    uint4 xpack;
                    T* xp = reinterpret_cast<T*>(&xpack);
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        xp[i] = ElemTraits<T>::from_float(hn[u][i] * inv_rms * ElemTraits<T>::to_float(we[i]));
#pragma unroll
                    for (int r = 0; r < NVK_TP_MAX_RANKS; ++r) {
                        if (r < p.world) {
                            static_cast<uint4*>(p.out[r])[base + v] = hpack[u];
                            static_cast<uint4*>(q.norm[r])[base + v] = xpack;
                        }
                    }
                }
            }
        }
        __syncthreads();
        ok = exchange(p, 1, epoch, &s_timed_out);
    }

    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(reinterpret_cast<unsigned int*>(my_flags + 1), 1u) == gridDim.x - 1) {
            my_flags[1] = 0u;
            my_flags[0] = epoch;
            __threadfence();
        }
    }
}

}  // namespace
}  // namespace nvk

extern "C" size_t nvk_tp_allreduce_flag_bytes(void) {
    return (4 + 2 * nvk::kArBlocks * NVK_TP_MAX_RANKS) * sizeof(uint32_t);
}

extern "C" int nvk_tp_allreduce(const void* const* in_ptrs, void* const* out_ptrs, void* const* flag_ptrs, int rank, int world,
                                int64_t count, int dtype, void* stream) {
    using namespace nvk;
    if (!in_ptrs || !out_ptrs || !flag_ptrs) return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce: pointer tables must be defined");
    if (world < 2 || world > NVK_TP_MAX_RANKS || rank < 0 || rank >= world)
        return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce: world must be 2..%d and rank inside it", NVK_TP_MAX_RANKS);
    if (dtype != NVK_F16 && dtype != NVK_BF16) return fail(NVK_ERR_UNSUPPORTED, "tp all-reduce: dtype must be F16 or BF16");
    if (count <= 0 || count % (8 * world) != 0)
        return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce: count must be a positive multiple of 8 * world");
    ArParams p{};
    for (int r = 0; r < world; ++r) {
        if (!in_ptrs[r] || !out_ptrs[r] || !flag_ptrs[r]) return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce: null buffer of rank %d", r);
        if (!aligned_to(in_ptrs[r], 16) || !aligned_to(out_ptrs[r], 16) || !aligned_to(flag_ptrs[r], 4))
            return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce: buffers must be 16-byte aligned");
        p.in[r] = in_ptrs[r]; p.out[r] = out_ptrs[r]; p.flags[r] = static_cast<uint32_t*>(flag_ptrs[r]);
    }
    p.rank = rank; p.world = world; p.count = count;
    // blocks: about kArUnroll rounds of work per thread, the same number on every rank (it depends on count and world only)
    const int64_t chunk_vecs = count / world / 8;
    int64_t blocks = (chunk_vecs + kArThreads * kArUnroll - 1) / (kArThreads * kArUnroll);
    if (blocks < 4) blocks = 4;
    if (blocks > kArBlocks) blocks = kArBlocks;
    const unsigned grid = static_cast<unsigned>(blocks);
    if (dtype == NVK_BF16)
        allreduce_two_shot_kernel<__nv_bfloat16><<<grid, kArThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    else
        allreduce_two_shot_kernel<__half><<<grid, kArThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return check_launch("allreduce_two_shot_kernel launch");
}

extern "C" int nvk_tp_allreduce_status(const void* own_flags, void* stream, int* status) {
    using namespace nvk;
    if (!own_flags || !status) return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce status: null argument");
    uint32_t word = 0;
    cudaError_t e = cudaMemcpyAsync(&word, static_cast<const uint32_t*>(own_flags) + 2, sizeof(word), cudaMemcpyDeviceToHost,
                                    static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "tp all-reduce status: %s", cudaGetErrorString(e));
    *status = static_cast<int>(word);
    return NVK_OK;
}

extern "C" int nvk_tp_allreduce_add_rmsnorm(const void* const* in_ptrs, void* const* out_ptrs, void* const* norm_ptrs,
                                            void* const* flag_ptrs, const void* residual, const void* weight, float eps,
                                            int rank, int world, int rows, int cols, int dtype, void* stream) {
    using namespace nvk;
    if (!in_ptrs || !out_ptrs || !norm_ptrs || !flag_ptrs || !residual || !weight)
        return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce + add + rmsnorm: every pointer must be defined");
    if (world < 2 || world > NVK_TP_MAX_RANKS || rank < 0 || rank >= world)
        return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce + add + rmsnorm: world must be 2..%d and rank inside it", NVK_TP_MAX_RANKS);
    if (dtype != NVK_F16 && dtype != NVK_BF16) return fail(NVK_ERR_UNSUPPORTED, "tp all-reduce + add + rmsnorm: dtype must be F16 or BF16");
    if (rows <= 0 || rows % world != 0) return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce + add + rmsnorm: rows must be a positive multiple of world");
    if (cols <= 0 || cols % 8 != 0 || cols > kArThreads * kNormMaxVecs * 8)
        return fail(NVK_ERR_UNSUPPORTED, "tp all-reduce + add + rmsnorm: cols must be a multiple of 8 and at most %d", kArThreads * kNormMaxVecs * 8);
    if (!aligned_to(residual, 16) || !aligned_to(weight, 16))
        return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce + add + rmsnorm: residual and weight must be 16-byte aligned");
    ArNormParams q{};
    for (int r = 0; r < world; ++r) {
        if (!in_ptrs[r] || !out_ptrs[r] || !norm_ptrs[r] || !flag_ptrs[r])
            return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce + add + rmsnorm: null buffer of rank %d", r);
        if (!aligned_to(in_ptrs[r], 16) || !aligned_to(out_ptrs[r], 16) || !aligned_to(norm_ptrs[r], 16) || !aligned_to(flag_ptrs[r], 4))
            return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce + add + rmsnorm: buffers must be 16-byte aligned");
        q.ar.in[r] = in_ptrs[r]; q.ar.out[r] = out_ptrs[r]; q.norm[r] = norm_ptrs[r]; q.ar.flags[r] = static_cast<uint32_t*>(flag_ptrs[r]);
    }
    q.ar.rank = rank; q.ar.world = world; q.ar.count = static_cast<int64_t>(rows) * cols;
    q.residual = residual; q.weight = weight; q.eps = eps; q.rows = rows; q.cols = cols;
    int blocks = rows / world;
    if (blocks > kArBlocks) blocks = kArBlocks;
    if (dtype == NVK_BF16)
        allreduce_add_rmsnorm_kernel<__nv_bfloat16><<<blocks, kArThreads, 0, static_cast<cudaStream_t>(stream)>>>(q);
    else
        allreduce_add_rmsnorm_kernel<__half><<<blocks, kArThreads, 0, static_cast<cudaStream_t>(stream)>>>(q);
    return check_launch("allreduce_add_rmsnorm_kernel launch");
}
