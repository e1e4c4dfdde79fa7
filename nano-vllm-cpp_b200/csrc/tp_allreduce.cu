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
//   3. after a system-scope fence it tells every peer "slice c of chunk r has landed" (flag B) and waits for the same
//      from every peer, so when the kernel ends the whole `out` buffer of this rank is complete.
// Blocks never wait for other blocks of their own GPU, only for the block with the same index on the peers, so the
// ranks' kernels need not be co-scheduled block for block.  Flags carry a launch counter (epoch) kept in device memory,
// so a captured launch can be replayed.  Every wait is bounded (about one second): on a time-out the block raises an
// error word in its own flag area, skips its remaining waits and returns; the host reads the word with
// nvk_tp_allreduce_status.
#include "nvk_internal.cuh"

namespace nvk {
namespace {

constexpr int kArBlocks = 96;            // most blocks a launch uses = flag slots per phase
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
__device__ __forceinline__ bool exchange(const ArParams& p, int phase, uint32_t epoch, int* timed_out) {
    const int r = threadIdx.x;
    if (r < p.world) {
        st_release_sys(flag_slot(p.flags[r], phase, blockIdx.x, p.rank), epoch);
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
        __threadfence_system();   // this thread's peer stores are visible system-wide before the block says so
        __syncthreads();
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
