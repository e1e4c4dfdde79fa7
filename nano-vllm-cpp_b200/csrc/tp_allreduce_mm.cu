// Tensor-parallel all-reduce through the NVSwitch: the in-switch reduction (multimem.ld_reduce) and the in-switch
// broadcast (multimem.st) of an NVLink multicast object, for the same latency-bound decode-step messages as
// tp_allreduce.cu (NcclTensorParallelCommunicator::all_reduce_sum, src/utils/tensor_parallel.cpp:331-353 of the
// reference; called from src/layers/linear.cpp:315-318).
//
// Why a second kernel: the tagged-word kernel sends every byte twice (payload + tag) to every peer, so its wire time
// grows with the number of ranks (7 MiB out per rank for a 2 MiB message at 8 ranks).  Here a rank pulls the SUM of
// its rows from the switch (it receives rows / world reduced rows, each peer sends its slice once) and stores the
// result once, the switch copying it to all ranks: 2 MiB in and 2 MiB out per rank whatever the world size.
//
// Buffers: addend and result buffers live at the same offset in every rank's part of one symmetric
// allocation that is bound to a multicast object; the caller passes their MULTICAST addresses.  Every rank also owns a
// signal area (plain peer mapping, zeroed once) and a private flag area as in tp_allreduce.cu.  One launch:
//   1. barrier: block b tells block b of every peer "my addend is complete" (it was written by the kernel before this
//      one) and waits for theirs -- one word per (block, peer), valued with the launch's epoch;
//   2. the block pulls its rows' sums (fp32 accumulation in the switch, rounded once to the 16-bit type), adds the
//      residual (fused form) and stores the result rows through the multicast address;
//   3. a system-scope fence, then a second set of words says "block b's rows are stored" to every peer.  Plain form: the
//      block waits for the same word of every peer, so after the barriers of all blocks the whole result is local.
//      Fused form: nobody waits there; the rows of the peers' chunks are dealt out over all blocks of the (larger) grid,
//      each of which waits for the word of a row's block, reads the row from this rank's own copy of the result and
//      writes its RMSNorm -- so only result rows cross the wire, and every row has been awaited when the launch ends.
// Every wait is bounded and the error word is sticky, as in tp_allreduce.cu (same flag area layout, same status and
// reset calls).  A rank must not exit while its peers still run launches: its memory is bound to the multicast object.
#include "nvk_internal.cuh"

#include <atomic>

namespace nvk {
namespace {

constexpr int kMmThreads = 256;
constexpr int kMmBlocks = 128;            // most blocks per rank (signal words are laid out for this many)
constexpr int kMmMaxVecs = 4;             // 16-byte vectors of a row per thread: cols <= 8192

std::atomic<long long> g_mm_wait_cycles{20000000000LL};

struct MmParams {
    const void* mc_in; void* mc_out;                     // multicast addresses
    const void* out_local; void* norm;                   // fused form: this rank's own mapping of the result buffer, its norm buffer
    const void* residual; const void* weight;            // this rank's own memory
    uint32_t* signal[NVK_TP_MAX_RANKS];                  // every rank's signal area as mapped here (index = rank)
    uint32_t* flags;                                     // private: [0] epoch of the last launch, [1] blocks finished, [2] error
    long long wait_cycles;
    float eps;
    int rank, world, rows, cols;
};

template <typename T> struct MmOps;
template <> struct MmOps<__nv_bfloat16> {
    static __device__ __forceinline__ uint4 ld_reduce(const void* mc) {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
        return v;
    }
};
template <> struct MmOps<__half> {
    static __device__ __forceinline__ uint4 ld_reduce(const void* mc) {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
        return v;
    }
};
__device__ __forceinline__ void mc_store(void* mc, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_signal(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_signal_acquire(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Polls with relaxed loads and a short sleep between them (a block may wait for most of the launch, and system-scope acquire
// loads in a tight loop cost the memory system more than they gain); one acquire load once the word has the value.
__device__ __forceinline__ bool wait_signal(const uint32_t* word, uint32_t epoch, const MmParams& p, int* gave_up, unsigned int code) {
    long long start = 0;
    while (true) {
        uint32_t v;
        asm volatile("ld.relaxed.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(word) : "memory");
        if (v == epoch) { ld_signal_acquire(word); return true; }
        if (*reinterpret_cast<volatile int*>(gave_up)) return false;
        if (start == 0) start = clock64();
        else if (clock64() - start > p.wait_cycles) {
            *reinterpret_cast<volatile int*>(gave_up) = 1;
            atomicCAS(reinterpret_cast<unsigned int*>(p.flags + 2), 0u, code);
            return false;
        }
        __nanosleep(64);
    }
}

// Word layout of a signal area: [set (2)][block (kMmBlocks)][source rank (NVK_TP_MAX_RANKS)].
__device__ __forceinline__ int signal_index(int set, int block, int src) {
    return (set * kMmBlocks + block) * NVK_TP_MAX_RANKS + src;
}

// Block-level barrier with block `block` of every peer.  Threads 0 .. world-1 each handle one peer.  Returns false
// when a wait ran out (the error word is set; the caller stops touching data).
__device__ __forceinline__ bool peer_barrier(const MmParams& p, int set, int block, uint32_t epoch, int* gave_up, int code) {
    const int t = threadIdx.x;
    if (t < p.world && t != p.rank) {
        st_signal(p.signal[t] + signal_index(set, block, p.rank), epoch);
        wait_signal(p.signal[p.rank] + signal_index(set, block, t), epoch, p, gave_up, static_cast<unsigned int>(code));
    }
    __syncthreads();
    return *reinterpret_cast<volatile int*>(gave_up) == 0;
}

__device__ __forceinline__ float mm_block_sum(float v, float* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kMmThreads / 32; ++w) total += scratch[w];
    return total;
}

// x = h * rsqrt(mean(h^2) + eps) * weight for this thread's vectors of one row (h as rounded to T), stored to this
// rank's own norm buffer.
template <typename T>
__device__ __forceinline__ void mm_norm_row(const MmParams& p, const uint4 (&h)[kMmMaxVecs], int row_vecs, int64_t base, float* scratch) {
    float ss = 0.0f;
#pragma unroll
    for (int u = 0; u < kMmMaxVecs; ++u) {
        if (static_cast<int>(threadIdx.x) + u * kMmThreads < row_vecs) {
            const T* e = reinterpret_cast<const T*>(&h[u]);
#pragma unroll
            for (int i = 0; i < 8; ++i) { const float f = ElemTraits<T>::to_float(e[i]); ss += f * f; }
        }
    }
    const float inv_rms = rsqrtf(mm_block_sum(ss, scratch) / static_cast<float>(p.cols) + p.eps);
#pragma unroll
    for (int u = 0; u < kMmMaxVecs; ++u) {
        const int v = static_cast<int>(threadIdx.x) + u * kMmThreads;
        if (v < row_vecs) {
            const uint4 wv = __ldg(static_cast<const uint4*>(p.weight) + v);
            const T* we = reinterpret_cast<const T*>(&wv);
            const T* e = reinterpret_cast<const T*>(&h[u]);
            float x[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = ElemTraits<T>::to_float(e[i]) * inv_rms * ElemTraits<T>::to_float(we[i]);
            uint4 xv;
            xv.x = ElemTraits<T>::pack2(x[0], x[1]); xv.y = ElemTraits<T>::pack2(x[2], x[3]);
            xv.z = ElemTraits<T>::pack2(x[4], x[5]); xv.w = ElemTraits<T>::pack2(x[6], x[7]);
            static_cast<uint4*>(p.norm)[base + v] = xv;
        }
    }
}

// Grid: `reducers` = min(rows / world, kMmBlocks) blocks pull and broadcast the rows of this rank's chunk; in the fused
// form the grid may be larger, and all of its blocks then normalise the rows that arrive from the peers.
template <typename T, bool FUSED>
__global__ void __launch_bounds__(kMmThreads) allreduce_mm_kernel(const MmParams p) {
    __shared__ int s_gave_up;
    __shared__ float s_scratch[kMmThreads / 32];
    asm volatile("griddepcontrol.wait;\n" ::: "memory");             // the addend comes from the kernel before this one
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int tid = threadIdx.x, block = blockIdx.x, blocks = gridDim.x;
    if (tid == 0) s_gave_up = 0;
    __syncthreads();
    const uint32_t last = *reinterpret_cast<volatile uint32_t*>(p.flags);
    const uint32_t epoch = last + 1u == 0u ? 1u : last + 1u;          // never 0: signal areas start zeroed
    const bool poisoned = *reinterpret_cast<volatile uint32_t*>(p.flags + 2) != 0u;
    const int row_vecs = p.cols / 8;
    const int rows_per_rank = p.rows / p.world;
    const int reducers = rows_per_rank < kMmBlocks ? rows_per_rank : kMmBlocks;

    if (!poisoned) {
        if (block < reducers) {
            if (peer_barrier(p, 0, block, epoch, &s_gave_up, 1)) {
                // rows of this rank's chunk, strided over the reducing blocks (the same assignment on every rank)
                for (int r = block; r < rows_per_rank; r += reducers) {
                    const int64_t base = (static_cast<int64_t>(p.rank) * rows_per_rank + r) * row_vecs;
                    uint4 h[kMmMaxVecs];
#pragma unroll
                    for (int u = 0; u < kMmMaxVecs; ++u) {
                        const int v = tid + u * kMmThreads;
                        if (v < row_vecs) h[u] = MmOps<T>::ld_reduce(static_cast<const uint4*>(p.mc_in) + base + v);
                    }
                    if (FUSED) {
#pragma unroll
                        for (int u = 0; u < kMmMaxVecs; ++u) {
                            const int v = tid + u * kMmThreads;
                            if (v < row_vecs) {
                                const uint4 res = static_cast<const uint4*>(p.residual)[base + v];
                                const T* a = reinterpret_cast<const T*>(&h[u]);
                                const T* b = reinterpret_cast<const T*>(&res);
                                float f[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i)     // the sum arrives rounded to T; the residual is added in T
                                    f[i] = ElemTraits<T>::to_float(a[i]) + ElemTraits<T>::to_float(b[i]);
                                h[u].x = ElemTraits<T>::pack2(f[0], f[1]); h[u].y = ElemTraits<T>::pack2(f[2], f[3]);
                                h[u].z = ElemTraits<T>::pack2(f[4], f[5]); h[u].w = ElemTraits<T>::pack2(f[6], f[7]);
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < kMmMaxVecs; ++u) {
                        const int v = tid + u * kMmThreads;
                        if (v < row_vecs) mc_store(static_cast<uint4*>(p.mc_out) + base + v, h[u]);
                    }
                    if (FUSED) mm_norm_row<T>(p, h, row_vecs, base, s_scratch);   // the own rows' norm from registers
                }
            }
            // every store of this block is ordered before the signals: barrier, then a system-scope fence by the signalling threads
            __syncthreads();
            if (tid < p.world) __threadfence_system();
            if (FUSED) {
                // tell block `block`'s rows to every peer; nobody waits here: the rows are awaited where they are normalised
                if (tid < p.world && tid != p.rank && *reinterpret_cast<volatile int*>(&s_gave_up) == 0)
                    st_signal(p.signal[tid] + signal_index(1, block, p.rank), epoch);
            } else {
                peer_barrier(p, 1, block, epoch, &s_gave_up, 2);
            }
        }
        if (FUSED) {
            // rows of the peers' chunks, strided over ALL blocks: wait for the row's block on its rank, normalise it from this
            // rank's own copy of the result (only result rows cross the wire)
            // (separate blocks for this part, waiting from the start of the launch, measured 3 us slower at 2 ranks)
            const int64_t items = static_cast<int64_t>(p.world - 1) * rows_per_rank;
            for (int64_t item = block; item < items; item += blocks) {
                const int o = static_cast<int>(item / rows_per_rank);
                const int src = o < p.rank ? o : o + 1;
                const int r = static_cast<int>(item - static_cast<int64_t>(o) * rows_per_rank);
                if (tid == 0) wait_signal(p.signal[p.rank] + signal_index(1, r % reducers, src), epoch, p, &s_gave_up, 2u);
                __syncthreads();
                if (*reinterpret_cast<volatile int*>(&s_gave_up)) break;
                const int64_t base = (static_cast<int64_t>(src) * rows_per_rank + r) * row_vecs;
                uint4 h[kMmMaxVecs];
#pragma unroll
                for (int u = 0; u < kMmMaxVecs; ++u) {
                    const int v = tid + u * kMmThreads;
                    if (v < row_vecs) h[u] = __ldcg(static_cast<const uint4*>(p.out_local) + base + v);
                }
                mm_norm_row<T>(p, h, row_vecs, base, s_scratch);
            }
        }
    }

    __syncthreads();
    if (tid == 0) {   // the last block of the launch publishes the epoch for the next launch
        __threadfence();
        if (atomicAdd(reinterpret_cast<unsigned int*>(p.flags + 1), 1u) == static_cast<unsigned int>(blocks) - 1u) {
            p.flags[1] = 0u;
            p.flags[0] = epoch;
            __threadfence();
        }
    }
}

int launch_mm(const void* mc_in, void* mc_out, const void* out_local, void* norm, void* const* signal_ptrs, void* flags, const void* residual,
              const void* weight, float eps, int rank, int world, int rows, int cols, int dtype, bool fused, cudaStream_t stream) {
    const char* what = fused ? "tp all-reduce + add + rmsnorm (multimem)" : "tp all-reduce (multimem)";
    if (world < 2 || world > NVK_TP_MAX_RANKS || rank < 0 || rank >= world)
        return fail(NVK_ERR_INVALID_ARGUMENT, "%s: world must be 2..%d and rank inside it", what, NVK_TP_MAX_RANKS);
    if (dtype != NVK_F16 && dtype != NVK_BF16) return fail(NVK_ERR_UNSUPPORTED, "%s: dtype must be F16 or BF16", what);
    if (rows <= 0 || rows % world != 0) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: rows must be a positive multiple of world", what);
    if (cols <= 0 || cols % 8 != 0 || cols > kMmThreads * kMmMaxVecs * 8)
        return fail(NVK_ERR_UNSUPPORTED, "%s: cols must be a multiple of 8 and at most %d", what, kMmThreads * kMmMaxVecs * 8);
    if (!mc_in || !mc_out || !signal_ptrs || !flags || (fused && (!out_local || !norm || !residual || !weight)))
        return fail(NVK_ERR_INVALID_ARGUMENT, "%s: every pointer must be defined", what);
    if (!aligned_to(mc_in, 16) || !aligned_to(mc_out, 16) || (fused && (!aligned_to(out_local, 16) || !aligned_to(norm, 16) || !aligned_to(residual, 16) || !aligned_to(weight, 16))))
        return fail(NVK_ERR_INVALID_ARGUMENT, "%s: buffers must be 16-byte aligned", what);
    MmParams p{};
    p.mc_in = mc_in; p.mc_out = mc_out; p.out_local = out_local; p.norm = norm; p.residual = residual; p.weight = weight;
    for (int r = 0; r < world; ++r) {
        if (!signal_ptrs[r] || !aligned_to(signal_ptrs[r], 16)) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: signal area of rank %d missing or misaligned", what, r);
        p.signal[r] = static_cast<uint32_t*>(signal_ptrs[r]);
    }
    p.flags = static_cast<uint32_t*>(flags);
    p.wait_cycles = g_mm_wait_cycles.load(std::memory_order_relaxed);
    p.eps = eps; p.rank = rank; p.world = world; p.rows = rows; p.cols = cols;
    const int per_rank = rows / world;
    int blocks = per_rank < kMmBlocks ? per_rank : kMmBlocks;             // the reducing blocks
    if (fused) {                                                          // and up to one block per row that arrives
        const int64_t items = static_cast<int64_t>(world - 1) * per_rank;
        blocks = static_cast<int>(items < kMmBlocks ? (items > blocks ? items : blocks) : kMmBlocks);
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(blocks));
    cfg.blockDim = dim3(kMmThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e;
    if (fused) e = dtype == NVK_BF16 ? cudaLaunchKernelEx(&cfg, allreduce_mm_kernel<__nv_bfloat16, true>, p) : cudaLaunchKernelEx(&cfg, allreduce_mm_kernel<__half, true>, p);
    else e = dtype == NVK_BF16 ? cudaLaunchKernelEx(&cfg, allreduce_mm_kernel<__nv_bfloat16, false>, p) : cudaLaunchKernelEx(&cfg, allreduce_mm_kernel<__half, false>, p);
    if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
    return check_launch(what);
}

}  // namespace

void set_multimem_wait_cycles(long long cycles) { g_mm_wait_cycles.store(cycles, std::memory_order_relaxed); }

}  // namespace nvk

extern "C" size_t nvk_tp_allreduce_signal_bytes(void) { return static_cast<size_t>(2) * nvk::kMmBlocks * NVK_TP_MAX_RANKS * sizeof(uint32_t); }

extern "C" int nvk_tp_allreduce_multimem(const void* mc_in, void* mc_out, void* const* signal_ptrs, void* flags, int rank, int world,
                                         int rows, int cols, int dtype, void* stream) {
    return nvk::launch_mm(mc_in, mc_out, nullptr, nullptr, signal_ptrs, flags, nullptr, nullptr, 0.0f, rank, world, rows, cols, dtype, false,
                          static_cast<cudaStream_t>(stream));
}

extern "C" int nvk_tp_allreduce_add_rmsnorm_multimem(const void* mc_in, void* mc_out, const void* out, void* norm, void* const* signal_ptrs, void* flags,
                                                     const void* residual, const void* weight, float eps, int rank, int world, int rows,
                                                     int cols, int dtype, void* stream) {
    return nvk::launch_mm(mc_in, mc_out, out, norm, signal_ptrs, flags, residual, weight, eps, rank, world, rows, cols, dtype, true,
                          static_cast<cudaStream_t>(stream));
}
