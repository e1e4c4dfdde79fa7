// Tensor-parallel all-reduce (sum) over NVLink peer memory for the small, latency-bound messages of a decode step.
//
// Replaces, for that case, NcclTensorParallelCommunicator::all_reduce_sum (src/utils/tensor_parallel.cpp:331-353 of the
// reference), which the row-parallel linears call after o_proj and down_proj (src/layers/linear.cpp:315-318): 72
// all-reduces of [rows, hidden] 16-bit per decode step, 2 MiB each at 256 rows -- far too small to be bandwidth bound.
// The message crosses the wire in under 3 us; what such a collective costs is synchronisation, so this one has none
// that is separate from the data: no flag exchange, no memory fence, no peer load.
//
// One process per GPU.  Every rank owns a staging area that all ranks have mapped (plain peer mappings, no multicast);
// addend, result, residual and norm buffers are ordinary memory of the rank that owns them -- peers never touch them.
// Data crosses NVLink as self-validating words: a 16-byte vector of payload is stored as two 16-byte vectors
// {w0, epoch, w1, epoch} {w2, epoch, w3, epoch}; each 8-byte half arrives atomically, so a receiver that sees `epoch`
// in both tags of a vector holds its payload (the low-latency protocol NCCL uses for small messages).  The epoch is a
// launch counter kept in device memory: the same on every rank, because all ranks run the same sequence of launches,
// and different from whatever an earlier launch left in the slot.  One launch is a two-shot all-reduce, chunk r of
// the message (count / world elements; whole rows in the fused form) being reduced by rank r:
//   1. push    every rank stores the slices of its addend that belong to the other ranks' chunks into their staging
//              areas (region A, indexed by source rank);
//   2. reduce  it adds its own slice and the world - 1 slices arriving in its region A in fp32, in rank order, rounds
//              once (the fused form then adds the residual row and computes the row's RMSNorm);
//   3. push    it stores the result slice into every other rank's region B and into its own output buffers;
//   4. gather  it copies the other chunks' results from its region B into its output buffers as they arrive (the fused
//              form computes their RMSNorm on the way, so only one row per result crosses the wire).
// Blocks only ever wait for data, and only for the data of the same-numbered block of the peers.  A staging slot is
// never overwritten before it was read: a rank can only start launch L + 1 after every peer finished reducing launch L
// (it holds their results), and it writes region B of launch L + 1 only after every peer pushed region A of L + 1,
// which they do after finishing all of L.
//
// Every wait is bounded (nvk_tp_allreduce_set_wait_limit_ms, 10 s unless set).  A block whose wait runs out raises the
// error word in its rank's flag area; from then on every launch of that rank returns at once (the error is sticky), so
// a dead peer costs one time-out, not one per launch, and peers of a rank that gave up time out once themselves.
// Results since the last zero status are invalid; see nvk_tp_allreduce_reset for re-arming.
//
// The same device code also runs `world` ranks on ONE device in one cooperative launch
// (nvk_tp_allreduce_inprocess): the counterpart of the reference's in-process communicator
// (src/utils/tensor_parallel.cpp:165-277), used to test the protocol where only one GPU is present.
#include "nvk_internal.cuh"

#include <atomic>

namespace nvk {
namespace {

constexpr int kArBlocks = 128;           // most blocks per rank
constexpr int kArThreads = 256;
constexpr int kMaxVecs = 4;              // 16-byte vectors of a row per thread (fused form): cols <= 256 * 4 * 8 = 8192
constexpr int kFlagWords = 64;           // flag area: [0] epoch of the last completed launch, [1] blocks finished, [2] error word

std::atomic<long long> g_wait_cycles{20000000000LL};   // about 10 s at 2 GHz

struct ArParams {
    const void* in;                          // this rank's addend
    void* out;                               // this rank's result buffer (h_new in the fused form)
    void* norm;                              // fused form: this rank's buffer for x
    const void* residual;                    // fused form: [rows, cols], this rank's copy (identical on all ranks)
    const void* weight;                      // fused form: [cols]
    uint4* stage[NVK_TP_MAX_RANKS];          // every rank's staging area as mapped in this process (index = rank)
    uint32_t* flags;                         // this rank's flag area
    int64_t region_b;                        // offset of region B inside a staging area, in uint4
    int64_t chunk_vecs;                      // 16-byte payload vectors per rank chunk
    int64_t seg_vecs;                        // payload vectors per block segment (fused form: one row)
    long long wait_cycles;
    float eps;
    int rank, world, cols;
    int pushed;                              // 1: the producer of the addend already pushed the other ranks' slices (gemm_fused.cu)
};
struct ArGroup { ArParams r[NVK_TP_MAX_RANKS]; };   // in-process form: one parameter set per rank

__device__ __forceinline__ void st_tagged(uint4* slot, const uint4& v, uint32_t ep) {
    // one 32-byte store per payload vector: a warp writes 1 KiB of contiguous, fully covered 128-byte lines (two 16-byte
    // stores per lane left every sector half written per instruction, which costs NVLink packets)
    asm volatile("st.volatile.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n"
                 ::"l"(slot), "r"(v.x), "r"(ep), "r"(v.y), "r"(ep), "r"(v.z), "r"(ep), "r"(v.w), "r"(ep) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile16(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Waits until the tagged vectors slot[k] (k < n, k != skip; at most NVK_TP_MAX_RANKS) all carry `ep`, returns their
// payloads.  All loads of a round are issued before any tag is looked at, so the round costs one memory latency.
// Every index is a compile-time constant after unrolling (the arrays stay in registers).  Gives up (payload
// undefined) when the limit runs out or another thread of the block already gave up.
struct Waiter {
    const ArParams& p;
    int* gave_up;          // shared: set by the first thread whose wait ran out
    int code;
    __device__ __forceinline__ void poll(const uint4* const (&slot)[NVK_TP_MAX_RANKS], int n, int skip, uint32_t ep,
                                         uint4 (&payload)[NVK_TP_MAX_RANKS]) const {
        long long start = 0;
        while (true) {
            uint4 a[NVK_TP_MAX_RANKS], b[NVK_TP_MAX_RANKS];
#pragma unroll
            for (int k = 0; k < NVK_TP_MAX_RANKS; ++k)
                if (k < n && k != skip) { a[k] = ld_volatile16(slot[k]); b[k] = ld_volatile16(slot[k] + 1); }
            bool ready = true;
#pragma unroll
            for (int k = 0; k < NVK_TP_MAX_RANKS; ++k)
                if (k < n && k != skip) {
                    ready = ready && a[k].y == ep && a[k].w == ep && b[k].y == ep && b[k].w == ep;
                    payload[k] = make_uint4(a[k].x, a[k].z, b[k].x, b[k].z);
                }
            if (ready) return;
            if (*reinterpret_cast<volatile int*>(gave_up)) return;
            if (start == 0) start = clock64();
            else if (clock64() - start > p.wait_cycles) {
                *reinterpret_cast<volatile int*>(gave_up) = 1;
                atomicCAS(reinterpret_cast<unsigned int*>(p.flags + 2), 0u, static_cast<unsigned int>(code));
                return;
            }
        }
    }
};

template <typename T>
__device__ __forceinline__ void accumulate(float (&acc)[8], const uint4& v) {
    const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += ElemTraits<T>::to_float(e[i]);
}
template <typename T>
__device__ __forceinline__ uint4 round_pack(const float (&acc)[8]) {
    uint4 r;
    r.x = ElemTraits<T>::pack2(acc[0], acc[1]); r.y = ElemTraits<T>::pack2(acc[2], acc[3]);
    r.z = ElemTraits<T>::pack2(acc[4], acc[5]); r.w = ElemTraits<T>::pack2(acc[6], acc[7]);
    return r;
}

// Block-wide sum of one float per thread (every thread gets the total).  `scratch` holds kArThreads / 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();   // scratch of the previous use has been read by everyone
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kArThreads / 32; ++w) total += scratch[w];
    return total;
}

// x = h * rsqrt(mean(h^2) + eps) * weight for this thread's vectors of one row; h as rounded to T.
template <typename T>
__device__ __forceinline__ void norm_row(const ArParams& p, const uint4 (&h)[kMaxVecs], int row_vecs, int64_t row_base,
                                         float* scratch) {
    float ss = 0.0f;
#pragma unroll
    for (int u = 0; u < kMaxVecs; ++u) {
        if (static_cast<int>(threadIdx.x) + u * kArThreads < row_vecs) {
            const T* e = reinterpret_cast<const T*>(&h[u]);
#pragma unroll
            for (int i = 0; i < 8; ++i) { const float f = ElemTraits<T>::to_float(e[i]); ss += f * f; }
        }
    }
    const float inv_rms = rsqrtf(block_sum(ss, scratch) / static_cast<float>(p.cols) + p.eps);
#pragma unroll
    for (int u = 0; u < kMaxVecs; ++u) {
        const int v = static_cast<int>(threadIdx.x) + u * kArThreads;
        if (v < row_vecs) {
            const uint4 wv = __ldg(static_cast<const uint4*>(p.weight) + v);
            const T* we = reinterpret_cast<const T*>(&wv);
            const T* e = reinterpret_cast<const T*>(&h[u]);
            float x[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = ElemTraits<T>::to_float(e[i]) * inv_rms * ElemTraits<T>::to_float(we[i]);
            static_cast<uint4*>(p.norm)[row_base + v] = round_pack<T>(x);
        }
    }
}

// One rank's part of one launch, as block `block` of `blocks`.
template <typename T, bool FUSED>
__device__ __forceinline__ void allreduce_body(const ArParams& p, int block, int blocks) {
    __shared__ int s_gave_up;
    __shared__ float s_scratch[kArThreads / 32];
    if (threadIdx.x == 0) s_gave_up = 0;
    __syncthreads();
    const uint32_t last = *reinterpret_cast<volatile uint32_t*>(p.flags);
    const uint32_t epoch = last + 1u == 0u ? 1u : last + 1u;     // never 0: staging areas start zeroed
    const bool poisoned = *reinterpret_cast<volatile uint32_t*>(p.flags + 2) != 0u;
    const int tid = threadIdx.x;
    const uint4* in = static_cast<const uint4*>(p.in);
    uint4* out = static_cast<uint4*>(p.out);
    const int64_t segs = (p.chunk_vecs + p.seg_vecs - 1) / p.seg_vecs;      // segments per chunk
    const int seg_len = static_cast<int>(p.seg_vecs);

    if (!poisoned) {
        // ---- 1. push this rank's slices of the other ranks' chunks ---------------------------------------------
        if (FUSED) {
            // work items = (other rank, row of its chunk), strided over all blocks: with many ranks a chunk has fewer rows than
            // the launch has blocks, and the pushes are what the wire time is made of
            const int64_t items = static_cast<int64_t>(p.world - 1) * segs;
            for (int64_t item = block; item < items && !p.pushed; item += blocks) {
                const int o = static_cast<int>(item / segs);
                const int r = o < p.rank ? o : o + 1;
                const int64_t v0 = (item - o * segs) * p.seg_vecs;
                uint4 mine[kMaxVecs];
#pragma unroll
                for (int u = 0; u < kMaxVecs; ++u)
                    if (tid + u * kArThreads < seg_len) mine[u] = in[r * p.chunk_vecs + v0 + tid + u * kArThreads];
#pragma unroll
                for (int u = 0; u < kMaxVecs; ++u)
                    if (tid + u * kArThreads < seg_len)
                        st_tagged(p.stage[r] + 2 * (p.rank * p.chunk_vecs + v0 + tid + u * kArThreads), mine[u], epoch);
            }
        } else {
            for (int64_t seg = block; seg < segs && !p.pushed; seg += blocks) {
                const int64_t v0 = seg * p.seg_vecs;
                const int n = static_cast<int>(min(static_cast<int64_t>(seg_len), p.chunk_vecs - v0));
                for (int v = tid; v < n; v += kArThreads) {
                    uint4 mine[NVK_TP_MAX_RANKS];
#pragma unroll
                    for (int r = 0; r < NVK_TP_MAX_RANKS; ++r)
                        if (r < p.world && r != p.rank) mine[r] = in[r * p.chunk_vecs + v0 + v];
#pragma unroll
                    for (int r = 0; r < NVK_TP_MAX_RANKS; ++r)
                        if (r < p.world && r != p.rank) st_tagged(p.stage[r] + 2 * (p.rank * p.chunk_vecs + v0 + v), mine[r], epoch);
                }
            }
        }
        // ---- 2. reduce this rank's chunk, 3. push the results ---------------------------------------------------
        const uint4* stage_a = p.stage[p.rank];
        const Waiter waiter_a{p, &s_gave_up, 1};
        for (int64_t seg = block; seg < segs; seg += blocks) {
            const int64_t v0 = seg * p.seg_vecs;
            const int n = static_cast<int>(min(static_cast<int64_t>(seg_len), p.chunk_vecs - v0));
            const int64_t base = p.rank * p.chunk_vecs + v0;            // position in the whole message
            auto reduce_one = [&](int v) -> uint4 {
                const uint4 own = in[base + v];
                const uint4* slot[NVK_TP_MAX_RANKS];
                uint4 got[NVK_TP_MAX_RANKS];
#pragma unroll
                for (int r = 0; r < NVK_TP_MAX_RANKS; ++r) slot[r] = stage_a + 2 * (r * p.chunk_vecs + v0 + v);
                waiter_a.poll(slot, p.world, p.rank, epoch, got);
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int r = 0; r < NVK_TP_MAX_RANKS; ++r) {      // rank order, whoever does the adding
                    if (r < p.world) {
                        if (r == p.rank) accumulate<T>(acc, own);
                        else accumulate<T>(acc, got[r]);
                    }
                }
                if (FUSED) {
                    // the sum is rounded to T first (what the all-reduce alone would deliver), then the residual is added in T
                    const uint4 res = static_cast<const uint4*>(p.residual)[base + v];
                    const T* e0 = reinterpret_cast<const T*>(&res);
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        acc[i] = ElemTraits<T>::to_float(e0[i]) + ElemTraits<T>::to_float(ElemTraits<T>::from_float(acc[i]));
                }
                const uint4 h = round_pack<T>(acc);
                // a rank that gave up publishes nothing more: a peer that is merely late must run into its own
                // time-out instead of accepting a result made from slices that never arrived
                if (*reinterpret_cast<volatile int*>(&s_gave_up)) return h;
#pragma unroll
                for (int r = 0; r < NVK_TP_MAX_RANKS; ++r)
                    if (r < p.world && r != p.rank) st_tagged(p.stage[r] + 2 * (p.region_b + base + v), h, epoch);
                out[base + v] = h;
                return h;
            };
            if (FUSED) {                       // a segment is one row, at most kMaxVecs vectors per thread: keep them for the norm
                uint4 h[kMaxVecs];
#pragma unroll
                for (int u = 0; u < kMaxVecs; ++u)
                    if (tid + u * kArThreads < n) h[u] = reduce_one(tid + u * kArThreads);
                norm_row<T>(p, h, n, base, s_scratch);
            } else {
                for (int v = tid; v < n; v += kArThreads) reduce_one(v);
            }
        }
        // ---- 4. gather the other chunks' results ---------------------------------------------------------------
        const uint4* stage_b = p.stage[p.rank] + 2 * p.region_b;
        const Waiter waiter_b{p, &s_gave_up, 2};
        if (FUSED) {
            const int64_t items = static_cast<int64_t>(p.world - 1) * segs;   // (other rank, row of its chunk), as in the push
            for (int64_t item = block; item < items; item += blocks) {
                const int o = static_cast<int>(item / segs);
                const int s = o < p.rank ? o : o + 1;
                const int64_t v0 = (item - o * segs) * p.seg_vecs;
                const int n = seg_len;
                {
                    const int64_t base = s * p.chunk_vecs + v0;
                    uint4 h[kMaxVecs];
                    {
                        const uint4* slot[NVK_TP_MAX_RANKS];
                        uint4 got[NVK_TP_MAX_RANKS];
                        const int mine = tid < n ? (n - tid + kArThreads - 1) / kArThreads : 0;   // this thread's vectors: u < mine
#pragma unroll
                        for (int u = 0; u < kMaxVecs; ++u) slot[u] = stage_b + 2 * (base + tid + u * kArThreads);
                        waiter_b.poll(slot, mine, -1, epoch, got);
                        const bool abandoned = *reinterpret_cast<volatile int*>(&s_gave_up) != 0;
#pragma unroll
                        for (int u = 0; u < kMaxVecs; ++u)
                            if (u < mine) { h[u] = got[u]; if (!abandoned) out[base + tid + u * kArThreads] = got[u]; }
                    }
                    norm_row<T>(p, h, n, base, s_scratch);
                }
            }
        } else {
            for (int64_t seg = block; seg < segs; seg += blocks) {
                const int64_t v0 = seg * p.seg_vecs;
                const int n = static_cast<int>(min(static_cast<int64_t>(seg_len), p.chunk_vecs - v0));
                for (int v = tid; v < n; v += kArThreads) {
                    const uint4* slot[NVK_TP_MAX_RANKS];
                    uint4 got[NVK_TP_MAX_RANKS];
#pragma unroll
                    for (int r = 0; r < NVK_TP_MAX_RANKS; ++r) slot[r] = stage_b + 2 * (r * p.chunk_vecs + v0 + v);
                    waiter_b.poll(slot, p.world, p.rank, epoch, got);
                    if (*reinterpret_cast<volatile int*>(&s_gave_up)) break;
#pragma unroll
                    for (int r = 0; r < NVK_TP_MAX_RANKS; ++r)
                        if (r < p.world && r != p.rank) out[r * p.chunk_vecs + v0 + v] = got[r];
                }
            }
        }
    }

    // the last block of the launch publishes the epoch for the next launch
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(reinterpret_cast<unsigned int*>(p.flags + 1), 1u) == static_cast<unsigned int>(blocks) - 1u) {
            p.flags[1] = 0u;
            p.flags[0] = epoch;
            __threadfence();
        }
    }
}

template <typename T, bool FUSED>
__global__ void __launch_bounds__(kArThreads) allreduce_ll_kernel(const ArParams p) {
    asm volatile("griddepcontrol.wait;\n" ::: "memory");             // the addend comes from the kernel before this one
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    allreduce_body<T, FUSED>(p, blockIdx.x, gridDim.x);
}

// `world` ranks on one device: blockIdx.y is the rank.  Launched cooperatively, so all blocks are resident and the
// ranks can wait for one another's data.
template <typename T, bool FUSED>
__global__ void __launch_bounds__(kArThreads) allreduce_ll_inprocess_kernel(const ArGroup g) {
    allreduce_body<T, FUSED>(g.r[blockIdx.y], blockIdx.x, gridDim.x);
}

struct Plan { int64_t chunk_vecs, seg_vecs; int blocks; };

// Blocks per rank and segment size: the same on every rank (they depend on the message only).
Plan plan_plain(int64_t count, int world) {
    Plan pl{};
    pl.chunk_vecs = count / world / 8;
    int64_t blocks = (pl.chunk_vecs + kArThreads - 1) / kArThreads;    // about one vector per thread
    if (blocks < 1) blocks = 1;
    if (blocks > kArBlocks) blocks = kArBlocks;
    pl.seg_vecs = (pl.chunk_vecs + blocks - 1) / blocks;
    pl.blocks = static_cast<int>((pl.chunk_vecs + pl.seg_vecs - 1) / pl.seg_vecs);
    return pl;
}
Plan plan_fused(int rows, int cols, int world) {
    Plan pl{};
    pl.seg_vecs = cols / 8;
    pl.chunk_vecs = static_cast<int64_t>(rows / world) * pl.seg_vecs;
    // one block per row of the own chunk for the reduction; more, up to one per (other rank, row), for the pushes and the gather
    const int64_t items = static_cast<int64_t>(world - 1) * (rows / world);
    pl.blocks = static_cast<int>(items < kArBlocks ? items : kArBlocks);
    return pl;
}

int check_common(const char* what, void* const* stage_ptrs, const void* flags, int rank, int world, int dtype, size_t stage_bytes,
                 int64_t count) {
    if (!stage_ptrs || !flags) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: staging table and flag area must be defined", what);
    if (world < 2 || world > NVK_TP_MAX_RANKS || rank < 0 || rank >= world)
        return fail(NVK_ERR_INVALID_ARGUMENT, "%s: world must be 2..%d and rank inside it", what, NVK_TP_MAX_RANKS);
    if (dtype != NVK_F16 && dtype != NVK_BF16) return fail(NVK_ERR_UNSUPPORTED, "%s: dtype must be F16 or BF16", what);
    if (count <= 0 || count % (8 * world) != 0)
        return fail(NVK_ERR_INVALID_ARGUMENT, "%s: count must be a positive multiple of 8 * world", what);
    if (stage_bytes < nvk_tp_allreduce_stage_bytes(count))
        return fail(NVK_ERR_INVALID_ARGUMENT, "%s: staging areas of %zu bytes given, %zu needed for %lld elements", what, stage_bytes,
                    nvk_tp_allreduce_stage_bytes(count), static_cast<long long>(count));
    for (int r = 0; r < world; ++r) {
        if (!stage_ptrs[r]) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: null staging area of rank %d", what, r);
        if (!aligned_to(stage_ptrs[r], 32)) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: staging areas must be 32-byte aligned", what);
    }
    if (!aligned_to(flags, 16)) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: the flag area must be 16-byte aligned", what);
    return NVK_OK;
}

void fill_common(ArParams& p, void* const* stage_ptrs, void* flags, int rank, int world, size_t stage_bytes, const Plan& pl) {
    for (int r = 0; r < world; ++r) p.stage[r] = static_cast<uint4*>(stage_ptrs[r]);
    p.flags = static_cast<uint32_t*>(flags);
    p.region_b = static_cast<int64_t>(stage_bytes / 2 / 32);   // in payload vectors: two uint4 each
    p.chunk_vecs = pl.chunk_vecs; p.seg_vecs = pl.seg_vecs;
    p.wait_cycles = g_wait_cycles.load(std::memory_order_relaxed);
    p.rank = rank; p.world = world;
}

template <bool FUSED>
int launch(const ArParams& p, int blocks, int dtype, cudaStream_t stream) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(blocks));
    cfg.blockDim = dim3(kArThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = dtype == NVK_BF16 ? cudaLaunchKernelEx(&cfg, allreduce_ll_kernel<__nv_bfloat16, FUSED>, p)
                                             : cudaLaunchKernelEx(&cfg, allreduce_ll_kernel<__half, FUSED>, p);
    if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "tp all-reduce launch: %s", cudaGetErrorString(e));
    return check_launch("tp all-reduce launch");
}

}  // namespace
}  // namespace nvk

extern "C" size_t nvk_tp_allreduce_flag_bytes(void) { return nvk::kFlagWords * sizeof(uint32_t); }

// Two regions (incoming addend slices, incoming results), each holding the whole message as tagged vectors (2 x payload).
extern "C" size_t nvk_tp_allreduce_stage_bytes(int64_t max_count) {
    if (max_count <= 0) return 0;
    const size_t region = (static_cast<size_t>(max_count) * 2 * 2 + 255) / 256 * 256;
    return 2 * region;
}

extern "C" void nvk_tp_allreduce_set_wait_limit_ms(int ms) {
    if (ms < 1) ms = 1;
    nvk::g_wait_cycles.store(static_cast<long long>(ms) * 2000000LL, std::memory_order_relaxed);   // cycles at 2 GHz
    nvk::set_multimem_wait_cycles(static_cast<long long>(ms) * 2000000LL);
}

extern "C" int nvk_tp_allreduce(const void* in, void* out, void* const* stage_ptrs, size_t stage_bytes, void* flags, int rank,
                                int world, int64_t count, int dtype, void* stream) {
    using namespace nvk;
    const int rc = check_common("tp all-reduce", stage_ptrs, flags, rank, world, dtype, stage_bytes, count);
    if (rc != NVK_OK) return rc;
    if (!in || !out) return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce: addend and result must be defined");
    if (!aligned_to(in, 16) || !aligned_to(out, 16)) return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce: buffers must be 16-byte aligned");
    const Plan pl = plan_plain(count, world);
    ArParams p{};
    fill_common(p, stage_ptrs, flags, rank, world, stage_bytes, pl);
    p.in = in; p.out = out;
    return launch<false>(p, pl.blocks, dtype, static_cast<cudaStream_t>(stream));
}

namespace nvk {
int launch_allreduce_add_rmsnorm(const void* in, void* out, void* norm, void* const* stage_ptrs, size_t stage_bytes, void* flags,
                                 const void* residual, const void* weight, float eps, int rank, int world, int rows, int cols,
                                 int dtype, bool pushed, cudaStream_t stream) {
    const char* what = "tp all-reduce + add + rmsnorm";
    if (rows <= 0 || world <= 0 || rows % world != 0) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: rows must be a positive multiple of world", what);
    if (cols <= 0 || cols % 8 != 0 || cols > kArThreads * kMaxVecs * 8)
        return fail(NVK_ERR_UNSUPPORTED, "%s: cols must be a multiple of 8 and at most %d", what, kArThreads * kMaxVecs * 8);
    const int rc = check_common(what, stage_ptrs, flags, rank, world, dtype, stage_bytes, static_cast<int64_t>(rows) * cols);
    if (rc != NVK_OK) return rc;
    if (!in || !out || !norm || !residual || !weight) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: every pointer must be defined", what);
    if (!aligned_to(in, 16) || !aligned_to(out, 16) || !aligned_to(norm, 16) || !aligned_to(residual, 16) || !aligned_to(weight, 16))
        return fail(NVK_ERR_INVALID_ARGUMENT, "%s: buffers must be 16-byte aligned", what);
    const Plan pl = plan_fused(rows, cols, world);
    ArParams p{};
    fill_common(p, stage_ptrs, flags, rank, world, stage_bytes, pl);
    p.in = in; p.out = out; p.norm = norm; p.residual = residual; p.weight = weight; p.eps = eps; p.cols = cols;
    p.pushed = pushed ? 1 : 0;
    return launch<true>(p, pl.blocks, dtype, stream);
}
}  // namespace nvk

extern "C" int nvk_tp_allreduce_add_rmsnorm(const void* in, void* out, void* norm, void* const* stage_ptrs, size_t stage_bytes,
                                            void* flags, const void* residual, const void* weight, float eps, int rank, int world,
                                            int rows, int cols, int dtype, void* stream) {
    return nvk::launch_allreduce_add_rmsnorm(in, out, norm, stage_ptrs, stage_bytes, flags, residual, weight, eps, rank, world, rows,
                                             cols, dtype, false, static_cast<cudaStream_t>(stream));
}

namespace nvk {
int launch_allreduce_inprocess(const void* const* in_ptrs, void* const* out_ptrs, void* const* norm_ptrs, void* const* stage_ptrs,
                               size_t stage_bytes, void* const* flag_ptrs, const void* const* residual_ptrs, const void* weight,
                               float eps, int world, int rows, int cols, int dtype, bool pushed, cudaStream_t stream) {
    const char* what = "tp all-reduce (in-process)";
    const bool fused = norm_ptrs != nullptr;
    if (!in_ptrs || !out_ptrs || !flag_ptrs) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: pointer tables must be defined", what);
    if (rows <= 0 || cols <= 0 || cols % 8 != 0) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: rows and cols must be positive, cols a multiple of 8", what);
    if (fused && (world <= 0 || rows % world != 0 || cols > kArThreads * kMaxVecs * 8 || !residual_ptrs || !weight))
        return fail(NVK_ERR_INVALID_ARGUMENT, "%s: the fused form needs rows %% world == 0, cols <= %d, residuals and a weight", what,
                    kArThreads * kMaxVecs * 8);
    const int64_t count = static_cast<int64_t>(rows) * cols;
    if (world < 2 || world > NVK_TP_MAX_RANKS) return fail(NVK_ERR_INVALID_ARGUMENT, "%s: world must be 2..%d", what, NVK_TP_MAX_RANKS);
    ArGroup g{};
    Plan pl{};
    for (int r = 0; r < world; ++r) {
        const int rc = check_common(what, stage_ptrs, flag_ptrs[r], r, world, dtype, stage_bytes, count);
        if (rc != NVK_OK) return rc;
        if (!in_ptrs[r] || !out_ptrs[r] || (fused && (!norm_ptrs[r] || !residual_ptrs[r])))
            return fail(NVK_ERR_INVALID_ARGUMENT, "%s: null buffer of rank %d", what, r);
        pl = fused ? plan_fused(rows, cols, world) : plan_plain(count, world);
        fill_common(g.r[r], stage_ptrs, flag_ptrs[r], r, world, stage_bytes, pl);
        g.r[r].in = in_ptrs[r]; g.r[r].out = out_ptrs[r];
        if (fused) { g.r[r].norm = norm_ptrs[r]; g.r[r].residual = residual_ptrs[r]; g.r[r].weight = weight; g.r[r].eps = eps; g.r[r].cols = cols; }
        g.r[r].pushed = pushed ? 1 : 0;
    }
    // every block of every rank must be resident at once: ask the occupancy calculator, shrink the grid if needed
    const void* fn = fused ? (dtype == NVK_BF16 ? reinterpret_cast<const void*>(allreduce_ll_inprocess_kernel<__nv_bfloat16, true>)
                                                : reinterpret_cast<const void*>(allreduce_ll_inprocess_kernel<__half, true>))
                           : (dtype == NVK_BF16 ? reinterpret_cast<const void*>(allreduce_ll_inprocess_kernel<__nv_bfloat16, false>)
                                                : reinterpret_cast<const void*>(allreduce_ll_inprocess_kernel<__half, false>));
    int device = 0, sms = 0, per_sm = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kArThreads, 0);
    if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    int blocks = pl.blocks;
    const int fit = sms * per_sm / world;
    if (fit < 1) return fail(NVK_ERR_UNSUPPORTED, "%s: %d ranks do not fit on this device at once", what, world);
    if (blocks > fit) blocks = fit;   // blocks stride over the segments, any count is valid
    void* args[] = {&g};
    e = cudaLaunchCooperativeKernel(fn, dim3(static_cast<unsigned>(blocks), static_cast<unsigned>(world)), dim3(kArThreads), args, 0, stream);
    if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return check_launch("tp all-reduce (in-process) launch");
}
}  // namespace nvk

extern "C" int nvk_tp_allreduce_inprocess(const void* const* in_ptrs, void* const* out_ptrs, void* const* norm_ptrs,
                                          void* const* stage_ptrs, size_t stage_bytes, void* const* flag_ptrs,
                                          const void* const* residual_ptrs, const void* weight, float eps, int world, int rows,
                                          int cols, int dtype, void* stream) {
    return nvk::launch_allreduce_inprocess(in_ptrs, out_ptrs, norm_ptrs, stage_ptrs, stage_bytes, flag_ptrs, residual_ptrs, weight, eps,
                                           world, rows, cols, dtype, false, static_cast<cudaStream_t>(stream));
}

extern "C" int nvk_tp_allreduce_status(const void* flags, void* stream, int* status) {
    using namespace nvk;
    if (!flags || !status) return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce status: null argument");
    uint32_t word = 0;
    cudaError_t e = cudaMemcpyAsync(&word, static_cast<const uint32_t*>(flags) + 2, sizeof(word), cudaMemcpyDeviceToHost,
                                    static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "tp all-reduce status: %s", cudaGetErrorString(e));
    *status = static_cast<int>(word);
    return NVK_OK;
}

extern "C" int nvk_tp_allreduce_reset(void* flags, void* stream) {
    using namespace nvk;
    if (!flags) return fail(NVK_ERR_INVALID_ARGUMENT, "tp all-reduce reset: null argument");
    cudaError_t e = cudaMemsetAsync(flags, 0, kFlagWords * sizeof(uint32_t), static_cast<cudaStream_t>(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NVK_ERR_CUDA, "tp all-reduce reset: %s", cudaGetErrorString(e));
    return NVK_OK;
}
