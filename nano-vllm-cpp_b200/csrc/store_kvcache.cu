// store_kvcache for sm_100a: scatter new K/V rows into the paged cache by slot_mapping.
//
// Replaces src/kernels/kvcache.cu:19-80 of the reference (one 256-thread block per token,
// half of it idle at 2 KiB rows).  Here the copy is a flat, grid-strided stream of 16-byte
// vectors over (K|V, token, column): every thread owns UNROLL independent vectors per trip so
// that several loads are in flight before the first store, the grid is sized from the SM count
// and consecutive lanes touch consecutive 16-byte pieces of one row (full 128-byte lines on
// both sides).  HBM-bound: algorithmic traffic is 2 * num_tokens * row_bytes read and the same
// written, plus 4 or 8 bytes of slot per token.
#include "nvk_internal.cuh"

namespace nvk {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

template <typename VecT, typename SlotT>
__global__ void __launch_bounds__(kThreads)
store_rows_kernel(const VecT* __restrict__ key, const VecT* __restrict__ value,
                  VecT* __restrict__ k_cache, VecT* __restrict__ v_cache,
                  const SlotT* __restrict__ slot_mapping, int64_t num_tokens, int64_t row_vecs,
                  int64_t cache_rows) {
    const int64_t per_tensor = num_tokens * row_vecs;
    const int64_t total = 2 * per_tensor;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads * kUnroll;
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * kThreads * kUnroll + threadIdx.x; base < total;
         base += stride) {
        VecT data[kUnroll];
        int64_t dst[kUnroll];
        bool is_v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t i = base + static_cast<int64_t>(u) * kThreads;
            dst[u] = -1;
            is_v[u] = false;
            if (i < total) {
                is_v[u] = i >= per_tensor;
                const int64_t j = is_v[u] ? i - per_tensor : i;
                const int64_t token = j / row_vecs;
                const int64_t col = j - token * row_vecs;
                const int64_t slot = static_cast<int64_t>(__ldg(slot_mapping + token));
                if (slot >= 0 && slot < cache_rows) {
                    dst[u] = slot * row_vecs + col;
                    data[u] = is_v[u] ? value[j] : key[j];
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (dst[u] >= 0) {
                if (is_v[u]) v_cache[dst[u]] = data[u]; else k_cache[dst[u]] = data[u];
            }
        }
    }
}

template <typename VecT>
int launch_typed(const void* key, const void* value, void* k_cache, void* v_cache, const void* slot_mapping,
                 bool slot_i64, int64_t num_tokens, int64_t row_bytes, int64_t cache_rows, cudaStream_t stream) {
    const int64_t row_vecs = row_bytes / static_cast<int64_t>(sizeof(VecT));
    const int64_t total = 2 * num_tokens * row_vecs;
    int device = 0, sms = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int64_t per_block = static_cast<int64_t>(kThreads) * kUnroll;
    int64_t blocks = (total + per_block - 1) / per_block;
    const int64_t cap = static_cast<int64_t>(sms) * 8;  // 8 resident 256-thread blocks per SM
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (slot_i64) {
        store_rows_kernel<VecT, int64_t><<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(
            static_cast<const VecT*>(key), static_cast<const VecT*>(value), static_cast<VecT*>(k_cache),
            static_cast<VecT*>(v_cache), static_cast<const int64_t*>(slot_mapping), num_tokens, row_vecs, cache_rows);
    } else {
        store_rows_kernel<VecT, int32_t><<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(
            static_cast<const VecT*>(key), static_cast<const VecT*>(value), static_cast<VecT*>(k_cache),
            static_cast<VecT*>(v_cache), static_cast<const int32_t*>(slot_mapping), num_tokens, row_vecs, cache_rows);
    }
    return check_launch("store_kvcache kernel launch");
}

}  // namespace

int launch_store_kvcache(const void* key, const void* value, void* k_cache, void* v_cache,
                         const void* slot_mapping, bool slot_i64, int64_t num_tokens, int64_t row_bytes,
                         int64_t cache_rows, cudaStream_t stream) {
    // Widest vector that divides the row and matches the alignment of all four base pointers.
    size_t width = 16;
    while (width > 1 && (row_bytes % static_cast<int64_t>(width) != 0 || !aligned_to(key, width) ||
                         !aligned_to(value, width) || !aligned_to(k_cache, width) || !aligned_to(v_cache, width))) {
        width >>= 1;
    }
    switch (width) {
        case 16: return launch_typed<uint4>(key, value, k_cache, v_cache, slot_mapping, slot_i64, num_tokens, row_bytes, cache_rows, stream);
        case 8: return launch_typed<uint2>(key, value, k_cache, v_cache, slot_mapping, slot_i64, num_tokens, row_bytes, cache_rows, stream);
        case 4: return launch_typed<uint32_t>(key, value, k_cache, v_cache, slot_mapping, slot_i64, num_tokens, row_bytes, cache_rows, stream);
        case 2: return launch_typed<uint16_t>(key, value, k_cache, v_cache, slot_mapping, slot_i64, num_tokens, row_bytes, cache_rows, stream);
        default: return launch_typed<uint8_t>(key, value, k_cache, v_cache, slot_mapping, slot_i64, num_tokens, row_bytes, cache_rows, stream);
    }
}

}  // namespace nvk
