// Shared declarations of the kernel library: error reporting, dtype traits and the small set
// of PTX wrappers (cp.async, ldmatrix, mma.sync, ex2) the attention kernels are written with.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstddef>
#include <cstdint>
#include <cstdio>

#include "../../include/nvk.h"

namespace nvk {

// ---- host-side error reporting -------------------------------------------------------------
// Stores a printf-formatted message for nvk_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);
// Checks cudaPeekAtLastError() right after a launch (the reference's convention,
// src/kernels/attention.cu:442); returns NVK_OK or NVK_ERR_CUDA.
int check_launch(const char* what);

inline bool aligned_to(const void* p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; }
inline size_t dtype_size(int dtype) {
    switch (dtype) {
        case NVK_F16: case NVK_BF16: return 2;
        case NVK_F32: case NVK_I32: return 4;
        case NVK_I64: return 8;
        case NVK_I8: return 1;
        default: return 0;
    }
}

// An index tensor of the boundary (cu_seqlens_*, context_lens, block_tables): int32 or int64 elements, each tensor
// on its own, as the reference's kernels accept them (src/kernels/attention.cu:644-660, :708-735).  The width is a
// launch-uniform flag read where an index is loaded; values are widened to 64 bits.
struct IndexArray {
    const void* ptr = nullptr;
    int wide = 0;   // 1 = int64 elements, 0 = int32
    IndexArray() = default;
    __host__ __device__ IndexArray(const void* p, int w) : ptr(p), wide(w) {}
    __host__ __device__ explicit operator bool() const { return ptr != nullptr; }
    __host__ __device__ bool operator==(std::nullptr_t) const { return ptr == nullptr; }
    __host__ __device__ bool operator!=(std::nullptr_t) const { return ptr != nullptr; }
    __host__ __device__ IndexArray operator+(int64_t n) const {
        return IndexArray(static_cast<const char*>(ptr) + n * (wide ? 8 : 4), wide);
    }
#ifdef __CUDACC__
    __device__ __forceinline__ int64_t operator[](int64_t i) const {
        return wide ? static_cast<const int64_t*>(ptr)[i] : static_cast<int64_t>(static_cast<const int32_t*>(ptr)[i]);
    }
#endif
};

// ---- launchers (one per .cu file) -----------------------------------------------------------
struct DecodeArgs {
    const void* q; const void* k_cache; const void* v_cache;
    IndexArray context_lens; IndexArray block_tables;
    void* out;
    int64_t batch, max_blocks, num_cache_blocks;
    int num_heads, num_kv_heads, head_dim, block_size;
    float scale;
    int dtype;
    void* workspace; size_t workspace_bytes;
    cudaStream_t stream;
};
struct DecodeInt8Args {          // 8-bit caches (int8, or e4m3 when fp8 is set) with one fp16 scale per (cache row, KV head)
    DecodeArgs base;
    const void* k_scale; const void* v_scale;
    bool fp8 = false;
};
struct PrefillArgs {
    const void* q; const void* k; const void* v;          // dense keys (k, v) or paged (caches)
    const void* k_cache; const void* v_cache;
    IndexArray cu_q; IndexArray cu_k; IndexArray block_tables;
    void* out;
    int64_t num_seqs, total_q, total_k, max_blocks, num_cache_blocks;
    int max_seqlen_q, num_heads, num_kv_heads, head_dim, block_size;
    float scale;
    int dtype;
    cudaStream_t stream;
};

int launch_store_kvcache(const void* key, const void* value, void* k_cache, void* v_cache,
                         const void* slot_mapping, bool slot_i64, int64_t num_tokens,
                         int64_t row_bytes, int64_t cache_rows, cudaStream_t stream);
int launch_fused_prologue(const void* qkv, const int32_t* positions, const void* qw, const void* kw,
                          float eps, const float* cos_sin, int64_t max_positions,
                          const int32_t* slot_mapping, void* k_cache, void* v_cache,
                          int64_t cache_rows, int64_t rows, int hq, int hkv, int d, void* q_out,
                          int dtype, cudaStream_t stream);
// General SIMT attention (any dtype of F16/BF16/F32, head_dim <= 256, any block size).
int launch_rowwise_decode(const DecodeArgs& a);
int launch_rowwise_prefill(const PrefillArgs& a);
// Tensor-core paths (F16/BF16, head_dim 128).
bool decode_mma_supported(const DecodeArgs& a);
size_t decode_mma_workspace_bytes(int64_t batch, int num_heads, int num_kv_heads, int head_dim,
                                  int64_t max_blocks, int block_size);
int launch_decode_mma(const DecodeArgs& a);
namespace dec { struct DecodeParams; }
int decode_plan(const DecodeArgs& a, dec::DecodeParams* out);
int launch_decode_merge(const dec::DecodeParams& p, int64_t batch, int dtype, cudaStream_t stream);
// Fused all-reduce launchers (tp_allreduce.cu); `pushed`: the other ranks' slices were already pushed by the GEMM
// that produced the addend (gemm_fused.cu), the kernel starts with the reduction.
void set_multimem_wait_cycles(long long cycles);   // tp_allreduce_mm.cu: the wait limit of the multimem kernels
int launch_allreduce_add_rmsnorm(const void* in, void* out, void* norm, void* const* stage_ptrs, size_t stage_bytes, void* flags,
                                 const void* residual, const void* weight, float eps, int rank, int world, int rows, int cols,
                                 int dtype, bool pushed, cudaStream_t stream);
int launch_allreduce_inprocess(const void* const* in_ptrs, void* const* out_ptrs, void* const* norm_ptrs, void* const* stage_ptrs,
                               size_t stage_bytes, void* const* flag_ptrs, const void* const* residual_ptrs, const void* weight,
                               float eps, int world, int rows, int cols, int dtype, bool pushed, cudaStream_t stream);
// One launch for a step that holds prefill sequences and decode sequences (prefill_attn_tc.cu), then the split merge.
bool mixed_step_supported(const PrefillArgs& p, const DecodeArgs& d);
int launch_mixed_step(const PrefillArgs& p, const DecodeArgs& d, int prefill_blocks);
// int8 KV cache (kv_int8.cu; tensor-core decode in decode_attn.cu)
int launch_store_int8(const void* key, const void* value, void* k_cache, void* v_cache, void* k_scale, void* v_scale,
                      const int32_t* slot_mapping, int64_t num_tokens, int num_kv_heads, int head_dim, int64_t cache_rows,
                      int dtype, cudaStream_t stream);
int launch_rowwise_decode_int8(const DecodeInt8Args& a);
bool decode_int8_mma_supported(const DecodeInt8Args& a);
int launch_decode_int8_mma(const DecodeInt8Args& a);
int launch_store_fp8(const void* key, const void* value, void* k_cache, void* v_cache, void* k_scale, void* v_scale,
                     const int32_t* slot_mapping, int64_t num_tokens, int num_kv_heads, int head_dim, int64_t cache_rows,
                     int dtype, cudaStream_t stream);
bool prefill_mma_supported(const PrefillArgs& a);
int launch_prefill_mma(const PrefillArgs& a);
// tcgen05 / TMEM / TMA path (F16/BF16, head_dim 128, paged block_size % 128 == 0).
bool prefill_tc_supported(const PrefillArgs& a);
int launch_prefill_tc(const PrefillArgs& a);

// ---- device helpers --------------------------------------------------------------------------
#ifdef __CUDACC__

template <typename T> struct ElemTraits;
template <> struct ElemTraits<__nv_bfloat16> {
    static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
    static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
        __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&p);
    }
};
template <> struct ElemTraits<__half> {
    static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
    static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
        __half2 p = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&p);
    }
};
template <> struct ElemTraits<float> {
    static __device__ __forceinline__ float to_float(float v) { return v; }
    static __device__ __forceinline__ float from_float(float v) { return v; }
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous global->shared copy that bypasses L1; src_bytes == 0 zero-fills.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// D(16x8, f32) += A(16x16) * B(16x8); A row-major, B column-major fragments.
template <typename T>
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                  uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 2^x, approximate (ex2.approx: 2 ulp, exp2(-inf) = +0).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

constexpr float kLog2e = 1.4426950408889634f;

#endif  // __CUDACC__

}  // namespace nvk
