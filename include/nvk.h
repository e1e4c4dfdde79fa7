/*
 * nvk.h -- C ABI of the B200 (sm_100a) attention / paged-KV kernels.
 *
 * Every entry point takes plain device pointers and sizes, enqueues its work on the given
 * CUDA stream of the CURRENT device and returns without synchronising.  No entry point
 * allocates, frees, synchronises or reads device data on the host; nvk_store_kvcache,
 * nvk_fused_split_norm_rope_store, nvk_decode_attention_paged and nvk_prefill_attention_varlen
 * may therefore be recorded into a CUDA graph.  Device-side behaviour on bad data follows the
 * reference: invalid slots are skipped, empty contexts produce zero rows, block-table entries
 * beyond ceil(len / block_size) are never dereferenced (and ids outside the cache read as 0).
 *
 * Return value: NVK_OK, or an error code; nvk_last_error() then returns a thread-local
 * message.  The C++ operator layer maps NVK_ERR_INVALID_ARGUMENT / NVK_ERR_UNSUPPORTED to
 * std::invalid_argument and NVK_ERR_CUDA to std::runtime_error, which is the reference's
 * error convention (src/kernels/kvcache.cu:160-178, src/utils/cuda_common.cpp:39-43).
 *
 * dtype codes follow the reference's ScalarType order (include/utils/tensor.h:21-28).
 * The stream argument is a cudaStream_t passed as void* (NULL = legacy default stream).
 *
 * Index tensors (slot_mapping, context_lens, block_tables, cu_seqlens_q, cu_seqlens_k) are passed as
 * `const void*` plus a dtype code, NVK_I32 or NVK_I64, one code per tensor: the reference's kernels take
 * either width for each of them independently (src/kernels/attention.cu:644-660, :708-735,
 * src/kernels/kvcache.cu:160).
 */
#ifndef NVK_H
#define NVK_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NVK_OK 0
#define NVK_ERR_INVALID_ARGUMENT 1
#define NVK_ERR_CUDA 2
#define NVK_ERR_UNSUPPORTED 3

#define NVK_F16 0
#define NVK_BF16 1
#define NVK_F32 2
#define NVK_I32 3
#define NVK_I64 4
#define NVK_I8 5

/* ABI revision of this header. */
int nvk_abi_version(void);

/* Message of the last failing call made by the calling thread ("" if none). */
const char* nvk_last_error(void);

/*
 * Replaces nano_vllm::store_kvcache (include/kernels/kvcache.h:7-12; kernels
 * src/kernels/kvcache.cu:19-47 and :53-80).
 *   key, value        [num_tokens, row_elems] contiguous, `dtype` in {F16, BF16, F32}
 *   k_cache, v_cache  [cache_rows, row_elems], same dtype
 *   slot_mapping      [num_tokens] of `slot_dtype` in {I32, I64}
 * cache row slot_mapping[t] receives row t; rows with slot < 0 or slot >= cache_rows are
 * skipped.  Pure byte copy (bit-exact).  num_tokens must be >= 1 (the reference throws on an
 * empty slot_mapping, kvcache.cu:164-167).
 */
int nvk_store_kvcache(const void* key, const void* value, void* k_cache, void* v_cache,
                      const void* slot_mapping, int slot_dtype, int64_t num_tokens,
                      int64_t row_elems, int64_t cache_rows, int dtype, void* stream);

/*
 * Replaces nano_vllm::fused_split_norm_rope_store (include/kernels/split_qkv.h:22-33; kernel
 * src/kernels/split_qkv.cu:62-154): split packed qkv rows, per-head RMSNorm of q and k
 * (fp32, eps inside the rsqrt, weight in model dtype), neox RoPE from the fp32 table
 * cos_sin_cache [max_positions, head_dim] = [cos | sin] (rows outside [0, max_positions) stay
 * un-rotated), q -> q_out [rows, Hq, D], k and v -> cache row slot_mapping[row] when that slot
 * is >= 0 (and < cache_rows: the reference checks only the lower bound, writing out of bounds
 * otherwise).  dtype in {F16, BF16}; positions and slot_mapping are int32.  head_dim in {64, 128,
 * 256}; every tensor (the table included) starts on a 16-byte boundary.
 * Two forms serve the unfused route of the reference's TransformerAttention::forward
 * (src/models/transformer.cpp:144-153: split_qkv, optional q / k norm, rotary) with the same kernel:
 *   slot_mapping == NULL                   k and v of row r go to row r of k_cache / v_cache, which are then plain
 *                                          [rows, Hkv, D] tensors (cache_rows = rows);
 *   q_norm_weight == k_norm_weight == NULL the RMSNorm is skipped (models without q / k norm).
 */
int nvk_fused_split_norm_rope_store(const void* qkv, const int32_t* positions,
                                    const void* q_norm_weight, const void* k_norm_weight,
                                    float norm_eps, const float* cos_sin_cache,
                                    int64_t max_positions, const int32_t* slot_mapping,
                                    void* k_cache, void* v_cache, int64_t cache_rows,
                                    int64_t rows, int num_q_heads, int num_kv_heads,
                                    int head_dim, void* q_out, int dtype, void* stream);

/*
 * Scratch size for nvk_decode_attention_paged (split-K partial results).  Depends only on
 * host-known sizes, never on context_lens, so the value is stable across graph replays.
 */
size_t nvk_decode_attention_workspace_bytes(int64_t batch, int num_heads, int num_kv_heads,
                                            int head_dim, int64_t max_blocks, int block_size);

/*
 * Replaces nano_vllm::launch_decode_attention_paged (include/kernels/attention.h:31-41; kernel
 * src/kernels/attention.cu:313-405) and flash_attn_decode_kvcache
 * (include/kernels/flash_attn.h:39-50).
 *   query, output   [batch, num_heads, head_dim]
 *   k_cache,v_cache [num_cache_blocks, block_size, num_kv_heads, head_dim]
 *   context_lens    [batch] int32 / int64 (includes the token being generated)
 *   block_tables    [batch, max_blocks] int32 / int64, zero padded
 *   out[b,h] = softmax(scale * q[b,h] . K[b, h*Hkv/Hq]^T) V over context_lens[b] keys; key k of
 *   sequence b lives in cache row block_tables[b][k / block_size] * block_size + k % block_size.
 *   context_lens[b] <= 0 gives a zero row; a value beyond max_blocks * block_size (more keys than the table row
 *   can address) is treated as max_blocks * block_size.
 * workspace may be NULL (then every sequence is processed by one thread block per KV head);
 * otherwise it must hold nvk_decode_attention_workspace_bytes(...) bytes, 16-byte aligned.
 * dtype F16/BF16 with head_dim 128 take the tensor-core path; other shapes and F32 take the
 * general SIMT path.
 */
int nvk_decode_attention_paged(const void* query, const void* k_cache, const void* v_cache,
                               const void* context_lens, int context_lens_dtype,
                               const void* block_tables, int block_tables_dtype,
                               int64_t batch, int64_t max_blocks, int64_t num_cache_blocks,
                               int num_heads, int num_kv_heads, int head_dim, int block_size,
                               float scale, void* output, int dtype, void* workspace,
                               size_t workspace_bytes, void* stream);

/*
 * int8 KV cache.  Replaces nano_vllm::store_kvcache_int8 (include/kernels/kvcache.h:14-24; kernel
 * src/kernels/kvcache.cu:222-296) and nano_vllm::launch_decode_attention_paged_int8
 * (include/kernels/attention.h:43-56; kernel src/kernels/attention.cu:746-842).
 *   key, value        [num_tokens, num_kv_heads, head_dim], dtype F16 / BF16 / F32
 *   k_cache, v_cache  int8 [cache_rows, num_kv_heads, head_dim]  (cache_rows = num_cache_blocks * block_size)
 *   k_scale, v_scale  fp16 [cache_rows, num_kv_heads]: scale = max(absmax / 127, 1e-10) of the head vector,
 *                     quantised value = clamp(rint(x * 127 / max(absmax, 1e-10)), -127, 127)
 * The store skips tokens whose slot is < 0 or >= cache_rows and writes caches and scales bit-identical to the
 * reference's.  The decode entry point has the semantics of nvk_decode_attention_paged with
 * k = int8 * k_scale, v = int8 * v_scale; workspace as there (same nvk_decode_attention_workspace_bytes).
 * F16 / BF16 queries with head_dim 128 take the tensor-core path, other shapes and F32 the general one.
 */
int nvk_store_kvcache_int8(const void* key, const void* value, void* k_cache, void* v_cache, void* k_scale,
                           void* v_scale, const int32_t* slot_mapping, int64_t num_tokens, int num_kv_heads,
                           int head_dim, int64_t cache_rows, int dtype, void* stream);
int nvk_decode_attention_paged_int8(const void* query, const void* k_cache, const void* v_cache,
                                    const void* k_scale, const void* v_scale, const void* context_lens,
                                    int context_lens_dtype, const void* block_tables, int block_tables_dtype,
                                    int64_t batch, int64_t max_blocks,
                                    int64_t num_cache_blocks, int num_heads, int num_kv_heads, int head_dim,
                                    int block_size, float scale, void* output, int dtype, void* workspace,
                                    size_t workspace_bytes, void* stream);

/*
 * fp8 (e4m3) KV cache.  NO COUNTERPART IN THE REFERENCE (it has the int8 cache above and names an fp8 cache as a next step);
 * the layout and the arithmetic follow the int8 cache with the range of the type:
 *   k_cache, v_cache  e4m3 bytes [cache_rows, num_kv_heads, head_dim]
 *   k_scale, v_scale  fp16 [cache_rows, num_kv_heads]: scale = max(absmax / 448, 1e-10) of the head vector,
 *                     element = e4m3(x * 448 / max(absmax, 1e-10)), round to nearest even from the fp32 product, saturating
 * key / value F16 or BF16, head_dim 64 / 128 / 256 for the store; the decode entry point has the semantics of
 * nvk_decode_attention_paged with k = e4m3 * k_scale, v = e4m3 * v_scale and takes the shapes of the tensor-core path only
 * (F16 / BF16 queries, head_dim 128, at most 8 query heads per KV head, block_size a multiple of 16); workspace as there.
 */
int nvk_store_kvcache_fp8(const void* key, const void* value, void* k_cache, void* v_cache, void* k_scale,
                          void* v_scale, const int32_t* slot_mapping, int64_t num_tokens, int num_kv_heads,
                          int head_dim, int64_t cache_rows, int dtype, void* stream);
int nvk_decode_attention_paged_fp8(const void* query, const void* k_cache, const void* v_cache,
                                   const void* k_scale, const void* v_scale, const void* context_lens,
                                   int context_lens_dtype, const void* block_tables, int block_tables_dtype,
                                   int64_t batch, int64_t max_blocks, int64_t num_cache_blocks, int num_heads,
                                   int num_kv_heads, int head_dim, int block_size, float scale, void* output,
                                   int dtype, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Same computation as nvk_decode_attention_paged for callers that cannot provide a workspace and
 * must not allocate device memory.  (No counterpart in the reference: its decode entry point simply
 * has no scratch.)  Typical callers: a wrapper with the reference's launch_decode_attention_paged
 * signature, which has no allocator argument; an engine that has already handed all free HBM to
 * its KV-cache pool; a serving loop or plug-in that is forbidden to call cudaMalloc after start-up.
 *
 * The split-K partial results go to a 32 MiB array that is part of this library's device code, so
 * every GPU that uses the library keeps those 32 MiB reserved until the process exits.  The call
 * performs no cudaMalloc / cudaFree and uses no allocating library routine.
 *   - Limit: nvk_decode_attention_workspace_bytes(...) for the given sizes must be <= 32 MiB
 *     (e.g. batch 256 x 32 heads x 4 splits = 16.9 MB); larger problems are rejected with
 *     NVK_ERR_INVALID_ARGUMENT and nothing is launched.
 *   - The first call on each device looks the array's address up (cudaGetSymbolAddress) with that
 *     device current; make that first call during start-up, before any stream capture.
 *   - All calls on one device share the array, and it keeps whatever the previous call left in it.
 *     The kernels overwrite every entry they later read, so no clearing is needed, but two calls
 *     whose kernels overlap on the GPU (different streams) race on it: serialise them.
 */
size_t nvk_decode_attention_static_scratch_bytes(void);   /* the limit above, for callers that size their batches by it */
int nvk_decode_attention_paged_static(const void* query, const void* k_cache, const void* v_cache,
                                      const void* context_lens, int context_lens_dtype,
                                      const void* block_tables, int block_tables_dtype,
                                      int64_t batch, int64_t max_blocks, int64_t num_cache_blocks,
                                      int num_heads, int num_kv_heads, int head_dim, int block_size,
                                      float scale, void* output, int dtype, void* stream);

/*
 * Tensor-parallel all-reduce (sum, F16 / BF16) over NVLink peer memory for the latency-bound messages of a decode
 * step.  Replaces, for that case, NcclTensorParallelCommunicator::all_reduce_sum
 * (src/utils/tensor_parallel.cpp:331-353), called after o_proj and down_proj (src/layers/linear.cpp:315-318).
 *
 * One process per GPU.  Every rank owns a STAGING area of at least nvk_tp_allreduce_stage_bytes(largest count) bytes
 * and a FLAG area of nvk_tp_allreduce_flag_bytes() bytes, both zeroed once.  The staging areas are mapped into every
 * process (cudaIpc* or equivalent; plain peer mappings, no multicast); stage_ptrs is a HOST array of `world` device
 * pointers as mapped in the calling process (32-byte aligned), index = rank, and stage_bytes the size every one of them
 * has (the same on all ranks).  The addend `in`, the result `out` and the flag area are ordinary device memory of the calling
 * rank: peers never access them, so a GEMM may write `in` and read `out` in place.  Every rank calls with the same
 * count (a multiple of 8 * world elements) in the same order; the result, identical on all ranks, is in `out` when the
 * launch completes.  The launch may be captured in a CUDA graph.
 *
 * Failure contract.  A kernel waits only for data, and every wait is bounded (nvk_tp_allreduce_set_wait_limit_ms;
 * 10 s unless set -- far above any skew between healthy ranks, since a rank that is merely late must not be taken
 * for dead).  When a wait runs out the rank's error word becomes non-zero and STAYS so: every later launch of that
 * rank returns at once without touching data, and its peers run into one time-out themselves.  nvk_tp_allreduce_status
 * copies the word to the host (synchronises the stream): 0 = ok, 1 = an addend slice never arrived, 2 = a result slice
 * never arrived.  A non-zero status means that the group is out of step and that every result since the last zero
 * status is invalid.  To reuse the buffers all ranks must, under a host-side barrier and with no launch in flight,
 * zero their staging areas and call nvk_tp_allreduce_reset (zeroes the flag area: error word and launch counter).
 */
#define NVK_TP_MAX_RANKS 8
size_t nvk_tp_allreduce_flag_bytes(void);
size_t nvk_tp_allreduce_stage_bytes(int64_t max_count);
void nvk_tp_allreduce_set_wait_limit_ms(int ms);   /* process-wide; applies to launches made (or captured) afterwards */
int nvk_tp_allreduce(const void* in, void* out, void* const* stage_ptrs, size_t stage_bytes, void* flags, int rank,
                     int world, int64_t count, int dtype, void* stream);
int nvk_tp_allreduce_status(const void* flags, void* stream, int* status);
int nvk_tp_allreduce_reset(void* flags, void* stream);
/*
 * The same all-reduce with the residual add and the RMSNorm that follow it in a decoder layer folded in:
 *   h_new = residual + bf16(sum over ranks of addend)   -> out   [rows, cols]
 *   x     = rmsnorm(h_new, eps) * weight                -> norm  [rows, cols]
 * rows must be a multiple of world (a rank reduces rows / world whole rows), cols a multiple of 8, at most 8192.
 * residual [rows, cols] is the caller's own copy (identical on all ranks; it may be `out` itself), weight [cols].
 * Rounding follows the unfused sequence (sum rounded to the 16-bit type, added to the residual in it, normalised from the
 * rounded h_new), so results agree with all-reduce + add + rms_norm to within one unit of the 16-bit type.
 */
int nvk_tp_allreduce_add_rmsnorm(const void* in, void* out, void* norm, void* const* stage_ptrs, size_t stage_bytes,
                                 void* flags, const void* residual, const void* weight, float eps, int rank, int world,
                                 int rows, int cols, int dtype, void* stream);
/*
 * The same two operations through the NVSwitch (multimem.ld_reduce / multimem.st on an NVLink multicast object): a rank
 * pulls the sum of its rows / world rows from the switch and stores the result rows once, the switch copying them to every
 * rank, so the bytes on a rank's links do not grow with the number of ranks.  No counterpart in the reference (it calls
 * ncclAllReduce, src/utils/tensor_parallel.cpp:331-353).
 *
 * mc_in and mc_out are MULTICAST addresses of the addend and the result: the buffers lie at the same offset in every rank's part of one
 * symmetric allocation bound to a multicast object (cuMulticastCreate / cuMulticastBindMem, or a library that does it);
 * every rank writes its addend through its ordinary mapping of that memory before the call and reads the result rows
 * through it afterwards.  In the fused form `out` is that ordinary mapping of the result buffer (the kernel reads the rows
 * its peers broadcast from it; only result rows cross the wire) and `norm` [rows, cols] ordinary memory of the calling rank
 * that receives the RMSNorm of every row.  signal_ptrs is a HOST array of `world` device pointers: every rank's signal area of
 * nvk_tp_allreduce_signal_bytes() bytes (plain peer mappings, zeroed once), index = rank.  flags is a private flag area
 * as above (nvk_tp_allreduce_flag_bytes, nvk_tp_allreduce_status, nvk_tp_allreduce_reset; a reset also needs the signal areas
 * zeroed); residual and weight are the caller's own memory.  rows a multiple of world, cols a multiple of 8, at most 8192.
 * Sums are accumulated in fp32 inside the switch in an order the hardware chooses and rounded once to the 16-bit type, so
 * results agree with the other entry points to within one unit of that type, and are identical on all ranks.
 * Every wait is bounded and the error word sticky, as above.  A process must not exit while its peers still run launches
 * on the multicast object.
 */
size_t nvk_tp_allreduce_signal_bytes(void);
int nvk_tp_allreduce_multimem(const void* mc_in, void* mc_out, void* const* signal_ptrs, void* flags, int rank, int world,
                              int rows, int cols, int dtype, void* stream);
int nvk_tp_allreduce_add_rmsnorm_multimem(const void* mc_in, void* mc_out, const void* out, void* norm, void* const* signal_ptrs, void* flags,
                                          const void* residual, const void* weight, float eps, int rank, int world, int rows,
                                          int cols, int dtype, void* stream);
/*
 * All `world` ranks of either form on ONE device in one cooperative launch: in_ptrs / out_ptrs / stage_ptrs /
 * flag_ptrs (and, for the fused form, norm_ptrs / residual_ptrs; pass norm_ptrs == NULL for the plain sum) are host
 * arrays of `world` pointers into the current device's memory, one buffer set per rank.  Same kernels, same protocol,
 * same results as `world` processes; the counterpart of the reference's InProcessTensorParallelCommunicator
 * (src/utils/tensor_parallel.cpp:165-277), for tests and single-GPU bring-up.
 */
int nvk_tp_allreduce_inprocess(const void* const* in_ptrs, void* const* out_ptrs, void* const* norm_ptrs,
                               void* const* stage_ptrs, size_t stage_bytes, void* const* flag_ptrs,
                               const void* const* residual_ptrs, const void* weight, float eps, int world, int rows,
                               int cols, int dtype, void* stream);

/*
 * Replaces nano_vllm::launch_prefill_attention_dense / launch_prefill_attention_paged
 * (include/kernels/attention.h:7-29; kernels src/kernels/attention.cu:114-202 and :205-302)
 * and flash_attn_varlen_fwd (include/kernels/flash_attn.h:15-26).
 *   query, output  [total_q, num_heads, head_dim]
 *   dense keys:    key, value [total_k, num_kv_heads, head_dim], block_tables == NULL
 *   paged keys:    k_cache, v_cache [num_cache_blocks, block_size, num_kv_heads, head_dim] and
 *                  block_tables [num_seqs, max_blocks] int32 / int64; key/value ignored
 *   cu_seqlens_q, cu_seqlens_k  [num_seqs + 1] int32 / int64; both NULL (dense only) = one sequence
 * Causal mask, bottom-right aligned: query i of a sequence sees keys
 * 0 .. (k_len - q_len) + i  (attention.cu:147, :244); rows with no visible key are zero.
 * max_seqlen_q may be 0 when unknown.
 * The tensor-core path (F16 / BF16, head_dim 128, an even number of query heads per KV head) runs persistent
 * blocks that take their work from a counter inside the library; 64 such counters rotate, one per call, and the
 * last block of a launch re-arms its counter.  So up to 64 prefill launches may be in flight on one device at a
 * time (any streams); a CUDA graph that captured the call keeps the counter it was given, and graphs replayed
 * concurrently on one device must hold different ones (capture them back to back and they do).
 *
 * Every wait inside the tensor-core kernels is bounded (about two seconds).  A block whose wait runs out stops, leaves
 * its output rows unwritten and records which wait it was in a per-device error word; the launch itself still
 * completes.  nvk_prefill_status synchronises `stream`, copies that word to *status (0 = every launch since the last
 * call completed normally) and clears it.  The C++ layer turns a non-zero word into std::runtime_error.
 */
int nvk_prefill_status(void* stream, int* status);
int nvk_prefill_attention_varlen(const void* query, const void* key, const void* value,
                                 const void* k_cache, const void* v_cache,
                                 const void* cu_seqlens_q, int cu_seqlens_q_dtype,
                                 const void* cu_seqlens_k, int cu_seqlens_k_dtype,
                                 const void* block_tables, int block_tables_dtype, int64_t num_seqs, int64_t total_q,
                                 int64_t total_k, int64_t max_blocks, int64_t num_cache_blocks,
                                 int max_seqlen_q, int num_heads, int num_kv_heads, int head_dim,
                                 int block_size, float scale, void* output, int dtype,
                                 void* stream);

/*
 * One continuous-batching step that holds BOTH prefill sequences and decode sequences, as one launch (plus the small
 * merge of the decode splits).  The reference never mixes the two in a step (src/engine/scheduler.cpp:65-67, :103-106)
 * and names the mixed step as its next one (docs/interview_star.md:54); with two launches the tensor-bound prefill
 * part and the HBM-bound decode part run one after the other and every SM idles at the boundary.  Here the persistent
 * blocks of the prefill kernel also take the decode kernel's (KV head, split, sequence) items from a second queue:
 * `prefill_blocks` of them start with the prefill items, the rest with the decode items, every block finishes with
 * what is left of the other kind.  Results are those of nvk_prefill_attention_varlen on the prefill rows and of
 * nvk_decode_attention_paged (same split policy, so the same bits) on the decode rows.
 *   prefill part   p_query / p_output [total_q, Hq, D]; keys dense (p_key, p_value [total_k, Hkv, D], p_block_tables
 *                  NULL) or paged through p_block_tables [num_seqs, p_max_blocks]; cu_seqlens_* as in
 *                  nvk_prefill_attention_varlen
 *   decode part    d_query / d_output [batch, Hq, D], context_lens [batch], d_block_tables [batch, d_max_blocks]
 *   both read      k_cache, v_cache [num_cache_blocks, block_size, Hkv, D] (new K / V already stored)
 * workspace: nvk_decode_attention_workspace_bytes(batch, ...) bytes, required.  prefill_blocks: how many of the
 * device's SMs start on the prefill part (the caller's scheduler knows both parts' sizes; about
 * SMs * t_prefill / (t_prefill + t_decode)); 0 = the library's estimate from the sizes it is given.
 * Supported where both single-purpose tensor-core paths are: F16 / BF16, head_dim 128, 2, 4, 6 or 8 query heads per KV
 * head, paged block sizes that are multiples of 128; NVK_ERR_UNSUPPORTED otherwise (then make the two calls).
 */
int nvk_attention_mixed_step(const void* p_query, const void* p_key, const void* p_value, const void* k_cache, const void* v_cache,
                             const void* cu_seqlens_q, int cu_seqlens_q_dtype, const void* cu_seqlens_k, int cu_seqlens_k_dtype,
                             const void* p_block_tables, int p_block_tables_dtype, int64_t num_seqs, int64_t total_q,
                             int64_t total_k, int64_t p_max_blocks, int max_seqlen_q, void* p_output, const void* d_query,
                             const void* context_lens, int context_lens_dtype, const void* d_block_tables,
                             int d_block_tables_dtype, int64_t batch, int64_t d_max_blocks, void* d_output,
                             int64_t num_cache_blocks, int num_heads, int num_kv_heads, int head_dim, int block_size, float scale,
                             int dtype, void* workspace, size_t workspace_bytes, int prefill_blocks, void* stream);

/*
 * The linears on either side of attention, as tcgen05 GEMMs whose epilogue does what follows them.  Weights are
 * [out_features, in_features] row-major (how the reference's Linear layers and its loader keep them,
 * src/layers/linear.cpp:77-140), activations [rows, in_features]; F16 / BF16, fp32 accumulation, the product rounded
 * to the 16-bit type before anything else is done with it (so the results are those of the unfused sequence to
 * within one unit of that type).  out_features must be a multiple of 128, in_features a multiple of 8, pointers
 * 16-byte aligned.  A bounded wait inside these kernels that runs out is reported by nvk_gemm_status (synchronises the
 * stream, reads and clears the device's error word; 0 = every launch completed).
 *
 * nvk_linear: out = x * weight^T and nothing else (Linear::forward without bias; it exists so that the GEMM core can
 * be tested on its own).
 *
 * nvk_qkv_linear_norm_rope_store: QKVParallelLinear::forward (src/layers/linear.cpp:348-420) followed by
 * fused_split_norm_rope_store (src/kernels/split_qkv.cu:62-154) -- the first half of
 * TransformerAttention::forward (src/models/transformer.cpp:118-139) -- as ONE launch: head_dim 128 makes a 128-column
 * tile of the product one head, so the RMSNorm, the rotation and the scatter into the paged cache happen on the
 * accumulator and the packed qkv tensor is never written.  qkv_weight [(Hq + 2 Hkv) * 128, in_features]; the other
 * arguments as in nvk_fused_split_norm_rope_store (slot_mapping NULL = rows go to rows; both norm weights NULL = no norm).
 *
 * nvk_tp_row_linear_allreduce_add_rmsnorm: RowParallelLinear::forward with its all-reduce (src/layers/linear.cpp:306-320)
 * plus the residual add and the RMSNorm that follow in the decoder layer.  The GEMM's epilogue delivers every row of
 * this rank's partial sum to the rank that reduces it -- its own rows into `addend` (scratch, [rows, out_features]), the
 * others as tagged vectors over NVLink into the owners' staging areas -- so the transfer overlaps the remaining tiles,
 * and the all-reduce kernel that follows starts with the reduction.  Buffers, contract and results as for
 * nvk_tp_allreduce_add_rmsnorm (same staging areas and flag area; calls of either kind may alternate).
 * The _inprocess form runs all ranks on one device (one GEMM launch per rank, one cooperative all-reduce launch).
 */
int nvk_linear(const void* x, const void* weight, void* out, int64_t rows, int64_t out_features, int64_t in_features, int dtype,
               void* stream);
int nvk_qkv_linear_norm_rope_store(const void* x, const void* qkv_weight, int64_t rows, int64_t in_features,
                                   const int32_t* positions, const void* q_norm_weight, const void* k_norm_weight,
                                   float norm_eps, const float* cos_sin_cache, int64_t max_positions,
                                   const int32_t* slot_mapping, void* k_cache, void* v_cache, int64_t cache_rows,
                                   int num_q_heads, int num_kv_heads, int head_dim, void* q_out, int dtype, void* stream);
int nvk_tp_row_linear_allreduce_add_rmsnorm(const void* x, const void* weight, int64_t rows, int64_t out_features,
                                            int64_t in_features, void* addend, void* out, void* norm, void* const* stage_ptrs,
                                            size_t stage_bytes, void* flags, const void* residual, const void* norm_weight,
                                            float eps, int rank, int world, int dtype, void* stream);
int nvk_tp_row_linear_allreduce_add_rmsnorm_inprocess(const void* const* x_ptrs, const void* const* weight_ptrs, int64_t rows,
                                                      int64_t out_features, int64_t in_features, void* const* addend_ptrs,
                                                      void* const* out_ptrs, void* const* norm_ptrs, void* const* stage_ptrs,
                                                      size_t stage_bytes, void* const* flag_ptrs,
                                                      const void* const* residual_ptrs, const void* norm_weight, float eps,
                                                      int world, int dtype, void* stream);
int nvk_gemm_status(void* stream, int* status);

#ifdef __cplusplus
}
#endif
#endif /* NVK_H */
