// Per-step attention metadata and KV-cache layout: the part of the reference's ModelRunner that feeds
// the attention path (src/engine/model_runner.cpp:355-475 allocate_kv_cache, :482-562 prepare_prefill,
// :564-632 prepare_decode, :748-769 build_block_tables).
//
// The array construction is pure host code (build_prefill_arrays / build_decode_arrays) so that it can
// be checked without a GPU; StepUploader then ships ALL arrays of a step in one pinned staging block
// and one host-to-device copy (the reference issues five to six small copies per prefill step) and
// publishes them through set_context().
#pragma once

#include "utils/cuda_allocator.h"
#include "utils/tensor.h"

#include <cstdint>
#include <memory>
#include <vector>

namespace nano_vllm {

// The fields of the reference's Sequence (include/engine/sequence.h:17-58) the builders read.
struct SequenceView {
    const int32_t* token_ids = nullptr;
    int32_t num_tokens = 0;
    int32_t last_token = -1;
    int32_t num_cached_tokens = 0;       // prefix-cache hit, multiple of the block size
    int32_t num_computed_tokens = 0;     // chunked prefill watermark
    int32_t num_tokens_to_process = 0;   // chunk size set by the scheduler (0 = legacy / decode)
    const int32_t* block_table = nullptr;
    int32_t block_table_len = 0;
};

struct StepArrays {
    bool is_prefill = false;
    std::vector<int32_t> input_ids, positions;
    std::vector<int32_t> cu_seqlens_q, cu_seqlens_k;   // prefill
    std::vector<int32_t> slot_mapping;
    std::vector<int32_t> context_lens;                 // decode
    std::vector<int32_t> block_tables;                 // [num_seqs, max_blocks] zero padded; empty = none
    int64_t max_blocks = 0;
    int max_seqlen_q = 0, max_seqlen_k = 0;
};

// slot = block_table[t / block_size] * block_size + t % block_size for every token of the chunk;
// cu_seqlens_k counts all keys attended so far; block tables only when some sequence has keys beyond
// its new tokens (prefix hit or later chunk), exactly as the reference decides (model_runner.cpp:548-551).
StepArrays build_prefill_arrays(const std::vector<SequenceView>& seqs, int block_size);

// input = last token, position = len - 1, context_len = len, slot of the last token; block tables padded
// to the longest table of the batch.
StepArrays build_decode_arrays(const std::vector<SequenceView>& seqs, int block_size);

// KV-cache sizing and per-layer slicing of one [2, L, blocks, block_size, Hkv / tp, D] allocation.
struct KvCachePlan {
    int num_layers = 0, block_size = 0, local_kv_heads = 0, head_dim = 0;
    int64_t num_blocks = 0;
    uint64_t bytes_per_block = 0;      // K and V of all layers for one block
    size_t layer_elements = 0;         // elements of one layer's K (or V) cache
    size_t kind_elements = 0;          // offset of the V half, in elements
    size_t k_offset(int layer) const { return static_cast<size_t>(layer) * layer_elements; }
    size_t v_offset(int layer) const { return kind_elements + static_cast<size_t>(layer) * layer_elements; }
};
KvCachePlan plan_kv_cache(int num_layers, int block_size, int num_kv_heads, int tensor_parallel_size, int head_dim,
                          size_t element_size, int64_t configured_blocks, size_t free_bytes, float gpu_memory_utilization,
                          int max_model_len, int max_num_seqs);

struct KvCache {
    Tensor storage;                 // [2, L, blocks, block_size, Hkv_local, D], zero filled
    std::vector<Tensor> k, v;       // per-layer views [blocks, block_size, Hkv_local, D]
};
KvCache allocate_kv_cache(const KvCachePlan& plan, ScalarType dtype, Device device, DeviceAllocator& allocator,
                          cudaStream_t stream = nullptr);

struct ModelInputs {
    Tensor input_ids;
    Tensor positions;
};

class StepUploader {
public:
    StepUploader(DeviceAllocator& allocator, Device device);
    ~StepUploader();
    StepUploader(const StepUploader&) = delete;
    StepUploader& operator=(const StepUploader&) = delete;

    // One staging copy + one cudaMemcpyAsync; every returned tensor is a view of one device block.
    // Also calls set_context() for the calling thread.
    ModelInputs upload(const StepArrays& arrays, cudaStream_t stream = nullptr);

private:
    struct Staging;
    DeviceAllocator& allocator_;
    Device device_;
    std::unique_ptr<Staging> staging_[2];   // alternate so that a copy still in flight is never overwritten
    int next_ = 0;
};

}  // namespace nano_vllm
