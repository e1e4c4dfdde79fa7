// Step metadata builders, KV-cache planning and the single-copy uploader (interface: engine/step_metadata.h).
#include "engine/step_metadata.h"

#include "utils/context.h"
#include "utils/cuda_common.h"

#include <algorithm>
#include <cstring>
#include <stdexcept>

namespace nano_vllm {

namespace {

int blocks_for(int tokens, int block_size) { return (tokens + block_size - 1) / block_size; }

void check_sequence(const char* who, const SequenceView& s) {
    if (s.num_tokens <= 0) throw std::invalid_argument(std::string(who) + " does not support empty sequences");
    if (s.block_table == nullptr || s.block_table_len <= 0)
        throw std::invalid_argument(std::string(who) + " requires a non-empty block_table");
}

void fill_block_tables(const std::vector<SequenceView>& seqs, StepArrays& out) {
    int64_t widest = 0;
    for (const SequenceView& s : seqs) widest = std::max<int64_t>(widest, s.block_table_len);
    out.max_blocks = widest;
    out.block_tables.assign(seqs.size() * static_cast<size_t>(widest), 0);
    for (size_t row = 0; row < seqs.size(); ++row) {
        std::copy(seqs[row].block_table, seqs[row].block_table + seqs[row].block_table_len,
                  out.block_tables.begin() + static_cast<std::ptrdiff_t>(row * static_cast<size_t>(widest)));
    }
}

}  // namespace

StepArrays build_prefill_arrays(const std::vector<SequenceView>& seqs, int block_size) {
    if (seqs.empty()) throw std::invalid_argument("prepare_prefill requires at least one sequence");
    if (block_size <= 0) throw std::invalid_argument("block size must be positive");
    StepArrays out;
    out.is_prefill = true;
    out.cu_seqlens_q.push_back(0);
    out.cu_seqlens_k.push_back(0);
    for (const SequenceView& s : seqs) {
        check_sequence("prepare_prefill", s);
        if (s.token_ids == nullptr) throw std::invalid_argument("prepare_prefill requires token ids");
        if (s.block_table_len != blocks_for(s.num_tokens, block_size))
            throw std::invalid_argument("prepare_prefill requires allocated block_table entries for each logical block");
        int begin, end;
        if (s.num_tokens_to_process > 0) {               // chunk chosen by the scheduler
            begin = s.num_computed_tokens;
            end = begin + s.num_tokens_to_process;
        } else {                                          // whole prompt minus the prefix-cache hit;
            begin = std::min(s.num_cached_tokens, s.num_tokens - 1);   // a fully cached prompt recomputes its last token
            end = s.num_tokens;
        }
        end = std::min(end, s.num_tokens);
        for (int t = begin; t < end; ++t) {
            out.input_ids.push_back(s.token_ids[t]);
            out.positions.push_back(t);
            out.slot_mapping.push_back(s.block_table[t / block_size] * block_size + t % block_size);
        }
        const int q_len = end - begin, k_len = end;
        out.cu_seqlens_q.push_back(out.cu_seqlens_q.back() + q_len);
        out.cu_seqlens_k.push_back(out.cu_seqlens_k.back() + k_len);
        out.max_seqlen_q = std::max(out.max_seqlen_q, q_len);
        out.max_seqlen_k = std::max(out.max_seqlen_k, k_len);
    }
    if (out.cu_seqlens_k.back() > out.cu_seqlens_q.back()) fill_block_tables(seqs, out);
    return out;
}

StepArrays build_decode_arrays(const std::vector<SequenceView>& seqs, int block_size) {
    if (seqs.empty()) throw std::invalid_argument("prepare_decode requires at least one sequence");
    if (block_size <= 0) throw std::invalid_argument("block size must be positive");
    StepArrays out;
    out.is_prefill = false;
    for (const SequenceView& s : seqs) {
        check_sequence("prepare_decode", s);
        out.input_ids.push_back(s.last_token);
        out.positions.push_back(s.num_tokens - 1);
        out.context_lens.push_back(s.num_tokens);
        const int in_last_block = s.num_tokens - (blocks_for(s.num_tokens, block_size) - 1) * block_size;
        out.slot_mapping.push_back(s.block_table[s.block_table_len - 1] * block_size + in_last_block - 1);
    }
    fill_block_tables(seqs, out);
    return out;
}

KvCachePlan plan_kv_cache(int num_layers, int block_size, int num_kv_heads, int tensor_parallel_size, int head_dim,
                          size_t element_size, int64_t configured_blocks, size_t free_bytes, float gpu_memory_utilization,
                          int max_model_len, int max_num_seqs) {
    if (num_layers <= 0 || block_size <= 0 || num_kv_heads <= 0 || head_dim <= 0 || element_size == 0)
        throw std::invalid_argument("ModelRunner requires positive layer, block, and KV-head counts");
    if (tensor_parallel_size <= 0 || num_kv_heads % tensor_parallel_size != 0)
        throw std::invalid_argument("num_key_value_heads must be divisible by tensor_parallel_size");
    KvCachePlan plan;
    plan.num_layers = num_layers;
    plan.block_size = block_size;
    plan.local_kv_heads = num_kv_heads / tensor_parallel_size;
    plan.head_dim = head_dim;
    plan.bytes_per_block = uint64_t(2) * uint64_t(num_layers) * uint64_t(block_size) * uint64_t(plan.local_kv_heads) *
                           uint64_t(head_dim) * uint64_t(element_size);
    if (configured_blocks > 0) {
        plan.num_blocks = configured_blocks;
    } else {
        const float util = std::min(1.0f, std::max(0.0f, gpu_memory_utilization));
        const int64_t fit = static_cast<int64_t>(static_cast<long double>(free_bytes) * util /
                                                 static_cast<long double>(plan.bytes_per_block));
        const int64_t wanted = std::max<int64_t>(1, int64_t(blocks_for(max_model_len, block_size)) * max_num_seqs);
        plan.num_blocks = std::max<int64_t>(1, std::min(wanted, fit));
    }
    plan.layer_elements = static_cast<size_t>(plan.num_blocks) * block_size * plan.local_kv_heads * head_dim;
    plan.kind_elements = static_cast<size_t>(num_layers) * plan.layer_elements;
    return plan;
}

KvCache allocate_kv_cache(const KvCachePlan& plan, ScalarType dtype, Device device, DeviceAllocator& allocator,
                          cudaStream_t stream) {
    KvCache cache;
    cache.storage = Tensor::zeros({2, plan.num_layers, plan.num_blocks, plan.block_size, plan.local_kv_heads, plan.head_dim},
                                  dtype, device, allocator, stream);
    const std::vector<int64_t> view = {plan.num_blocks, plan.block_size, plan.local_kv_heads, plan.head_dim};
    for (int layer = 0; layer < plan.num_layers; ++layer) {
        cache.k.push_back(Tensor::from_memory(cache.storage.memory(), view, dtype, plan.k_offset(layer)));
        cache.v.push_back(Tensor::from_memory(cache.storage.memory(), view, dtype, plan.v_offset(layer)));
    }
    return cache;
}

// ---- StepUploader -----------------------------------------------------------------------------------
struct StepUploader::Staging {
    std::unique_ptr<PinnedHostBuffer> buffer;
    cudaEvent_t done = nullptr;
    bool in_flight = false;
};

StepUploader::StepUploader(DeviceAllocator& allocator, Device device) : allocator_(allocator), device_(device) {
    for (auto& s : staging_) s.reset(new Staging());
}

StepUploader::~StepUploader() {
    for (auto& s : staging_) {
        if (s && s->done != nullptr) cudaEventDestroy(s->done);
    }
}

ModelInputs StepUploader::upload(const StepArrays& a, cudaStream_t stream) {
    // layout of the packed block, every piece padded to 4 elements (16 bytes)
    const std::vector<int32_t>* pieces[] = {&a.input_ids, &a.positions, &a.slot_mapping, &a.cu_seqlens_q,
                                            &a.cu_seqlens_k, &a.context_lens, &a.block_tables};
    size_t offsets[7], total = 0;
    for (int i = 0; i < 7; ++i) {
        offsets[i] = total;
        total += (pieces[i]->size() + 3) / 4 * 4;
    }
    if (total == 0) throw std::invalid_argument("step has no metadata to upload");
    const size_t bytes = total * sizeof(int32_t);

    Staging& st = *staging_[next_];
    next_ ^= 1;
    if (st.in_flight) {   // the copy issued two steps ago from this buffer must have drained
        throw_if_cuda_error(cudaEventSynchronize(st.done), "cudaEventSynchronize (metadata staging)");
        st.in_flight = false;
    }
    if (!st.buffer || st.buffer->bytes() < bytes) {
        size_t cap = st.buffer ? st.buffer->bytes() : size_t(256) << 10;
        while (cap < bytes) cap *= 2;
        st.buffer.reset(new PinnedHostBuffer(cap));
    }
    if (st.done == nullptr) throw_if_cuda_error(cudaEventCreateWithFlags(&st.done, cudaEventDisableTiming), "cudaEventCreate");
    int32_t* host = static_cast<int32_t*>(st.buffer->data());
    std::memset(host, 0, bytes);
    for (int i = 0; i < 7; ++i) {
        if (!pieces[i]->empty()) std::memcpy(host + offsets[i], pieces[i]->data(), pieces[i]->size() * sizeof(int32_t));
    }
    Tensor packed = Tensor::empty({static_cast<int64_t>(total)}, ScalarType::kInt32, device_, allocator_);
    allocator_.copy_to_device_async(packed.data(), host, bytes, stream);
    throw_if_cuda_error(cudaEventRecord(st.done, stream), "cudaEventRecord (metadata staging)");
    st.in_flight = true;

    auto view = [&](int piece, std::vector<int64_t> sizes) {
        return pieces[piece]->empty() ? Tensor() : Tensor::from_memory(packed.memory(), sizes, ScalarType::kInt32, offsets[piece]);
    };
    const int64_t tokens = static_cast<int64_t>(a.input_ids.size());
    ModelInputs inputs{view(0, {tokens}), view(1, {tokens})};
    const int64_t seqs = a.is_prefill ? static_cast<int64_t>(a.cu_seqlens_q.size()) - 1
                                      : static_cast<int64_t>(a.context_lens.size());
    Tensor tables = a.block_tables.empty() ? Tensor() : view(6, {seqs, a.max_blocks});
    if (a.is_prefill) {
        set_context(true, view(3, {seqs + 1}), view(4, {seqs + 1}), a.max_seqlen_q, a.max_seqlen_k,
                    view(2, {static_cast<int64_t>(a.slot_mapping.size())}), Tensor(), tables);
    } else {
        set_context(false, Tensor(), Tensor(), 0, 0, view(2, {seqs}), view(5, {seqs}), tables);
    }
    return inputs;
}

}  // namespace nano_vllm
