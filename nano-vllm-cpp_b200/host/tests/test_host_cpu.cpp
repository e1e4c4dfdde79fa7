// CPU-only tests of the operator layer's host logic: tensor views, the step context, the metadata
// builders (expected arrays taken from the reference's tests/test_model_runner.cpp:114-280) and the
// KV-cache plan (src/engine/model_runner.cpp:388-413, :437-458).  No CUDA call is made.
#include "check.h"

#include "engine/step_metadata.h"
#include "kernels/attention.h"
#include "kernels/kvcache.h"
#include "layers/attention.h"
#include "utils/context.h"
#include "utils/tensor.h"

#include <numeric>
#include <stdexcept>

using namespace nano_vllm;

namespace {

constexpr int kBlock = 256;   // Sequence::BLOCK_SIZE of the reference

Tensor host_tensor(std::vector<float>& storage, const std::vector<int64_t>& sizes, DeviceType type = DeviceType::kCPU) {
    auto mem = Memory::make_borrowed(storage.data(), storage.size() * sizeof(float), Device{type, 0});
    return Tensor::from_memory(mem, sizes, ScalarType::kFloat32);
}

SequenceView view_of(const std::vector<int32_t>& tokens, const std::vector<int32_t>& table, int cached = 0,
                     int computed = 0, int to_process = 0) {
    SequenceView s;
    s.token_ids = tokens.data();
    s.num_tokens = static_cast<int32_t>(tokens.size());
    s.last_token = tokens.back();
    s.num_cached_tokens = cached;
    s.num_computed_tokens = computed;
    s.num_tokens_to_process = to_process;
    s.block_table = table.data();
    s.block_table_len = static_cast<int32_t>(table.size());
    return s;
}

}  // namespace

TEST_CASE(scalar_types_keep_the_abi_order) {
    CHECK_EQ(static_cast<int>(ScalarType::kFloat16), 0);
    CHECK_EQ(static_cast<int>(ScalarType::kBFloat16), 1);
    CHECK_EQ(static_cast<int>(ScalarType::kFloat32), 2);
    CHECK_EQ(static_cast<int>(ScalarType::kInt32), 3);
    CHECK_EQ(static_cast<int>(ScalarType::kInt64), 4);
    CHECK_EQ(static_cast<int>(ScalarType::kInt8), 5);
    CHECK_EQ(scalar_type_size(ScalarType::kBFloat16), size_t(2));
    CHECK_EQ(scalar_type_size(ScalarType::kInt64), size_t(8));
    CHECK_EQ(to_string(ScalarType::kBFloat16), std::string("bfloat16"));
}

TEST_CASE(tensor_views_share_memory_with_element_offsets) {
    std::vector<float> data(24);
    std::iota(data.begin(), data.end(), 0.0f);
    Tensor t = host_tensor(data, {2, 3, 4});
    CHECK(t.defined());
    CHECK(t.is_contiguous());
    CHECK_EQ(t.numel(), size_t(24));
    CHECK_EQ(t.nbytes(), size_t(96));
    CHECK_EQ(t.strides(), (std::vector<int64_t>{12, 4, 1}));
    Tensor second = t.slice(0, 1, 2);
    CHECK_EQ(second.memory_offset(), size_t(12));
    CHECK_EQ(*second.data_as<float>(), 12.0f);
    CHECK(second.is_contiguous());
    Tensor inner = t.slice(1, 1, 3);
    CHECK(!inner.is_contiguous());
    CHECK_THROWS(inner.reshape({4, 4}), std::invalid_argument);
    Tensor flat = t.reshape({6, 4});
    CHECK_EQ(flat.sizes(), (std::vector<int64_t>{6, 4}));
    CHECK_THROWS(t.reshape({5, 5}), std::invalid_argument);
    CHECK_THROWS(t.slice(3, 0, 1), std::invalid_argument);
    CHECK_THROWS(Tensor::from_memory(t.memory(), {25}, ScalarType::kFloat32), std::invalid_argument);
    Tensor at = Tensor::from_memory(t.memory(), {2, 2}, ScalarType::kFloat32, 20);
    CHECK_EQ(at.data_as<float>()[3], 23.0f);
    CHECK(!Tensor().defined());
}

TEST_CASE(context_is_set_and_reset_per_thread) {
    std::vector<float> a(4), b(4);
    Tensor cu_q = host_tensor(a, {4});
    Tensor slots = host_tensor(b, {4});
    set_context(true, cu_q, Tensor(), 3, 3, slots, Tensor(), Tensor());
    CHECK(get_context().is_prefill);
    CHECK(get_context().cu_seqlens_q.defined());
    CHECK(get_context().slot_mapping.defined());
    CHECK_EQ(get_context().max_seqlen_q, 3);
    reset_context();
    CHECK(!get_context().is_prefill);
    CHECK(!get_context().cu_seqlens_q.defined());
    CHECK(!get_context().slot_mapping.defined());
}

// tests/test_model_runner.cpp:114-180: two prompts sharing a 256-token prefix; the second one hits the cache.
TEST_CASE(prefill_arrays_with_a_prefix_cache_hit) {
    std::vector<int32_t> seq0(kBlock, 0), seq1(kBlock, 0);
    seq0.push_back(1);
    seq1.push_back(2);
    const std::vector<int32_t> table0 = {0, 1}, table1 = {0, 2};
    const StepArrays a = build_prefill_arrays({view_of(seq0, table0), view_of(seq1, table1, kBlock)}, kBlock);
    std::vector<int32_t> ids(kBlock, 0), pos(kBlock), slots(kBlock);
    std::iota(pos.begin(), pos.end(), 0);
    std::iota(slots.begin(), slots.end(), 0);
    ids.push_back(1); ids.push_back(2);
    pos.push_back(kBlock); pos.push_back(kBlock);
    slots.push_back(kBlock); slots.push_back(2 * kBlock);
    CHECK(a.is_prefill);
    CHECK_EQ(a.input_ids, ids);
    CHECK_EQ(a.positions, pos);
    CHECK_EQ(a.slot_mapping, slots);
    CHECK_EQ(a.cu_seqlens_q, (std::vector<int32_t>{0, kBlock + 1, kBlock + 2}));
    CHECK_EQ(a.cu_seqlens_k, (std::vector<int32_t>{0, kBlock + 1, 2 * kBlock + 2}));
    CHECK_EQ(a.block_tables, (std::vector<int32_t>{0, 1, 0, 2}));
    CHECK_EQ(a.max_blocks, int64_t(2));
    CHECK_EQ(a.max_seqlen_q, kBlock + 1);
    CHECK_EQ(a.max_seqlen_k, kBlock + 1);
}

// tests/test_model_runner.cpp:182-239: a fully cached prompt recomputes its last token and writes a slot in
// the block it shares with the first sequence of the same batch.
TEST_CASE(prefill_keeps_one_query_token_for_a_fully_cached_prompt) {
    const std::vector<int32_t> prompt(kBlock, 0);
    const std::vector<int32_t> table = {0};
    const StepArrays a = build_prefill_arrays({view_of(prompt, table), view_of(prompt, table, kBlock)}, kBlock);
    CHECK_EQ(a.input_ids.size(), size_t(kBlock + 1));
    CHECK_EQ(a.positions.back(), kBlock - 1);
    CHECK_EQ(a.slot_mapping.back(), kBlock - 1);
    CHECK_EQ(a.cu_seqlens_q, (std::vector<int32_t>{0, kBlock, kBlock + 1}));
    CHECK_EQ(a.cu_seqlens_k, (std::vector<int32_t>{0, kBlock, 2 * kBlock}));
    CHECK_EQ(a.block_tables, (std::vector<int32_t>{0, 0}));
}

TEST_CASE(prefill_without_cached_keys_sends_no_block_tables) {
    const std::vector<int32_t> tokens = {5, 6, 7};
    const std::vector<int32_t> table = {3};
    const StepArrays a = build_prefill_arrays({view_of(tokens, table)}, kBlock);
    CHECK(a.block_tables.empty());
    CHECK_EQ(a.slot_mapping, (std::vector<int32_t>{3 * kBlock, 3 * kBlock + 1, 3 * kBlock + 2}));
}

// src/engine/model_runner.cpp:508-512: a chunk may start anywhere; keys = everything computed so far.
TEST_CASE(chunked_prefill_uses_the_scheduler_chunk) {
    std::vector<int32_t> tokens(600);
    std::iota(tokens.begin(), tokens.end(), 100);
    const std::vector<int32_t> table = {4, 9, 2};
    const StepArrays a = build_prefill_arrays({view_of(tokens, table, 0, 300, 200)}, kBlock);
    CHECK_EQ(a.input_ids.size(), size_t(200));
    CHECK_EQ(a.input_ids.front(), 400);
    CHECK_EQ(a.positions.front(), 300);
    CHECK_EQ(a.slot_mapping.front(), 9 * kBlock + 44);
    CHECK_EQ(a.cu_seqlens_q, (std::vector<int32_t>{0, 200}));
    CHECK_EQ(a.cu_seqlens_k, (std::vector<int32_t>{0, 500}));
    CHECK_EQ(a.block_tables, table);
    // the chunk is clipped at the end of the prompt
    const StepArrays tail = build_prefill_arrays({view_of(tokens, table, 0, 500, 300)}, kBlock);
    CHECK_EQ(tail.cu_seqlens_q.back(), 100);
    CHECK_EQ(tail.cu_seqlens_k.back(), 600);
}

// tests/test_model_runner.cpp:241-280
TEST_CASE(decode_arrays_follow_the_last_token) {
    const std::vector<int32_t> tokens = {0, 7};
    const std::vector<int32_t> table = {0};
    const StepArrays a = build_decode_arrays({view_of(tokens, table)}, kBlock);
    CHECK(!a.is_prefill);
    CHECK_EQ(a.input_ids, (std::vector<int32_t>{7}));
    CHECK_EQ(a.positions, (std::vector<int32_t>{1}));
    CHECK_EQ(a.slot_mapping, (std::vector<int32_t>{1}));
    CHECK_EQ(a.context_lens, (std::vector<int32_t>{2}));
    CHECK_EQ(a.block_tables, (std::vector<int32_t>{0}));
    // a sequence that just crossed a block boundary writes offset 0 of its new block; tables are zero padded
    std::vector<int32_t> long_seq(kBlock + 1, 3);
    const std::vector<int32_t> long_table = {5, 8};
    const StepArrays b = build_decode_arrays({view_of(tokens, table), view_of(long_seq, long_table)}, kBlock);
    CHECK_EQ(b.slot_mapping, (std::vector<int32_t>{1, 8 * kBlock}));
    CHECK_EQ(b.context_lens, (std::vector<int32_t>{2, kBlock + 1}));
    CHECK_EQ(b.block_tables, (std::vector<int32_t>{0, 0, 5, 8}));
    CHECK_EQ(b.max_blocks, int64_t(2));
}

TEST_CASE(metadata_builders_reject_bad_batches) {
    CHECK_THROWS(build_prefill_arrays({}, kBlock), std::invalid_argument);
    CHECK_THROWS(build_decode_arrays({}, kBlock), std::invalid_argument);
    const std::vector<int32_t> tokens(300, 1);
    const std::vector<int32_t> short_table = {0};
    CHECK_THROWS(build_prefill_arrays({view_of(tokens, short_table)}, kBlock), std::invalid_argument);
    SequenceView empty;
    CHECK_THROWS(build_decode_arrays({empty}, kBlock), std::invalid_argument);
}

TEST_CASE(kv_cache_plan_matches_the_reference_formulas) {
    // Qwen3-8B, bf16, TP 2: 36 layers, 8 KV heads -> 4 per rank, head_dim 128
    const KvCachePlan p = plan_kv_cache(36, 256, 8, 2, 128, 2, 0, size_t(400) << 30, 0.5f, 4096, 512);
    CHECK_EQ(p.local_kv_heads, 4);
    CHECK_EQ(p.bytes_per_block, uint64_t(2) * 36 * 256 * 4 * 128 * 2);
    CHECK_EQ(p.num_blocks, int64_t(16 * 512));   // wanted = ceil(4096 / 256) * 512 (144 GiB) fits in 200 GiB
    CHECK_EQ(p.layer_elements, size_t(p.num_blocks) * 256 * 4 * 128);
    CHECK_EQ(p.k_offset(3), 3 * p.layer_elements);
    CHECK_EQ(p.v_offset(3), 36 * p.layer_elements + 3 * p.layer_elements);
    const KvCachePlan tight = plan_kv_cache(36, 256, 8, 1, 128, 2, 0, size_t(8) << 30, 0.5f, 4096, 512);
    CHECK_EQ(tight.num_blocks, int64_t((size_t(4) << 30) / tight.bytes_per_block));
    const KvCachePlan fixed = plan_kv_cache(1, 256, 1, 1, 2, 4, 4, 0, 0.9f, 4096, 8);
    CHECK_EQ(fixed.num_blocks, int64_t(4));
    CHECK_THROWS(plan_kv_cache(36, 256, 8, 3, 128, 2, 0, 1 << 30, 0.9f, 4096, 8), std::invalid_argument);
}

TEST_CASE(operators_reject_bad_operands_before_any_cuda_call) {
    std::vector<float> k(12), c(24), s(3);
    Tensor key = host_tensor(k, {3, 1, 4});
    Tensor cache = host_tensor(c, {2, 3, 1, 4});
    Tensor slots = host_tensor(s, {3});
    Tensor undefined;
    CHECK_THROWS(store_kvcache(undefined, key, cache, cache, slots), std::invalid_argument);
    CHECK_THROWS(store_kvcache(key, key, cache, cache, slots), std::invalid_argument);          // not on CUDA
    Tensor dev_key = host_tensor(k, {3, 1, 4}, DeviceType::kCUDA);                              // pretend-device views:
    Tensor dev_cache = host_tensor(c, {2, 3, 1, 4}, DeviceType::kCUDA);                         // checks only, never launched
    Tensor dev_slots = host_tensor(s, {3}, DeviceType::kCUDA);
    CHECK_THROWS(store_kvcache(dev_key, dev_key, dev_cache, dev_cache, dev_slots), std::invalid_argument);   // float slots
    CHECK_THROWS(launch_prefill_attention_paged(dev_key, nullptr, dev_cache, dev_cache, nullptr, dev_slots, 1, 4, 3,
                                                1.0f, dev_key),
                 std::invalid_argument);
    CHECK_THROWS(Attention(3, 2, 4, 256), std::invalid_argument);
    CHECK_THROWS(Attention(0, 1, 4, 256), std::invalid_argument);
    Attention attention(1, 1, 4, 3);
    CHECK_THROWS(attention.set_kv_cache(cache, cache), std::invalid_argument);                  // cache not on CUDA
    CHECK_THROWS(attention.set_kv_cache_int8(cache, cache, cache, cache), std::invalid_argument);       // not on CUDA
    CHECK_THROWS(attention.set_kv_cache_int8(dev_cache, dev_cache, dev_cache, dev_cache), std::invalid_argument);   // not int8
    CHECK_THROWS(store_kvcache_int8(key, key, cache, cache, cache, cache, slots), std::invalid_argument);
    CHECK_THROWS(store_kvcache_int8(dev_key, dev_key, dev_cache, dev_cache, dev_cache, dev_cache, dev_slots), std::invalid_argument);
}

int main() { return check::run_all(); }
