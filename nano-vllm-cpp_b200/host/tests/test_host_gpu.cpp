// GPU tests of the C++ operator layer: the reference's own known-answer cases, written against the same
// API (tests/test_tensor.cpp:411-450 store_kvcache; tests/test_layers.cpp:82-116 dense prefill, :118-153
// decode through the block table, :155-191 paged prefill with a prefix), plus the single-copy metadata
// upload and the per-layer KV-cache views.  Tolerances are the reference's (1e-5 / 1e-6, fp32).
#include "check.h"

#include "engine/step_metadata.h"
#include "kernels/attention.h"
#include "kernels/kvcache.h"
#include "layers/attention.h"
#include "utils/context.h"
#include "utils/cuda_allocator.h"
#include "utils/cuda_common.h"

#include <cuda_runtime_api.h>

#include <cmath>
#include <numeric>
#include <stdexcept>

using namespace nano_vllm;

namespace {

const Device kDev{DeviceType::kCUDA, 0};

Tensor device_floats(const std::vector<int64_t>& sizes, const std::vector<float>& values) {
    CudaAllocator& alloc = CudaAllocator::instance();
    Tensor t = Tensor::empty(sizes, ScalarType::kFloat32, kDev, alloc);
    alloc.copy_to_device_async(t.data(), values.data(), t.nbytes(), nullptr);
    alloc.synchronize_stream(nullptr);
    return t;
}

Tensor device_ints(const std::vector<int64_t>& sizes, const std::vector<int32_t>& values) {
    CudaAllocator& alloc = CudaAllocator::instance();
    Tensor t = Tensor::empty(sizes, ScalarType::kInt32, kDev, alloc);
    alloc.copy_to_device_async(t.data(), values.data(), t.nbytes(), nullptr);
    alloc.synchronize_stream(nullptr);
    return t;
}

std::vector<float> to_host(const Tensor& t) {
    std::vector<float> out(t.numel());
    CudaAllocator& alloc = CudaAllocator::instance();
    alloc.copy_to_host_async(out.data(), t.data(), t.nbytes(), nullptr);
    alloc.synchronize_stream(nullptr);
    return out;
}

std::vector<int32_t> ints_to_host(const Tensor& t) {
    std::vector<int32_t> out(t.numel());
    CudaAllocator& alloc = CudaAllocator::instance();
    alloc.copy_to_host_async(out.data(), t.data(), t.nbytes(), nullptr);
    alloc.synchronize_stream(nullptr);
    return out;
}

}  // namespace

TEST_CASE(store_kvcache_writes_slots_and_skips_padding) {
    std::vector<float> keys(12), values(12);
    std::iota(keys.begin(), keys.end(), 1.0f);
    for (size_t i = 0; i < 12; ++i) values[i] = -keys[i];
    Tensor key = device_floats({3, 1, 4}, keys), value = device_floats({3, 1, 4}, values);
    CudaAllocator& alloc = CudaAllocator::instance();
    Tensor k_cache = Tensor::zeros({2, 3, 1, 4}, ScalarType::kFloat32, kDev, alloc);
    Tensor v_cache = Tensor::zeros({2, 3, 1, 4}, ScalarType::kFloat32, kDev, alloc);
    store_kvcache(key, value, k_cache, v_cache, device_ints({3}, {2, -1, 5}));
    const std::vector<float> k = to_host(k_cache), v = to_host(v_cache);
    for (size_t i = 0; i < 24; ++i) {
        float expect = 0.0f;
        if (i >= 8 && i < 12) expect = keys[i - 8];
        if (i >= 20) expect = keys[i - 12];
        CHECK_NEAR(k[i], expect, 1e-6);
        CHECK_NEAR(v[i], -expect, 1e-6);
    }
    CHECK_THROWS(store_kvcache(key, value, k_cache, v_cache, device_ints({0}, {})), std::invalid_argument);
}

TEST_CASE(attention_prefill_matches_reference) {
    CudaAllocator& alloc = CudaAllocator::instance();
    Attention attention(1, 1, 2, 2);
    Tensor q = device_floats({3, 1, 2}, {1, 0, 0, 1, 1, 1});
    Tensor k = device_floats({3, 1, 2}, {1, 0, 0, 1, 1, 1});
    Tensor v = device_floats({3, 1, 2}, {1, 2, 3, 4, 5, 6});
    Tensor cu = device_ints({2}, {0, 3});
    set_context(true, cu, cu, 3, 3, Tensor(), Tensor(), Tensor());
    const std::vector<float> got = to_host(attention.forward(q, k, v, alloc));
    reset_context();
    const float s = 1.0f / std::sqrt(2.0f);
    const float b0 = std::exp(-s), c0 = std::exp(-s);
    const std::vector<float> expect = {1, 2, (b0 + 3) / (b0 + 1), (2 * b0 + 4) / (b0 + 1),
                                       (c0 + 3 * c0 + 5) / (2 * c0 + 1), (2 * c0 + 4 * c0 + 6) / (2 * c0 + 1)};
    for (size_t i = 0; i < expect.size(); ++i) CHECK_NEAR(got[i], expect[i], 1e-5);
}

TEST_CASE(attention_decode_reads_kv_cache) {
    CudaAllocator& alloc = CudaAllocator::instance();
    Attention attention(1, 1, 2, 2);
    attention.set_kv_cache(device_floats({2, 2, 1, 2}, {1, 0, 0, 1, 0, 0, 0, 0}),
                           device_floats({2, 2, 1, 2}, {1, 2, 3, 4, 0, 0, 0, 0}));
    Tensor q = device_floats({1, 1, 2}, {1, 1}), k = device_floats({1, 1, 2}, {1, 1}), v = device_floats({1, 1, 2}, {5, 6});
    set_context(false, Tensor(), Tensor(), 0, 0, device_ints({1}, {2}), device_ints({1}, {3}), device_ints({1, 2}, {0, 1}));
    const std::vector<float> got = to_host(attention.forward(q, k, v, alloc));
    const std::vector<float> again = to_host(attention.forward_decode_flash_only(q, alloc));   // K/V already stored
    reset_context();
    const float s = 1.0f / std::sqrt(2.0f);
    const float p0 = std::exp(s - 2 * s);
    const float e0 = (p0 * 1 + p0 * 3 + 5) / (2 * p0 + 1), e1 = (p0 * 2 + p0 * 4 + 6) / (2 * p0 + 1);
    CHECK_NEAR(got[0], e0, 1e-5);
    CHECK_NEAR(got[1], e1, 1e-5);
    CHECK_NEAR(again[0], e0, 1e-5);
    CHECK_NEAR(again[1], e1, 1e-5);
    // decode without metadata is an error, as in the reference (src/layers/attention.cpp:182-184)
    set_context(false);
    CHECK_THROWS(attention.forward(q, k, v, alloc), std::invalid_argument);
    CHECK_THROWS(attention.forward_decode_flash_only(q, alloc), std::invalid_argument);
    reset_context();
}

TEST_CASE(attention_with_int8_kv_cache_quantises_on_store_and_dequantises_in_decode) {
    // Values chosen so that quantisation is exact (absmax 127 -> scale 1): the result must equal plain attention.
    CudaAllocator& alloc = CudaAllocator::instance();
    const int D = 64;
    Attention attention(2, 1, D, 4);
    Tensor kc = Tensor::zeros({2, 4, 1, D}, ScalarType::kInt8, kDev, alloc), vc = Tensor::zeros({2, 4, 1, D}, ScalarType::kInt8, kDev, alloc);
    Tensor ks = Tensor::zeros({2, 4, 1}, ScalarType::kFloat16, kDev, alloc), vs = Tensor::zeros({2, 4, 1}, ScalarType::kFloat16, kDev, alloc);
    attention.set_kv_cache_int8(kc, vc, ks, vs);
    CHECK(attention.is_int8());
    std::vector<float> q(2 * D, 0.0f), k1(D, 0.0f), v1(D, 0.0f), k2(D, 0.0f), v2(D, 0.0f);
    q[0] = 0.01f; q[D + 1] = 0.02f;           // head 0 looks along dimension 0, head 1 along dimension 1
    k1[0] = 127.0f; k1[1] = -127.0f;
    v1[0] = 127.0f; v1[1] = 64.0f; v1[2] = -32.0f;
    v2[3] = 127.0f; v2[0] = -1.0f;            // k2 is the zero vector: scale floors to 0, every score 0
    Tensor tq = device_floats({1, 2, D}, q);
    // token 1 -> physical block 1, row 4; a single key: the output is the dequantised value row, whatever the score
    set_context(false, Tensor(), Tensor(), 0, 0, device_ints({1}, {4}), device_ints({1}, {1}), device_ints({1, 2}, {1, 0}));
    std::vector<float> got = to_host(attention.forward(tq, device_floats({1, 1, D}, k1), device_floats({1, 1, D}, v1), alloc));
    for (int h = 0; h < 2; ++h) {
        CHECK_NEAR(got[h * D + 0], 127.0f, 1e-4);
        CHECK_NEAR(got[h * D + 1], 64.0f, 1e-4);
        CHECK_NEAR(got[h * D + 2], -32.0f, 1e-4);
        CHECK_NEAR(got[h * D + 3], 0.0f, 1e-6);
    }
    // token 2 -> row 5; two keys with scores (q . k1) / sqrt(D) and 0
    set_context(false, Tensor(), Tensor(), 0, 0, device_ints({1}, {5}), device_ints({1}, {2}), device_ints({1, 2}, {1, 0}));
    got = to_host(attention.forward(tq, device_floats({1, 1, D}, k2), device_floats({1, 1, D}, v2), alloc));
    const std::vector<float> again = to_host(attention.forward_decode_flash_only(tq, alloc));
    reset_context();
    const float inv_sqrt_d = 1.0f / std::sqrt(static_cast<float>(D));
    const float s_h0 = 0.01f * 127.0f * inv_sqrt_d, s_h1 = 0.02f * -127.0f * inv_sqrt_d;
    const float scores[2] = {s_h0, s_h1};
    for (int h = 0; h < 2; ++h) {
        const float p1 = std::exp(scores[h]) / (std::exp(scores[h]) + 1.0f), p2 = 1.0f - p1;
        CHECK_NEAR(got[h * D + 0], p1 * 127.0f + p2 * -1.0f, 2e-4);
        CHECK_NEAR(got[h * D + 1], p1 * 64.0f, 2e-4);
        CHECK_NEAR(got[h * D + 3], p2 * 127.0f, 2e-4);
        CHECK_NEAR(again[h * D + 0], got[h * D + 0], 1e-6);
    }
    // float (not fp16) scales and non-int8 caches are rejected
    CHECK_THROWS(attention.set_kv_cache_int8(kc, vc, device_floats({2, 4, 1}, std::vector<float>(8)), vs), std::invalid_argument);
    CHECK_THROWS(attention.set_kv_cache_int8(device_floats({2, 4, 1, D}, std::vector<float>(8 * D)), vc, ks, vs), std::invalid_argument);
}

TEST_CASE(attention_prefill_with_prefix_cache_reads_paged_kv_cache) {
    CudaAllocator& alloc = CudaAllocator::instance();
    Attention attention(1, 1, 2, 2);
    attention.set_kv_cache(device_floats({2, 2, 1, 2}, {1, 0, 0, 1, 0, 0, 0, 0}),
                           device_floats({2, 2, 1, 2}, {1, 2, 3, 4, 0, 0, 0, 0}));
    Tensor q = device_floats({1, 1, 2}, {1, 1}), k = device_floats({1, 1, 2}, {1, 1}), v = device_floats({1, 1, 2}, {5, 6});
    set_context(true, device_ints({2}, {0, 1}), device_ints({2}, {0, 3}), 1, 3, device_ints({1}, {2}), Tensor(),
                device_ints({1, 2}, {0, 1}));
    const std::vector<float> got = to_host(attention.forward(q, k, v, alloc));
    reset_context();
    const float s = 1.0f / std::sqrt(2.0f);
    const float p0 = std::exp(s - 2 * s);
    CHECK_NEAR(got[0], (p0 * 1 + p0 * 3 + 5) / (2 * p0 + 1), 1e-5);
    CHECK_NEAR(got[1], (p0 * 2 + p0 * 4 + 6) / (2 * p0 + 1), 1e-5);
}

TEST_CASE(attention_rejects_mismatched_operands) {
    CudaAllocator& alloc = CudaAllocator::instance();
    Attention attention(2, 1, 4, 256);
    Tensor q = device_floats({1, 2, 4}, std::vector<float>(8, 1.0f));
    Tensor k = device_floats({1, 1, 4}, std::vector<float>(4, 1.0f));
    Tensor wrong_heads = device_floats({1, 2, 4}, std::vector<float>(8, 1.0f));
    set_context(true);
    CHECK_THROWS(attention.forward(q, wrong_heads, wrong_heads, alloc), std::invalid_argument);
    CHECK_THROWS(attention.forward(q.reshape({2, 4}), k, k, alloc), std::invalid_argument);
    reset_context();
}

TEST_CASE(step_uploader_ships_one_block_and_sets_the_context) {
    CudaAllocator& alloc = CudaAllocator::instance();
    StepUploader uploader(alloc, kDev);
    std::vector<int32_t> seq0(256, 0), seq1(256, 0);
    seq0.push_back(1);
    seq1.push_back(2);
    const std::vector<int32_t> t0 = {0, 1}, t1 = {0, 2};
    SequenceView a, b;
    a.token_ids = seq0.data(); a.num_tokens = 257; a.last_token = 1; a.block_table = t0.data(); a.block_table_len = 2;
    b.token_ids = seq1.data(); b.num_tokens = 257; b.last_token = 2; b.block_table = t1.data(); b.block_table_len = 2;
    b.num_cached_tokens = 256;
    const StepArrays arrays = build_prefill_arrays({a, b}, 256);
    const ModelInputs inputs = uploader.upload(arrays);
    const Context& ctx = get_context();
    CHECK(ctx.is_prefill);
    CHECK_EQ(ints_to_host(inputs.input_ids), arrays.input_ids);
    CHECK_EQ(ints_to_host(inputs.positions), arrays.positions);
    CHECK_EQ(ints_to_host(ctx.cu_seqlens_q), arrays.cu_seqlens_q);
    CHECK_EQ(ints_to_host(ctx.cu_seqlens_k), arrays.cu_seqlens_k);
    CHECK_EQ(ints_to_host(ctx.slot_mapping), arrays.slot_mapping);
    CHECK_EQ(ints_to_host(ctx.block_tables), (std::vector<int32_t>{0, 1, 0, 2}));
    CHECK_EQ(ctx.block_tables.sizes(), (std::vector<int64_t>{2, 2}));
    CHECK(inputs.input_ids.memory() == ctx.slot_mapping.memory());   // one device block, one copy
    CHECK(!ctx.context_lens.defined());
    // three decode steps in a row reuse the two staging buffers
    for (int step = 0; step < 3; ++step) {
        a.num_tokens = 258 + step;
        const StepArrays d = build_decode_arrays({a}, 256);
        uploader.upload(d);
        CHECK(!get_context().is_prefill);
        CHECK_EQ(ints_to_host(get_context().context_lens), (std::vector<int32_t>{258 + step}));
        CHECK_EQ(ints_to_host(get_context().slot_mapping), (std::vector<int32_t>{1 * 256 + 1 + step}));
    }
    reset_context();
}

TEST_CASE(kv_cache_views_are_slices_of_one_zeroed_allocation) {
    CudaAllocator& alloc = CudaAllocator::instance();
    const KvCachePlan plan = plan_kv_cache(3, 256, 2, 2, 4, 4, 4, 0, 0.9f, 4096, 8);
    const KvCache cache = allocate_kv_cache(plan, ScalarType::kFloat32, kDev, alloc);
    CHECK_EQ(cache.storage.sizes(), (std::vector<int64_t>{2, 3, 4, 256, 1, 4}));
    CHECK_EQ(cache.k.size(), size_t(3));
    CHECK_EQ(cache.k[2].sizes(), (std::vector<int64_t>{4, 256, 1, 4}));
    CHECK_EQ(cache.k[1].memory_offset(), plan.layer_elements);
    CHECK_EQ(cache.v[0].memory_offset(), 3 * plan.layer_elements);
    const std::vector<float> zeros = to_host(cache.v[2]);
    bool all_zero = true;
    for (float z : zeros) all_zero = all_zero && z == 0.0f;
    CHECK(all_zero);
}

int main() {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        std::printf("no CUDA device: GPU tests of the operator layer not run\n");
        return 77;
    }
    throw_if_cuda_error(cudaSetDevice(0), "cudaSetDevice");
    return check::run_all();
}
