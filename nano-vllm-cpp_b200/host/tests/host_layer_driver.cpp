// Runs one prefill step and one decode step at model shapes through the C++ operator layer and writes what came out,
// for a checker outside this program to compare with an independent computation (tests/test_host_layer.py).
//
//   host_layer_driver <dir>
//
// <dir>/case.txt holds "name value" lines (sizes, see read_case below); every tensor is a raw little-endian file
// <dir>/<name>.bin (16-bit elements for activations / caches, int32 for index tensors).  Steps:
//   1. prefill  TransformerAttention::forward under a prefill Context (unfused route: split_norm_rope, then
//               Attention::forward = store_kvcache + paged varlen prefill; some sequences have a cached prefix)
//               -> out_prefill.bin, k_cache_prefill.bin, v_cache_prefill.bin
//   2. decode   the same layer under a decode Context (fused route: fused_split_norm_rope_store, then
//               forward_decode_flash_only with the split-K workspace from the allocator), eagerly
//               -> out_decode.bin, k_cache_decode.bin, v_cache_decode.bin
//   3. the decode step again from the cache state after step 1, captured into a CUDA graph with an ArenaAllocator
//      supplying q, the output and the split-K workspace (no cudaMalloc under capture), then replayed twice
//               -> out_decode_graph.bin, k_cache_decode_graph.bin
//   4. the decode step once more through the UNFUSED route (split_norm_rope + Attention::forward, i.e. store_kvcache +
//      decode), as the reference runs it for fp32 models -> out_decode_unfused.bin, k_cache_decode_unfused.bin
// Exit code 0 when every step ran; the numbers are checked by the caller.
#include "kernels/attention.h"
#include "layers/attention.h"
#include "models/transformer_attention.h"
#include "utils/context.h"
#include "utils/cuda_allocator.h"
#include "utils/cuda_common.h"

#include <cuda_runtime_api.h>

#include <cstdio>
#include <fstream>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

using namespace nano_vllm;

namespace {

const Device kDev{DeviceType::kCUDA, 0};
std::string g_dir;

std::map<std::string, long long> read_case() {
    std::ifstream in(g_dir + "/case.txt");
    if (!in) throw std::runtime_error("cannot open case.txt");
    std::map<std::string, long long> kv;
    std::string name;
    long long value;
    while (in >> name >> value) kv[name] = value;
    return kv;
}

std::vector<char> read_file(const std::string& name, size_t expect_bytes) {
    std::ifstream in(g_dir + "/" + name + ".bin", std::ios::binary);
    if (!in) throw std::runtime_error("cannot open " + name + ".bin");
    std::vector<char> buf((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
    if (buf.size() != expect_bytes)
        throw std::runtime_error(name + ".bin holds " + std::to_string(buf.size()) + " bytes, expected " + std::to_string(expect_bytes));
    return buf;
}

Tensor upload(const std::string& name, const std::vector<int64_t>& sizes, ScalarType dtype) {
    CudaAllocator& alloc = CudaAllocator::instance();
    Tensor t = Tensor::empty(sizes, dtype, kDev, alloc);
    const std::vector<char> host = read_file(name, t.nbytes());
    alloc.copy_to_device_async(t.data(), host.data(), t.nbytes(), nullptr);
    alloc.synchronize_stream(nullptr);
    return t;
}

void download(const std::string& name, const Tensor& t) {
    std::vector<char> host(t.nbytes());
    CudaAllocator& alloc = CudaAllocator::instance();
    alloc.copy_to_host_async(host.data(), t.data(), t.nbytes(), nullptr);
    alloc.synchronize_stream(nullptr);
    std::ofstream out(g_dir + "/" + name + ".bin", std::ios::binary);
    out.write(host.data(), static_cast<std::streamsize>(host.size()));
}

void copy_device(const Tensor& dst, const Tensor& src) {
    throw_if_cuda_error(cudaMemcpy(dst.data(), src.data(), src.nbytes(), cudaMemcpyDeviceToDevice), "cudaMemcpy D2D");
}

}  // namespace

int main(int argc, char** argv) {
    if (argc != 2) {
        std::fprintf(stderr, "usage: %s <case directory>\n", argv[0]);
        return 2;
    }
    g_dir = argv[1];
    try {
        throw_if_cuda_error(cudaSetDevice(0), "cudaSetDevice");
        auto c = read_case();
        const int hq = static_cast<int>(c.at("num_heads")), hkv = static_cast<int>(c.at("num_kv_heads"));
        const int d = static_cast<int>(c.at("head_dim")), bs = static_cast<int>(c.at("block_size"));
        const int64_t blocks = c.at("num_blocks"), seqs = c.at("num_seqs"), total_q = c.at("total_q");
        const int64_t max_blocks = c.at("max_blocks"), batch = c.at("decode_batch");
        const int max_pos = static_cast<int>(c.at("max_position"));
        const ScalarType dt = c.at("bf16") ? ScalarType::kBFloat16 : ScalarType::kFloat16;
        const ScalarType idx = c.at("index_int64") ? ScalarType::kInt64 : ScalarType::kInt32;   // cu_seqlens / lens / tables
        const int64_t width = static_cast<int64_t>(hq + 2 * hkv) * d;
        CudaAllocator& alloc = CudaAllocator::instance();

        Tensor qw = upload("q_norm_weight", {d}, dt), kw = upload("k_norm_weight", {d}, dt);
        TransformerAttention layer(hq, hkv, d, bs, max_pos, 1.0e6f, qw, kw, 1.0e-6f, kDev, alloc);
        download("cos_sin_cache", layer.cos_sin_cache());
        Tensor k_cache = upload("k_cache", {blocks, bs, hkv, d}, dt), v_cache = upload("v_cache", {blocks, bs, hkv, d}, dt);
        layer.set_kv_cache(k_cache, v_cache);

        // ---- 1. prefill with prefix hits -------------------------------------------------------------------
        {
            Tensor qkv = upload("prefill_qkv", {total_q, width}, dt);
            Tensor pos = upload("prefill_positions", {total_q}, ScalarType::kInt32);
            set_context(true, upload("cu_seqlens_q", {seqs + 1}, idx), upload("cu_seqlens_k", {seqs + 1}, idx),
                        static_cast<int>(c.at("max_seqlen_q")), static_cast<int>(c.at("max_seqlen_k")),
                        upload("prefill_slot_mapping", {total_q}, ScalarType::kInt32), Tensor(),
                        upload("prefill_block_tables", {seqs, max_blocks}, idx));
            Tensor out = layer.forward(pos, qkv, alloc, nullptr);
            if (layer.last_forward_was_fused()) throw std::runtime_error("prefill took the fused route");
            throw_if_prefill_error(nullptr);
            download("out_prefill", out);
            download("k_cache_prefill", k_cache);
            download("v_cache_prefill", v_cache);
        }
        Tensor k_saved = Tensor::empty(k_cache.sizes(), dt, kDev, alloc), v_saved = Tensor::empty(v_cache.sizes(), dt, kDev, alloc);
        copy_device(k_saved, k_cache);
        copy_device(v_saved, v_cache);

        // ---- 2. decode, eager, fused route -----------------------------------------------------------------
        Tensor dqkv = upload("decode_qkv", {batch, width}, dt);
        Tensor dpos = upload("decode_positions", {batch}, ScalarType::kInt32);
        set_context(false, Tensor(), Tensor(), 0, 0, upload("decode_slot_mapping", {batch}, ScalarType::kInt32),
                    upload("context_lens", {batch}, idx), upload("decode_block_tables", {batch, max_blocks}, idx));
        {
            Tensor out = layer.forward(dpos, dqkv, alloc, nullptr);
            if (!layer.last_forward_was_fused()) throw std::runtime_error("decode did not take the fused route");
            download("out_decode", out);
            download("k_cache_decode", k_cache);
            download("v_cache_decode", v_cache);
        }

        // ---- 3. the same step captured into a graph with an arena allocator --------------------------------
        {
            copy_device(k_cache, k_saved);
            copy_device(v_cache, v_saved);
            ArenaAllocator arena(size_t(256) << 20, kDev, alloc);
            cudaStream_t stream = nullptr;
            throw_if_cuda_error(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "cudaStreamCreate");
            arena.reset();
            Tensor warm = layer.forward(dpos, dqkv, arena, stream);          // warm-up pass: same addresses as the capture
            throw_if_cuda_error(cudaStreamSynchronize(stream), "warm-up");
            const size_t warm_used = arena.used();
            copy_device(k_cache, k_saved);
            copy_device(v_cache, v_saved);
            arena.reset();
            cudaGraph_t graph = nullptr;
            cudaGraphExec_t exec = nullptr;
            throw_if_cuda_error(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal), "begin capture");
            Tensor out = layer.forward(dpos, dqkv, arena, stream);
            throw_if_cuda_error(cudaStreamEndCapture(stream, &graph), "end capture");
            if (arena.used() != warm_used || out.data() != warm.data()) throw std::runtime_error("arena addresses moved between passes");
            throw_if_cuda_error(cudaGraphInstantiate(&exec, graph, 0), "instantiate");
            for (int rep = 0; rep < 2; ++rep) throw_if_cuda_error(cudaGraphLaunch(exec, stream), "graph launch");
            throw_if_cuda_error(cudaStreamSynchronize(stream), "graph replay");
            download("out_decode_graph", out);
            download("k_cache_decode_graph", k_cache);
            cudaGraphExecDestroy(exec);
            cudaGraphDestroy(graph);
            cudaStreamDestroy(stream);
        }

        // ---- 4. decode through the unfused route -----------------------------------------------------------
        {
            copy_device(k_cache, k_saved);
            copy_device(v_cache, v_saved);
            Tensor q = Tensor::empty({batch, hq, d}, dt, kDev, alloc), k = Tensor::empty({batch, hkv, d}, dt, kDev, alloc);
            Tensor v = Tensor::empty({batch, hkv, d}, dt, kDev, alloc);
            split_norm_rope(dqkv, dpos, qw, kw, 1.0e-6f, layer.cos_sin_cache(), hq, hkv, d, q, k, v, nullptr);
            Tensor out = layer.attn().forward(q, k, v, alloc, nullptr);
            download("out_decode_unfused", out);
            download("k_cache_decode_unfused", k_cache);
        }
        throw_if_cuda_error(cudaDeviceSynchronize(), "final sync");
        reset_context();
    } catch (const std::exception& e) {
        std::fprintf(stderr, "host_layer_driver: %s\n", e.what());
        return 1;
    }
    std::printf("host_layer_driver: ok\n");
    return 0;
}
