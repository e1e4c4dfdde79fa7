// CUDA error helpers, caching allocator, pinned buffer and the per-thread step context
// (interfaces: utils/cuda_common.h, utils/cuda_allocator.h, utils/context.h).
#include "utils/context.h"
#include "utils/cuda_allocator.h"
#include "utils/cuda_common.h"

#include <cuda_runtime_api.h>

#include <stdexcept>
#include <string>

namespace nano_vllm {

// ---- error helpers --------------------------------------------------------------------------------
std::string cuda_error_string(cudaError_t status) { return cudaGetErrorString(status); }

void throw_if_cuda_error(cudaError_t status, const char* context) {
    if (status == cudaSuccess) return;
    throw std::runtime_error(std::string(context) + ": " + cuda_error_string(status));
}

// ---- CudaAllocator --------------------------------------------------------------------------------
namespace {

// Runs `fn` with `device_index` current and restores the caller's device afterwards.
template <typename Fn>
void with_device(int device_index, Fn&& fn) {
    int previous = 0;
    throw_if_cuda_error(cudaGetDevice(&previous), "cudaGetDevice");
    if (previous != device_index) throw_if_cuda_error(cudaSetDevice(device_index), "cudaSetDevice");
    try {
        fn();
    } catch (...) {
        if (previous != device_index) cudaSetDevice(previous);
        throw;
    }
    if (previous != device_index) throw_if_cuda_error(cudaSetDevice(previous), "cudaSetDevice");
}

}  // namespace

CudaAllocator& CudaAllocator::instance() {
    static CudaAllocator allocator;
    return allocator;
}

// 512-byte granules up to 1 MiB, 2 MiB granules above: few distinct buckets, bounded waste.
size_t CudaAllocator::bucket_for(size_t bytes) {
    if (bytes == 0) bytes = 1;
    const size_t granule = bytes <= (size_t(1) << 20) ? 512 : (size_t(2) << 20);
    return (bytes + granule - 1) / granule * granule;
}

Memory::Ptr CudaAllocator::allocate(size_t bytes, Device device) {
    if (device.type != DeviceType::kCUDA) throw std::invalid_argument("CudaAllocator only serves CUDA devices");
    const size_t bucket = bucket_for(bytes);
    void* ptr = nullptr;
    {
        std::lock_guard<std::mutex> lock(mutex_);
        auto it = free_lists_.find({device.index, bucket});
        if (it != free_lists_.end() && !it->second.empty()) {
            ptr = it->second.back();
            it->second.pop_back();
        }
    }
    if (ptr == nullptr) {
        with_device(device.index, [&] { throw_if_cuda_error(cudaMalloc(&ptr, bucket), "cudaMalloc"); });
    }
    const int index = device.index;
    return Memory::make_owned(ptr, bytes, device, [this, index, bucket](void* p) { recycle(index, bucket, p); });
}

void CudaAllocator::recycle(int device_index, size_t bucket, void* ptr) {
    std::lock_guard<std::mutex> lock(mutex_);
    free_lists_[{device_index, bucket}].push_back(ptr);
}

void CudaAllocator::trim() {
    std::lock_guard<std::mutex> lock(mutex_);
    for (auto& entry : free_lists_) {
        const int index = entry.first.first;
        for (void* ptr : entry.second) {
            with_device(index, [&] { cudaFree(ptr); });
        }
        entry.second.clear();
    }
}

void CudaAllocator::memset_async(void* ptr, int value, size_t bytes, cudaStream_t stream) const {
    throw_if_cuda_error(cudaMemsetAsync(ptr, value, bytes, stream), "cudaMemsetAsync");
}

void CudaAllocator::copy_to_device_async(void* dst, const void* src, size_t bytes, cudaStream_t stream) const {
    throw_if_cuda_error(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream), "cudaMemcpyAsync H2D");
}

void CudaAllocator::copy_to_host_async(void* dst, const void* src, size_t bytes, cudaStream_t stream) const {
    throw_if_cuda_error(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, stream), "cudaMemcpyAsync D2H");
}

void CudaAllocator::synchronize_stream(cudaStream_t stream) const {
    throw_if_cuda_error(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
}

// ---- ArenaAllocator -------------------------------------------------------------------------------
ArenaAllocator::ArenaAllocator(size_t capacity, Device device, DeviceAllocator& delegate)
    : arena_(delegate.allocate(capacity, device)), device_(device), delegate_(delegate) {}

Memory::Ptr ArenaAllocator::allocate(size_t bytes, Device device) {
    if (device != device_) throw std::invalid_argument("ArenaAllocator serves one device only");
    const size_t rounded = (bytes + 255) / 256 * 256;
    if (offset_ + rounded > arena_->bytes())
        throw std::runtime_error("ArenaAllocator: " + std::to_string(offset_ + rounded) + " bytes needed, " +
                                 std::to_string(arena_->bytes()) + " reserved");
    void* ptr = static_cast<char*>(arena_->data()) + offset_;
    offset_ += rounded;
    if (offset_ > high_water_) high_water_ = offset_;
    return Memory::make_borrowed(ptr, bytes, device_);
}

void ArenaAllocator::memset_async(void* ptr, int value, size_t bytes, cudaStream_t stream) const {
    delegate_.memset_async(ptr, value, bytes, stream);
}
void ArenaAllocator::copy_to_device_async(void* dst, const void* src, size_t bytes, cudaStream_t stream) const {
    delegate_.copy_to_device_async(dst, src, bytes, stream);
}
void ArenaAllocator::copy_to_host_async(void* dst, const void* src, size_t bytes, cudaStream_t stream) const {
    delegate_.copy_to_host_async(dst, src, bytes, stream);
}
void ArenaAllocator::synchronize_stream(cudaStream_t stream) const { delegate_.synchronize_stream(stream); }

// ---- PinnedHostBuffer -----------------------------------------------------------------------------
PinnedHostBuffer::PinnedHostBuffer(size_t bytes) : bytes_(bytes) {
    if (bytes_ > 0) throw_if_cuda_error(cudaMallocHost(&data_, bytes_), "cudaMallocHost");
}

PinnedHostBuffer::~PinnedHostBuffer() {
    if (data_ != nullptr) cudaFreeHost(data_);
}

PinnedHostBuffer::PinnedHostBuffer(PinnedHostBuffer&& other) noexcept : data_(other.data_), bytes_(other.bytes_) {
    other.data_ = nullptr;
    other.bytes_ = 0;
}

PinnedHostBuffer& PinnedHostBuffer::operator=(PinnedHostBuffer&& other) noexcept {
    if (this != &other) {
        if (data_ != nullptr) cudaFreeHost(data_);
        data_ = other.data_;
        bytes_ = other.bytes_;
        other.data_ = nullptr;
        other.bytes_ = 0;
    }
    return *this;
}

// ---- Context --------------------------------------------------------------------------------------
namespace {
thread_local Context t_context;   // one per host thread = one per tensor-parallel rank
}

Context& get_context() { return t_context; }

void set_context(const Context& context) { t_context = context; }

void set_context(bool is_prefill, const Tensor& cu_seqlens_q, const Tensor& cu_seqlens_k, int max_seqlen_q,
                 int max_seqlen_k, const Tensor& slot_mapping, const Tensor& context_lens, const Tensor& block_tables) {
    Context& c = t_context;
    c.is_prefill = is_prefill;
    c.cu_seqlens_q = cu_seqlens_q;
    c.cu_seqlens_k = cu_seqlens_k;
    c.max_seqlen_q = max_seqlen_q;
    c.max_seqlen_k = max_seqlen_k;
    c.slot_mapping = slot_mapping;
    c.context_lens = context_lens;
    c.block_tables = block_tables;
}

void reset_context() { t_context = Context{}; }

}  // namespace nano_vllm
