// Device allocation interface of the operator layer (mirrors include/utils/cuda_allocator.h:13-77 of
// the reference).  Layers never call cudaMalloc themselves: outputs and scratch come from a
// DeviceAllocator so that a bump allocator can stand in while a CUDA graph is captured
// (src/engine/model_runner.cpp:57-100).
//
// Unlike the reference's CudaAllocator, the cache here is keyed by (device, bucket) and every entry
// point takes the lock, so one process can drive several GPUs from one thread per rank.
#pragma once

#include "utils/tensor.h"

#include <cstddef>
#include <map>
#include <mutex>
#include <utility>
#include <vector>

namespace nano_vllm {

class DeviceAllocator {
public:
    virtual ~DeviceAllocator() = default;
    virtual Memory::Ptr allocate(size_t bytes, Device device) = 0;
    virtual void memset_async(void* ptr, int value, size_t bytes, cudaStream_t stream) const = 0;
    virtual void copy_to_device_async(void* dst, const void* src, size_t bytes, cudaStream_t stream) const = 0;
    virtual void copy_to_host_async(void* dst, const void* src, size_t bytes, cudaStream_t stream) const = 0;
    virtual void synchronize_stream(cudaStream_t stream) const = 0;
};

// Caching cudaMalloc allocator: freed blocks return to a per-(device, bucket) free list.
class CudaAllocator final : public DeviceAllocator {
public:
    static CudaAllocator& instance();

    Memory::Ptr allocate(size_t bytes, Device device) override;
    void memset_async(void* ptr, int value, size_t bytes, cudaStream_t stream) const override;
    void copy_to_device_async(void* dst, const void* src, size_t bytes, cudaStream_t stream) const override;
    void copy_to_host_async(void* dst, const void* src, size_t bytes, cudaStream_t stream) const override;
    void synchronize_stream(cudaStream_t stream) const override;

    // Releases every cached block back to the driver (tests; end of process).
    void trim();

private:
    CudaAllocator() = default;
    static size_t bucket_for(size_t bytes);
    void recycle(int device_index, size_t bucket, void* ptr);

    mutable std::mutex mutex_;
    std::map<std::pair<int, size_t>, std::vector<void*>> free_lists_;
};

// Bump allocator over one device range reserved up front: nothing it hands out is ever freed individually, reset()
// rewinds it.  A CUDA graph is captured with one of these in place of the caching allocator, so that no cudaMalloc runs
// under capture and a warm-up pass and the capture pass receive identical addresses (the role of ScratchAllocator in
// src/engine/model_runner.cpp:57-100 of the reference).  Copies and memsets are forwarded to `delegate`.
class ArenaAllocator final : public DeviceAllocator {
public:
    ArenaAllocator(size_t capacity, Device device, DeviceAllocator& delegate);

    Memory::Ptr allocate(size_t bytes, Device device) override;   // 256-byte aligned; throws std::runtime_error when full
    void memset_async(void* ptr, int value, size_t bytes, cudaStream_t stream) const override;
    void copy_to_device_async(void* dst, const void* src, size_t bytes, cudaStream_t stream) const override;
    void copy_to_host_async(void* dst, const void* src, size_t bytes, cudaStream_t stream) const override;
    void synchronize_stream(cudaStream_t stream) const override;

    void reset() { offset_ = 0; }
    size_t used() const { return offset_; }
    size_t high_water() const { return high_water_; }

private:
    Memory::Ptr arena_;
    Device device_;
    DeviceAllocator& delegate_;
    size_t offset_ = 0, high_water_ = 0;
};

// Page-locked host staging buffer (metadata upload, src/engine/model_runner.cpp:805-831).
class PinnedHostBuffer {
public:
    explicit PinnedHostBuffer(size_t bytes);
    ~PinnedHostBuffer();
    PinnedHostBuffer(const PinnedHostBuffer&) = delete;
    PinnedHostBuffer& operator=(const PinnedHostBuffer&) = delete;
    PinnedHostBuffer(PinnedHostBuffer&& other) noexcept;
    PinnedHostBuffer& operator=(PinnedHostBuffer&& other) noexcept;

    void* data() const { return data_; }
    size_t bytes() const { return bytes_; }

private:
    void* data_ = nullptr;
    size_t bytes_ = 0;
};

}  // namespace nano_vllm
