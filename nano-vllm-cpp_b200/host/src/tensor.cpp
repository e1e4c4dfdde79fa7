// Tensor / Memory implementation of the operator layer (interface: utils/tensor.h).
#include "utils/tensor.h"

#include "utils/cuda_allocator.h"

#include <stdexcept>
#include <utility>

namespace nano_vllm {

std::string to_string(DeviceType device_type) { return device_type == DeviceType::kCUDA ? "cuda" : "cpu"; }

std::string to_string(ScalarType scalar_type) {
    static const char* const names[] = {"float16", "bfloat16", "float32", "int32", "int64", "int8"};
    const int i = static_cast<int>(scalar_type);
    return (i >= 0 && i < 6) ? names[i] : "unknown";
}

size_t scalar_type_size(ScalarType scalar_type) {
    static const size_t widths[] = {2, 2, 4, 4, 8, 1};
    const int i = static_cast<int>(scalar_type);
    if (i < 0 || i >= 6) throw std::invalid_argument("unknown scalar type");
    return widths[i];
}

std::vector<int64_t> make_contiguous_strides(const std::vector<int64_t>& sizes) {
    std::vector<int64_t> strides(sizes.size(), 1);
    int64_t running = 1;
    for (size_t i = sizes.size(); i-- > 0;) {
        strides[i] = running;
        running *= sizes[i] > 0 ? sizes[i] : 1;
    }
    return strides;
}

size_t compute_numel(const std::vector<int64_t>& sizes) {
    size_t n = 1;
    for (const int64_t s : sizes) {
        if (s < 0) throw std::invalid_argument("tensor sizes must be non-negative");
        n *= static_cast<size_t>(s);
    }
    return n;
}

// ---- Memory --------------------------------------------------------------------------------------
Memory::Memory(void* data, size_t bytes, Device device, std::function<void(void*)> deleter)
    : data_(data), bytes_(bytes), device_(device), deleter_(std::move(deleter)) {}

Memory::~Memory() {
    if (deleter_ && data_ != nullptr) deleter_(data_);
}

Memory::Ptr Memory::make_owned(void* data, size_t bytes, Device device, std::function<void(void*)> deleter) {
    return Ptr(new Memory(data, bytes, device, std::move(deleter)));
}

Memory::Ptr Memory::make_borrowed(void* data, size_t bytes, Device device) {
    return Ptr(new Memory(data, bytes, device, nullptr));
}

// ---- Tensor ---------------------------------------------------------------------------------------
Tensor::Tensor(Memory::Ptr memory, std::vector<int64_t> sizes, std::vector<int64_t> strides, ScalarType dtype,
               size_t memory_offset)
    : memory_(std::move(memory)), sizes_(std::move(sizes)), strides_(std::move(strides)), dtype_(dtype),
      memory_offset_(memory_offset) {}

Tensor Tensor::empty(const std::vector<int64_t>& sizes, ScalarType dtype, Device device, DeviceAllocator& allocator) {
    const size_t bytes = compute_numel(sizes) * scalar_type_size(dtype);
    Memory::Ptr memory = allocator.allocate(bytes, device);
    return Tensor(std::move(memory), sizes, make_contiguous_strides(sizes), dtype, 0);
}

Tensor Tensor::zeros(const std::vector<int64_t>& sizes, ScalarType dtype, Device device, DeviceAllocator& allocator,
                     cudaStream_t stream) {
    Tensor t = empty(sizes, dtype, device, allocator);
    if (t.nbytes() > 0) allocator.memset_async(t.data(), 0, t.nbytes(), stream);
    return t;
}

Tensor Tensor::from_memory(const Memory::Ptr& memory, const std::vector<int64_t>& sizes, ScalarType dtype,
                           size_t memory_offset) {
    if (!memory) throw std::invalid_argument("from_memory requires a memory object");
    const size_t need = (memory_offset + compute_numel(sizes)) * scalar_type_size(dtype);
    if (need > memory->bytes()) throw std::invalid_argument("tensor view exceeds its memory");
    return Tensor(memory, sizes, make_contiguous_strides(sizes), dtype, memory_offset);
}

size_t Tensor::numel() const { return defined() ? compute_numel(sizes_) : 0; }
size_t Tensor::element_size() const { return scalar_type_size(dtype_); }
size_t Tensor::nbytes() const { return numel() * element_size(); }

bool Tensor::is_contiguous() const {
    int64_t expect = 1;
    for (size_t i = sizes_.size(); i-- > 0;) {
        if (sizes_[i] == 1) continue;   // the stride of a unit dimension is irrelevant
        if (strides_[i] != expect) return false;
        expect *= sizes_[i];
    }
    return true;
}

Device Tensor::device() const { return memory_ ? memory_->device() : Device{}; }

void* Tensor::data() const {
    if (!memory_) return nullptr;
    return static_cast<unsigned char*>(memory_->data()) + memory_offset_ * element_size();
}

Tensor Tensor::reshape(const std::vector<int64_t>& sizes) const {
    if (!defined()) throw std::invalid_argument("cannot reshape an undefined tensor");
    if (!is_contiguous()) throw std::invalid_argument("reshape requires a contiguous tensor");
    if (compute_numel(sizes) != numel()) throw std::invalid_argument("reshape must preserve the element count");
    return Tensor(memory_, sizes, make_contiguous_strides(sizes), dtype_, memory_offset_);
}

Tensor Tensor::slice(int64_t dim, int64_t start, int64_t end) const {
    if (!defined()) throw std::invalid_argument("cannot slice an undefined tensor");
    if (dim < 0 || dim >= this->dim()) throw std::invalid_argument("slice dimension out of range");
    if (start < 0 || end < start || end > sizes_[static_cast<size_t>(dim)])
        throw std::invalid_argument("slice bounds out of range");
    std::vector<int64_t> sizes = sizes_;
    sizes[static_cast<size_t>(dim)] = end - start;
    const size_t offset = memory_offset_ + static_cast<size_t>(start * strides_[static_cast<size_t>(dim)]);
    return Tensor(memory_, std::move(sizes), strides_, dtype_, offset);
}

}  // namespace nano_vllm
