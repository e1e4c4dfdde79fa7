// Argument checks shared by the operator wrappers (same names and messages as the reference's
// src/kernels/kernel_types.cu:24-110, which its callers and tests rely on).
#pragma once

#include "utils/tensor.h"

#include <cstdint>

namespace nano_vllm {

void ensure_cuda_tensor(const char* name, const Tensor& tensor);
void ensure_same_device(const char* lhs_name, const Tensor& lhs, const char* rhs_name, const Tensor& rhs);
void ensure_same_shape(const char* lhs_name, const Tensor& lhs, const char* rhs_name, const Tensor& rhs);
void ensure_same_dtype(const char* lhs_name, const Tensor& lhs, const char* rhs_name, const Tensor& rhs);
void validate_supported_dtype(const char* name, ScalarType dtype);

struct MatrixShape {
    int64_t rows = 0;
    int64_t cols = 0;
};
MatrixShape flatten_by_leading_count(const char* name, const Tensor& tensor, int64_t leading_count);
int64_t cache_rows_from_tensor(const char* name, const Tensor& tensor, int64_t row_width);

// Throws std::invalid_argument / std::runtime_error for a non-zero status of the C ABI (include/nvk.h).
void throw_on_nvk_status(int status);

}  // namespace nano_vllm
