// CUDA status -> exception helpers (the reference's error convention, src/utils/cuda_common.cpp:39-43:
// std::runtime_error("<context>: <cuda error string>")).
#pragma once

#include <cuda_runtime_api.h>

#include <string>

namespace nano_vllm {

std::string cuda_error_string(cudaError_t status);
void throw_if_cuda_error(cudaError_t status, const char* context);

}  // namespace nano_vllm
