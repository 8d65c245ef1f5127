// Launch interface of top_k_rows (topk_rows.cu).
#pragma once

#include "psx_device.cuh"

namespace psx {

constexpr int kTopKMax = 4096;  // largest k the shared-memory sorter of one CTA holds (a power of two)

cudaError_t launch_topk_rows(const float* in, float* values, float* indices, size_t rows, size_t cols, size_t k,
                             bool largest, cudaStream_t stream);

}  // namespace psx
