// Launch interface of top_k_rows (topk_rows.cu).
#pragma once

#include "psx_device.cuh"

namespace psx {

constexpr int kTopKMax = 4096;  // largest k the shared-memory sorter of one CTA holds (a power of two)

// k <= kTopKMax: selection, then a sort of the k winners in shared memory.
cudaError_t launch_topk_rows(const float* in, float* values, float* indices, size_t rows, size_t cols, size_t k,
                             bool largest, cudaStream_t stream);
// Any k: the whole row is sorted in `scratch` (sort_rows_scratch_bytes bytes; the rows go through it
// in launches of *rows_per_launch rows).
size_t sort_rows_scratch_bytes(size_t rows, size_t cols, size_t* rows_per_launch);
cudaError_t launch_sort_rows(const float* in, float* values, float* indices, size_t rows, size_t cols, size_t k, bool largest,
                             void* scratch, cudaStream_t stream);

}  // namespace psx
