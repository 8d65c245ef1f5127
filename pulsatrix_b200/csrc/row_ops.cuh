// Launch interface of the row primitives (row_ops.cu).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace psx {

// out[r][j] = exp(in[r][j] - max_r) / sum_j exp(in[r][j] - max_r); out may alias in.
cudaError_t launch_softmax_rows(const float* in, float* out, size_t rows, size_t cols, cudaStream_t stream);
// out[r] = max_r + log(sum_j exp(in[r][j] - max_r)).
cudaError_t launch_logsumexp_rows(const float* in, float* out, size_t rows, size_t cols, cudaStream_t stream);
// out[i][:] = table[indices[i]][:]; indices are whole-number floats.
cudaError_t launch_gather_rows(const float* table, const float* indices, float* out, size_t count, size_t dim,
                               cudaStream_t stream);

}  // namespace psx
