// Launch interface of the language-model head (lm_head.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace psx {

// logits[m][j] = sum_p hidden[m][p] * w_j[p] for m < rows, j < vocab, accumulated in ascending p with
// every product and every sum rounded to float.  hidden: rows x d, contiguous.  weight: vocab x d
// (token_major: the tied embedding) or d x vocab (an untied Linear's weight).  logits: row m at
// logits + m * row_stride.
cudaError_t launch_lm_head(const float* hidden, int64_t rows, int64_t d, const float* weight, int64_t vocab, bool token_major,
                           float* logits, int64_t row_stride, cudaStream_t stream);

}  // namespace psx
