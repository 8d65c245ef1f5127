// Launch interface of the in-place ProcessLogits kernels (process_rows.cu).
#pragma once

#include "../../include/psx_b200.h"
#include "merge_rows.cuh"
#include "psx_device.cuh"

namespace psx {

struct ProcessParams {
    float* logits;                   // rows x vocab, in place; row r at logits + r*row_stride
    int64_t row_stride, rows, vocab;
    const int64_t* history_ids;      // device
    const int64_t* history_offsets;  // device, rows + 1
    const int64_t* banned_ids;       // device
    int32_t num_banned;
    int32_t apply_penalty;
    float penalty;
    int32_t apply_temperature;
    float temperature;
    int32_t filters_on;              // 1: blank the row, then write the survivors below back
    int32_t* row_status;             // device, rows: what the survivor stage said (filters_on only)
    const uint32_t* survivor_cols;   // rows * survivor_cap
    const float* survivor_vals;
    const uint32_t* survivor_counts; // rows
    int32_t survivor_cap;
};

// One or two launches on `stream` (the second only when filters_on).
cudaError_t launch_process_rows(const ProcessParams& p, cudaStream_t stream);

}  // namespace psx
