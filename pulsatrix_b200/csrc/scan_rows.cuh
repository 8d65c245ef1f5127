// Launch interface of the row pass (scan_rows.cu).
#pragma once

#include "psx_device.cuh"

namespace psx {

struct ScanParams {
    // input
    const float* logits;             // row r, column c of this GPU's slice at logits[r*row_stride + c]
    int64_t row_stride;
    int64_t rows;
    int64_t cols;                    // columns held by this GPU
    int64_t col_begin;               // global id of local column 0 (0 unless the vocabulary is sharded)
    int64_t vocab;                   // global vocabulary size (range check of history ids)
    const int64_t* history_ids;      // device
    const int64_t* history_offsets;  // device, rows + 1
    const int64_t* banned_ids;       // device: EOS ids while min_new_tokens holds them off
    int32_t num_banned;
    int32_t apply_penalty;
    float penalty;
    int32_t apply_temperature;
    float temperature;
    float log2e_over_t;              // log2(e) / temperature (log2(e) when the temperature is off)
    int32_t k_need;                  // every part hands on at least this many logits (or all it has)
    int32_t parts;                   // CTAs per row
    int32_t vecs_per_part;           // float4 vectors per part, <= kPartVecs
    int32_t inputs_ready;            // the inputs above are complete whatever the kernel before this one is doing
    uint64_t wait_limit_ns;          // a wait for a copy gives up after this long (the part then reports a time-out)
    int32_t test_short_copy;         // tests only: the copies deliver less than was announced, so that a wait runs out
    // The kernel before this one in the stream (launched so that the two may overlap) may still be reading the
    // scratch below.  1: every CTA waits for it to finish before its first write.  0: the caller alternates
    // between two sets of scratch and launches row pass and survivor stage in turn; then the set written here
    // was last read two kernels back, and it is enough that this kernel does not finish before the kernel
    // before it has (only the last CTA waits, just before it ends): the survivor stage that waits for this
    // kernel thereby starts after the survivor stage before it has finished, and so on down the stream.
    int32_t wait_before_writes;
    // output
    PartStats* stats;                // rows * parts
    uint32_t* part_counts;           // rows * parts: candidates handed on by the part
    uint2* candidates;               // rows * parts * kPartCap: the part's candidates, back to back
    // Optional: one counter per row, raised by one (a release at device scope) when a part of the row has
    // written everything above -- a kernel that runs under this one can then take the rows as they finish.
    uint32_t* row_ready;             // nullptr: off
};

constexpr uint64_t kDefaultWaitLimitNs = 1000000000ull;

// nucleus: also accumulate the processed-domain tail that a full-vocabulary top-p / min-p needs.
// configure: once per device, before the first launch (lifts the kernels' dynamic shared-memory limit).
cudaError_t configure_scan_rows();
cudaError_t launch_scan_rows(const ScanParams& p, bool nucleus, cudaStream_t stream);

}  // namespace psx
