// Launch interface of the survivor stage (merge_rows.cu).
#pragma once

#include "peer_exchange.cuh"
#include "psx_device.cuh"

struct psx_row_diag;  // include/psx_b200.h

namespace psx {

struct MergeParams {
    // what the row pass (or an all-gather of several GPUs' row passes) left behind
    // Addressed with byte strides, so that the same kernel reads the row pass's own arrays
    // (part-major within a row) and records gathered from several GPUs (GPU-major).
    const void* stats;           // PartStats of (row, part) at stats + row*stats_row_stride + part*stats_part_stride
    const void* part_counts;     // uint32 of (row, part) likewise: candidates in the part's list
    const void* candidates;      // uint2[part_cap] of (row, part) likewise
    int64_t stats_row_stride, stats_part_stride;
    int64_t count_row_stride, count_part_stride;
    int64_t cand_row_stride, cand_part_stride;
    int32_t parts;
    int32_t part_cap;            // slots of a part's list
    int32_t slot_shift;          // 2^slot_shift slots of every list are fetched before the counts are known;
                                 // parts << slot_shift <= 16 * kMergeThreads
    int64_t rows;                // rows this launch decides: row_begin .. row_begin + rows - 1
    int64_t row_begin;           // (every array below and above is indexed by the absolute row)
    int64_t vocab;               // global vocabulary size
    // settings (GenerationConfig, already validated)
    int32_t do_sample;
    int32_t apply_temperature;
    float temperature;
    float penalty;
    int64_t top_k;               // 0 < top_k < vocab: the top-k filter is on
    float top_p;
    float min_p;
    const double* uniforms;      // device, rows (unused when greedy)
    // output
    int64_t* tokens;
    float* log_probs;
    int32_t* row_status;
    psx_row_diag* diag;          // may be null
    int32_t sort_capacity;       // survivors + near-survivors the shared-memory sorter holds (power of two)
    // Optional: the surviving set itself (for ProcessLogits), up to survivor_cap per row; null = off.
    uint32_t* survivor_cols;     // rows * survivor_cap global columns, in no particular order
    float* survivor_vals;        // their processed logits
    uint32_t* survivor_counts;   // rows
    int32_t survivor_cap;
    int32_t gather_capacity;     // candidates of one row held in shared memory (<= 4 * sort_capacity)
    // Optional: the logits themselves (row r, global column c at logits[r*logits_row_stride + c -
    // logits_col_begin]).  With them the chosen token's raw logit is read back from there, and, when
    // `overlay` is set, the gathered candidates share their shared memory with the sort arrays that
    // are only needed once the list is built (smaller footprint, more rows per SM).  Only for
    // settings without a top-k.
    const float* logits;
    int64_t logits_row_stride;
    int64_t logits_col_begin;
    int32_t overlay;
    // Optional: what it takes to decide a row from the row itself (general_row), for the rows the
    // candidate lists cannot decide -- more survivors, or more ties at a cut, than they hold.
    // Needs `logits` (with logits_col_begin == 0: the whole vocabulary on this GPU).
    const int64_t* history_ids;      // as the row pass got them; null: no repetition penalty
    const int64_t* history_offsets;
    const int64_t* banned_ids;
    int32_t num_banned;
    int32_t general;                 // 0: off; 1: for rows the lists declined; 2: for every row (the lists are not looked at)
    float* process_out;              // ProcessLogits: general_row rewrites the row in place instead of drawing
    int32_t dyn_bytes;               // dynamic shared memory of the launch (filled in by launch_merge_rows)
    // Optional: one warp per row first (merge_rows_warp_impl.cuh), the block-per-row kernel afterwards only for
    // the rows the warps left undecided.  For greedy and for a top-k of at most 64, straight after a row pass.
    int32_t by_warp;                 // 0: off
    int32_t warp_slot_shift;         // 2^shift slots of every list per fetch; parts << shift <= 512
    int32_t warp_list_cap;           // entries a warp's list holds: 64 or 128
    int32_t only_undecided;          // (set by launch_merge_rows for the second kernel)
    // Optional (vocabulary shards that arrive over peer memory, peer_exchange.cuh): the row's lists are
    // complete once arrivals[row] has reached arrivals_target; the row's CTA waits for that, at most
    // arrivals_wait_ns nanoseconds (then the row reports PSX_ROW_DEVICE_TIMEOUT).  One block per row only.
    const uint32_t* arrivals;        // nullptr: nothing to wait for
    uint32_t arrivals_target;
    unsigned long long arrivals_wait_ns;
    // ... and the row's result goes straight into every rank's results section, with one more on this
    // rank's counter in each of their flags sections (the outputs above are still written: here they are
    // this rank's own block, indexed by the absolute row).
    int32_t publish;                 // 0: off
    PeerLayout peers;
};

constexpr int64_t kRowsByWarpFrom = 256;  // launches of fewer rows stay with one block per row
// Plans a launch by warps for lists that usually hold about `expected` candidates; false: not for this plan.
bool plan_merge_by_warp(MergeParams& p, int k_need, bool greedy, int expected);

// Row status between the survivor stage and ProcessLogits' write-back: general_row has already
// rewritten the row in place.  Never leaves the library.
constexpr int kRowDoneInPlace = 64;
// Row status between the two kernels of a launch by warps: the block-per-row kernel has yet to decide the row.
constexpr int kRowUndecided = 65;

size_t merge_rows_shared_bytes(int sort_capacity, int gather_capacity, bool overlay);
// The slot_shift for lists that usually hold about `expected` candidates, within the fetch budget.
int merge_slot_shift(int parts, int part_cap, int expected);
cudaError_t configure_merge_rows();  // once per device: lifts the kernel's dynamic shared-memory limit to the device's
// launched (optional): how many kernels the call launched, added to what is there.
cudaError_t launch_merge_rows(const MergeParams& p, cudaStream_t stream, uint64_t* launched = nullptr);

}  // namespace psx
