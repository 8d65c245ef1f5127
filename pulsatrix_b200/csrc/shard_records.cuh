// Vocabulary-sharded sampling: the fixed-size per-row record one GPU contributes to the all-gather
// (shard_records.cu packs it from the row pass's output).
//
// Record layout, `capacity` candidates: PartStats at byte 0, the candidate count (uint32) at
// byte 40, the candidates (uint2 each: raw logit bits, global column | flags) from byte 48.
// The survivor stage reads gathered records directly through byte strides.
#pragma once

#include "peer_exchange.cuh"
#include "psx_device.cuh"

namespace psx {

constexpr int kRecordStatsOffset = 0;
constexpr int kRecordCountOffset = 40;
constexpr int kRecordCandidatesOffset = 48;
static_assert(sizeof(PartStats) == 40, "record layout assumes a 40-byte PartStats");

// Candidates a record holds: the k the merged top-k needs from any one shard, plus room for
// ties at the shard's threshold.
inline int shard_record_capacity(bool sample, int64_t top_k) {
    if (!sample) return 64;
    const int64_t k = top_k < 1 ? 1 : (top_k > 960 ? 960 : top_k);
    return (int)((k + 64 + 63) / 64 * 64);
}
__host__ __device__ inline size_t shard_record_bytes(int capacity) { return (size_t)kRecordCandidatesOffset + 8u * (size_t)capacity; }

struct PackParams {
    const PartStats* stats;      // rows * parts, from the row pass
    const uint32_t* part_counts; // rows * parts
    const uint2* candidates;     // rows * parts * kPartCap
    int32_t parts;
    int64_t rows;
    int32_t apply_temperature;
    float temperature;
    float penalty;
    int32_t capacity;
    int32_t do_sample;
    int32_t top_k;               // > 0: the top-k filter is on (sampling); 0: greedy
    void* records;               // rows * shard_record_bytes(capacity); not used when the records go to peers
    // Optional: straight into the exchange buffers of the ranks that decide the rows (peer_exchange.cuh).
    // Row r belongs to rank r / rows_per_rank; its record goes to that rank's records section at
    // [this rank][r % rows_per_rank], and that rank's arrival counter of the row goes up by one.
    int32_t to_peers;            // 0: off
    PeerLayout peers;
    // With to_peers the kernel runs under the row pass instead of after it: a row's block waits (bounded)
    // until row_ready[row] has reached row_ready_target (all parts of the row written: ScanParams::row_ready)
    // and until *step_done has reached step_done_target (the step before has been read everywhere, so its
    // records may be overwritten: AwaitParams::step_done); a wait that runs out marks the record (bit 1 of
    // PartStats::nonfinite, as a copy that timed out does).
    const uint32_t* row_ready;
    uint32_t row_ready_target;
    const uint32_t* step_done;
    uint32_t step_done_target;
    unsigned long long wait_limit_ns;
};

cudaError_t launch_pack_records(const PackParams& p, cudaStream_t stream);

}  // namespace psx
