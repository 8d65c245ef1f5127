// Vocabulary-sharded sampling without a library collective: the GPUs of one box write to one
// another's memory over NVLink (plain peer stores into buffers opened through CUDA IPC) and tell one
// another so with counters, also in peer memory.
//
// Every rank owns one exchange buffer; a half of it (one for odd steps, one for even ones: c_abi.cu's
// psx_exchange says why) has this layout:
//   records    world x rows_per_rank records: [shard][row of this rank's block], what the ranks' packing
//              kernels write here, each its own shard's slice;
//   arrivals   rows_per_rank counters: +1 by every shard whose record of that row is complete;
//              after the half's t-th step a counter stands at t * world;
//   results    world blocks of 16 * rows_per_rank bytes (tokens | log-probs | status), block r written
//              row by row by rank r's survivor stage;
//   flags      world counters: flags[r] goes up by one for every row of rank r whose result has been written
//              here; after the half's t-th step it stands at t * (rows that rank r decides).
// Counters only ever grow, so nothing is reset between steps.  A half is written again two steps later,
// and only after the packing kernel of that step has seen, in a word of this GPU's own, that the step
// which used the half last is done everywhere: every row's result of it has arrived here, and a row's
// result is sent only after its records have been read.
//
// Every wait is bounded: after `wait_limit_ns` a waiting kernel gives up and reports
// PSX_ROW_DEVICE_TIMEOUT for the rows concerned.
#pragma once

#include <cstdint>

#include <cuda_runtime.h>

#include "psx_async.cuh"

namespace psx {

constexpr int kMaxPeers = 8;

struct PeerLayout {
    int32_t world;
    int32_t rank;
    int64_t rows_per_rank;
    int64_t record_bytes;
    int64_t records_offset, arrivals_offset, results_offset, flags_offset;  // the same in every rank's buffer
    char* base[kMaxPeers];                                                  // base[r]: rank r's buffer, as this process sees it
};

__host__ __device__ inline int64_t peer_results_block_bytes(int64_t rows_per_rank) { return 16 * rows_per_rank; }

// Bytes of one rank's exchange buffer and the offsets of its four sections (each 256-byte aligned).
inline int64_t peer_layout_offsets(int world, int64_t rows_per_rank, int64_t record_bytes, int64_t* records, int64_t* arrivals,
                                   int64_t* results, int64_t* flags) {
    auto up = [](int64_t v) { return (v + 255) / 256 * 256; };
    int64_t at = 0;
    *records = at;
    at = up(at + (int64_t)world * rows_per_rank * record_bytes);
    *arrivals = at;
    at = up(at + 4 * rows_per_rank);
    *results = at;
    at = up(at + (int64_t)world * peer_results_block_bytes(rows_per_rank));
    *flags = at;
    at = up(at + 4 * (int64_t)world);
    return at;
}

__device__ __forceinline__ uint32_t load_acquire_system(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void store_release_system(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void add_release_system(uint32_t* p, uint32_t v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t load_acquire_device(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void store_release_device(uint32_t* p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// The same wait as below for a word that only this GPU's kernels write.
__device__ __forceinline__ bool wait_until_at_least_device(const uint32_t* word, uint32_t target, unsigned long long limit_ns) {
    unsigned long long started = 0;
    for (uint32_t tries = 1;; ++tries) {
        if ((int32_t)(load_acquire_device(word) - target) >= 0) return true;
        if ((tries & 15u) == 0) {
            const unsigned long long now = global_nanoseconds();
            if (started == 0) started = now;
            else if (now - started > limit_ns) return false;
        }
    }
}

// Waits until *word >= target (as a wrapping difference), for at most limit_ns nanoseconds.
__device__ __forceinline__ bool wait_until_at_least(const uint32_t* word, uint32_t target, unsigned long long limit_ns) {
    unsigned long long started = 0;
    for (uint32_t tries = 1;; ++tries) {
        if ((int32_t)(load_acquire_system(word) - target) >= 0) return true;
        if ((tries & 15u) == 0) {
            const unsigned long long now = global_nanoseconds();
            if (started == 0) started = now;
            else if (now - started > limit_ns) return false;
        }
    }
}

struct AwaitParams {
    PeerLayout layout;
    int64_t rows;            // of the whole step: rank r decides rows r * rows_per_rank onwards, as many as there are
    uint32_t step;           // counted over both halves (the first is 1)
    uint32_t turn;           // the step's number among those of its half: the counters of layout stand at turn * rows
    unsigned long long wait_limit_ns;
    uint32_t* step_done;     // this GPU's own word: raised to `step` once every result of the step is here
};

// The last kernel of a step: one thread per rank waits until that rank's counter in this rank's flags
// section says that all its rows of the step have been written here; the rows of a rank that never
// gets there report PSX_ROW_DEVICE_TIMEOUT.  (The rows themselves are written by the survivor stage of
// the rank that decides them, one thread per destination: MergeParams::publish.)
cudaError_t launch_await_results(const AwaitParams& p, cudaStream_t stream);

}  // namespace psx
