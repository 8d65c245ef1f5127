// ProcessLogits on the device (src/generation.cpp:55-112): the processed row itself, in place.
//
// Without filters (greedy, or sampling with top_k, top_p and min_p all off) it is elementwise:
// repetition penalty for the columns the history names, -inf for banned EOS ids, the temperature
// divide.  With filters, the row pass and the survivor stage have already decided which columns
// survive (and with what processed value); this kernel then blanks the row to -inf and a second
// tiny kernel writes the survivors back.
#include "process_rows.cuh"

namespace psx {

namespace {

constexpr int kThreads = 256;
constexpr int kChunk = 16384;            // columns per CTA
constexpr int kWords = kChunk / 32;

__device__ __forceinline__ void mark(const int64_t* ids, int64_t begin, int64_t end, int64_t vocab, int64_t chunk_begin,
                                     int chunk_len, uint32_t* bitmap) {
    for (int64_t i = begin + threadIdx.x; i < end; i += kThreads) {
        const int64_t id = ids[i];
        if (id < 0 || id >= vocab) continue;  // src/generation.cpp:62
        const int64_t e = id - chunk_begin;
        if (e >= 0 && e < chunk_len) atomicOr(&bitmap[e >> 5], 1u << (e & 31));
    }
}

__global__ void __launch_bounds__(kThreads) process_rows_kernel(const ProcessParams p) {
    __shared__ uint32_t s_pen[kWords], s_ban[kWords];
    const int64_t row = (int64_t)blockIdx.z * 65535 + blockIdx.y;
    if (row >= p.rows) return;
    const int64_t chunk_begin = (int64_t)blockIdx.x * kChunk;
    const int chunk_len = (int)min((int64_t)kChunk, p.vocab - chunk_begin);
    float* out = p.logits + row * p.row_stride + chunk_begin;
    if (p.filters_on) {
        // The survivors come back in the next kernel; a row the device path declined stays as it was.
        const int status = p.row_status[row];
        if (status != PSX_ROW_OK && status != PSX_ROW_ALL_REMOVED) return;
        for (int i = threadIdx.x; i < chunk_len; i += kThreads) out[i] = -INFINITY;
        return;
    }
    for (int w = threadIdx.x; w < kWords; w += kThreads) { s_pen[w] = 0; s_ban[w] = 0; }
    __syncthreads();
    if (p.apply_penalty) {
        mark(p.history_ids, p.history_offsets[row], p.history_offsets[row + 1], p.vocab, chunk_begin, chunk_len, s_pen);
    }
    if (p.num_banned > 0) mark(p.banned_ids, 0, p.num_banned, p.vocab, chunk_begin, chunk_len, s_ban);
    __syncthreads();
    for (int i = threadIdx.x; i < chunk_len; i += kThreads) {
        const uint32_t bit = 1u << (i & 31);
        float l = out[i];
        if (s_ban[i >> 5] & bit) l = -INFINITY;                              // src/generation.cpp:69-73
        else if (s_pen[i >> 5] & bit) l = penalize(l, p.penalty);            // :59-68
        out[i] = temper(l, p.apply_temperature != 0, p.temperature);         // :77-79
    }
}

__global__ void __launch_bounds__(kThreads) scatter_survivors_kernel(const ProcessParams p) {
    const int64_t row = blockIdx.x;
    const int status = p.row_status[row];
    if (status == kRowDoneInPlace) {  // the survivor stage has rewritten this row itself
        if (threadIdx.x == 0) p.row_status[row] = PSX_ROW_OK;
        return;
    }
    if (status != PSX_ROW_OK) return;
    const int count = (int)p.survivor_counts[row];
    float* out = p.logits + row * p.row_stride;
    for (int i = threadIdx.x; i < count; i += kThreads) {
        out[p.survivor_cols[row * p.survivor_cap + i]] = p.survivor_vals[row * p.survivor_cap + i];
    }
}

}  // namespace

cudaError_t launch_process_rows(const ProcessParams& p, cudaStream_t stream) {
    if (p.rows <= 0) return cudaSuccess;
    if (p.rows > 65535ll * 65535ll) return cudaErrorInvalidConfiguration;
    const dim3 grid((unsigned)((p.vocab + kChunk - 1) / kChunk), (unsigned)(p.rows < 65535 ? p.rows : 65535),
                    (unsigned)((p.rows + 65534) / 65535));
    process_rows_kernel<<<grid, kThreads, 0, stream>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || !p.filters_on) return e;
    scatter_survivors_kernel<<<(unsigned)p.rows, kThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace psx
