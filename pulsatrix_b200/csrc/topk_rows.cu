// top_k_rows: the k best entries of every row in rank order, with their columns as floats.
//
// One CTA per row, any row length up to 2^24 and any alignment:
//   1. a 4 x 8-bit radix select over order-preserving keys (NaN above every number, -0.0 == +0.0,
//      `largest == 0` mirrors the order) finds the k-th key and how many entries tie with it;
//   2. one more sweep gathers every entry strictly above the k-th key into shared memory and
//      appends the lowest-column ties in column order (an ordered block-wide compaction);
//   3. a bitonic sort of (key, ~column) puts the gathered entries in rank order, equal values by
//      ascending column, and the values are copied from the input so that their bits (the sign
//      of zero, NaN payloads) are the input's.
// Pure selection: nothing is computed, so the result equals the host reference bit for bit
// (src/top_k_math.hpp:19-47).  The row is read five times, after the first time from L2.
#include "topk_rows.cuh"

namespace psx {

namespace {

using u64 = unsigned long long;
constexpr int kThreads = 256;

__device__ __forceinline__ uint32_t rank_key(float x, bool largest) {
    const uint32_t k = (x != x) ? 0xFFFFFFFFu : ordered_key(x);
    return largest ? k : ~k;
}

__global__ void __launch_bounds__(kThreads) topk_rows_kernel(const float* __restrict__ in, float* __restrict__ values,
                                                             float* __restrict__ indices, size_t cols, size_t k,
                                                             int largest_flag) {
    __shared__ uint32_t hist[256];
    __shared__ u64 above[kTopKMax];
    __shared__ uint32_t s_prefix, s_remaining, s_above, s_tie_base;
    __shared__ uint32_t s_warp_ties[kThreads / 32];

    const bool largest = largest_flag != 0;
    const float* row = in + (size_t)blockIdx.x * cols;
    float* out_v = values + (size_t)blockIdx.x * k;
    float* out_i = indices + (size_t)blockIdx.x * k;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t n = (uint32_t)cols;

    // ---- 1. radix select of the k-th key -----------------------------------------------------------
    if (tid == 0) {
        s_prefix = 0;
        s_remaining = (uint32_t)k;
    }
    uint32_t mask = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        for (uint32_t i = tid; i < n; i += kThreads) {
            const uint32_t key = rank_key(row[i], largest);
            if ((key & mask) == prefix) {
                const uint32_t digit = (key >> shift) & 255u;
                // One atomic per distinct digit in the warp, not per lane: rows are often full of ties.
                const uint32_t peers = __match_any_sync(__activemask(), digit);
                if ((peers & ((1u << lane) - 1u)) == 0) atomicAdd(&hist[digit], (uint32_t)__popc(peers));
            }
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t remaining = s_remaining, above_count = 0;
            int digit = 255;
            for (; digit > 0; --digit) {
                if (above_count + hist[digit] >= remaining) break;
                above_count += hist[digit];
            }
            s_remaining = remaining - above_count;
            s_prefix = prefix | ((uint32_t)digit << shift);
        }
        mask |= 255u << shift;
        __syncthreads();
    }
    const uint32_t kth = s_prefix;
    const uint32_t ties_wanted = s_remaining;           // entries equal to the k-th key to keep
    const uint32_t above_total = (uint32_t)k - ties_wanted;  // entries strictly above it
    if (tid == 0) {
        s_above = 0;
        s_tie_base = 0;
    }
    __syncthreads();

    // ---- 2. gather: strictly-above entries unordered, ties in column order ----------------------------
    for (uint32_t base = 0; base < n; base += kThreads) {
        const uint32_t i = base + tid;
        uint32_t key = 0;
        bool tie = false;
        if (i < n) {
            key = rank_key(row[i], largest);
            if (key > kth) {
                const uint32_t slot = atomicAdd(&s_above, 1u);
                above[slot] = ((u64)key << 32) | (uint32_t)~i;
            }
            tie = key == kth;
        }
        const uint32_t tie_base = s_tie_base;  // uniform: written before the last barrier
        if (tie_base < ties_wanted) {
            const uint32_t votes = __ballot_sync(0xFFFFFFFFu, tie);
            if (lane == 0) s_warp_ties[warp] = __popc(votes);
            __syncthreads();
            uint32_t before = tie_base, total = 0;
            for (int w = 0; w < kThreads / 32; ++w) {
                if (w < warp) before += s_warp_ties[w];
                total += s_warp_ties[w];
            }
            const uint32_t pos = before + __popc(votes & ((1u << lane) - 1u));
            if (tie && pos < ties_wanted) {
                out_v[above_total + pos] = row[i];
                out_i[above_total + pos] = (float)i;
            }
            __syncthreads();
            if (tid == 0) s_tie_base = tie_base + total;
            __syncthreads();
        }
    }
    __syncthreads();

    // ---- 3. rank order of the entries above the k-th key ------------------------------------------------
    uint32_t n_pad = 2;
    while (n_pad < above_total) n_pad <<= 1;
    for (uint32_t i = above_total + tid; i < n_pad; i += kThreads) above[i] = 0;
    __syncthreads();
    if (above_total > 1) block_bitonic_sort(above, (int)n_pad, /*descending=*/true);
    for (uint32_t j = tid; j < above_total; j += kThreads) {
        const uint32_t col = ~(uint32_t)above[j];
        out_v[j] = row[col];
        out_i[j] = (float)col;
    }
}

}  // namespace

cudaError_t launch_topk_rows(const float* in, float* values, float* indices, size_t rows, size_t cols, size_t k,
                             bool largest, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    topk_rows_kernel<<<(unsigned)rows, kThreads, 0, stream>>>(in, values, indices, cols, k, largest ? 1 : 0);
    return cudaGetLastError();
}

}  // namespace psx
