// top_k_rows: the k best entries of every row in rank order, with their columns as floats.
//
// A row belongs to a thread-block cluster of 1, 2, 4 or 8 CTAs (by its length); each CTA reads
// its slice of the row from HBM once, turns it into order-preserving keys (NaN above every
// number, -0.0 == +0.0, `largest == 0` mirrors the order) and keeps the keys in shared memory.
// Everything after that works on the keys:
//   1. a 4 x 8-bit radix select finds the k-th key: every CTA counts its slice's digits into a
//      histogram of its own, the cluster meets, and every CTA adds the cluster's histograms up
//      through distributed shared memory for itself;
//   2. when more entries tie with the k-th key than are wanted, a second radix select, over the
//      columns of the tying entries, finds the column up to which they are taken (the reference
//      keeps the lowest columns, src/top_k_math.hpp:19-47);
//   3. the entries above the k-th key and the chosen ties are collected in the first CTA's shared
//      memory (remote atomics and stores), sorted there by (key, ~column) -- rank order, equal
//      values by ascending column -- and written out; the values are copied from the input, so
//      that their bits (the sign of zero, NaN payloads) are the input's.
// Pure selection: nothing is computed, so the result equals the host reference bit for bit.
// HBM-bound in design: the row is read once, and k values again at the end.  Rows too long for
// the cluster's shared memory (more than 8 x 48K entries) are swept from global memory instead.
#include <cooperative_groups.h>

#include "topk_rows.cuh"

namespace cg = cooperative_groups;

namespace psx {

namespace {

using u64 = unsigned long long;
constexpr int kThreads = 256;
constexpr int kSliceMax = 48 * 1024;  // keys one CTA keeps in shared memory (192 KB)

__device__ __forceinline__ uint32_t rank_key(float x, bool largest) {
    const uint32_t k = (x != x) ? 0xFFFFFFFFu : ordered_key(x);
    return largest ? k : ~k;
}

struct TopKParams {
    const float* in;
    float* values;
    float* indices;
    size_t cols;
    size_t k;
    int largest;
    int cluster;     // CTAs per row
    uint32_t slice;  // entries per CTA (a multiple of 4)
    int in_shared;   // the slice's keys are kept in shared memory
    uint32_t k_pad;  // power of two >= k: slots of the collecting array
};

// The cluster's histograms of one pass, added up and scanned from the top by warp 0 of every CTA:
// the digit at which the count from the top reaches `remaining`, the count above that digit, and
// the count in it.  hist points at this CTA's 256 counters of the pass; the same address in every
// CTA of the cluster.
struct Found {
    uint32_t digit, above, inside;
};
__device__ __forceinline__ Found find_digit(cg::cluster_group& cluster, uint32_t* hist, int ranks, uint32_t remaining, int lane) {
    // lane L owns digits 255-8L down to 248-8L
    uint32_t bins[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < ranks; ++r) {
        const uint4* remote = reinterpret_cast<const uint4*>(cluster.map_shared_rank(hist, r));
        const uint4 lo = remote[62 - 2 * lane], hi = remote[63 - 2 * lane];
        bins[0] += hi.w; bins[1] += hi.z; bins[2] += hi.y; bins[3] += hi.x;
        bins[4] += lo.w; bins[5] += lo.z; bins[6] += lo.y; bins[7] += lo.x;
    }
    uint32_t local = 0;
#pragma unroll
    for (int q = 0; q < 8; ++q) local += bins[q];
    uint32_t incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
        if (lane >= o) incl += up;
    }
    const uint32_t excl = incl - local;
    const bool here = excl < remaining && remaining <= incl;
    uint32_t above = excl, inside = bins[0];
    int q_found = 0;
    if (here) {
#pragma unroll
        for (int q = 0; q < 7; ++q) {
            if (q_found == q && above + bins[q] < remaining) {
                above += bins[q];
                q_found = q + 1;
                inside = bins[q + 1];
            }
        }
    }
    const int src = max(0, __ffs(__ballot_sync(0xFFFFFFFFu, here)) - 1);  // exactly one lane while remaining <= total
    Found f;
    f.digit = __shfl_sync(0xFFFFFFFFu, (uint32_t)(255 - 8 * lane - q_found), src);
    f.above = __shfl_sync(0xFFFFFFFFu, above, src);
    f.inside = __shfl_sync(0xFFFFFFFFu, inside, src);
    return f;
}

__global__ void __launch_bounds__(kThreads) topk_rows_kernel(const TopKParams p) {
    extern __shared__ __align__(16) unsigned char dyn[];
    // layout: [k_pad collected entries, 8 bytes each][slice keys, 4 bytes each (when in_shared)]
    u64* collected = reinterpret_cast<u64*>(dyn);
    uint32_t* keys = reinterpret_cast<uint32_t*>(dyn + (size_t)p.k_pad * 8);
    __shared__ __align__(16) uint32_t s_hist[7][256];  // four passes over the key, three over the column
    __shared__ uint32_t s_prefix, s_remaining, s_inside, s_collected;

    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank(), ranks = p.cluster;
    const size_t row_index = blockIdx.x / (unsigned)ranks;
    const bool largest = p.largest != 0;
    const float* row = p.in + row_index * p.cols;
    const int tid = threadIdx.x, lane = tid & 31;
    const uint32_t n = (uint32_t)p.cols;
    const uint32_t begin = min(n, (uint32_t)rank * p.slice), end = min(n, begin + p.slice);
    const uint32_t mine = end - begin;
    const bool in_shared = p.in_shared != 0;

    for (int i = tid; i < 7 * 256; i += kThreads) (&s_hist[0][0])[i] = 0;
    if (tid == 0) s_collected = 0;
    // ---- the slice, once from HBM, as keys -----------------------------------------------------------
    if (in_shared) {
        const float* src = row + begin;
        const uint32_t head = min(mine, (uint32_t)((4 - ((reinterpret_cast<uintptr_t>(src) >> 2) & 3)) & 3));
        for (uint32_t i = tid; i < head; i += kThreads) keys[i] = rank_key(src[i], largest);
        const uint32_t vectors = (mine - head) / 4;
        const float4* src4 = reinterpret_cast<const float4*>(src + head);
        for (uint32_t v = tid; v < vectors; v += kThreads) {
            const float4 d = src4[v];
            uint32_t* to = keys + head + 4 * v;
            to[0] = rank_key(d.x, largest); to[1] = rank_key(d.y, largest);
            to[2] = rank_key(d.z, largest); to[3] = rank_key(d.w, largest);
        }
        for (uint32_t i = head + 4 * vectors + tid; i < mine; i += kThreads) keys[i] = rank_key(src[i], largest);
    }
    __syncthreads();
    auto key_at = [&](uint32_t i) { return in_shared ? keys[i] : rank_key(row[begin + i], largest); };

    // ---- 1. radix select of the k-th key ---------------------------------------------------------------
    uint32_t prefix = 0, mask = 0, remaining = (uint32_t)p.k, inside = 0;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        uint32_t* hist = s_hist[pass];
        for (uint32_t i = tid; i < mine; i += kThreads) {
            const uint32_t key = key_at(i);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        cluster.sync();
        if (tid < 32) {
            const Found f = find_digit(cluster, hist, ranks, remaining, lane);
            if (lane == 0) {
                s_prefix = prefix | (f.digit << shift);
                s_remaining = remaining - f.above;
                s_inside = f.inside;
            }
        }
        __syncthreads();
        prefix = s_prefix;
        remaining = s_remaining;
        inside = s_inside;
        mask |= 255u << shift;
    }
    const uint32_t kth = prefix;
    const uint32_t ties_wanted = remaining;  // entries equal to the k-th key to take; `inside` entries equal it

    // ---- 2. more ties than wanted: the column up to which they are taken ------------------------------------
    uint32_t last_tie_column = 0xFFFFFFFFu;
    if (inside > ties_wanted) {  // uniform over the cluster
        uint32_t cprefix = 0, cmask = 0, cremaining = ties_wanted;
        for (int pass = 0; pass < 3; ++pass) {
            const int shift = 16 - 8 * pass;
            uint32_t* hist = s_hist[4 + pass];
            for (uint32_t i = tid; i < mine; i += kThreads) {
                if (key_at(i) != kth) continue;
                const uint32_t inverted = ~(begin + i) & 0x00FFFFFFu;  // lower columns rank higher; columns are below 2^24
                if ((inverted & cmask) == cprefix) atomicAdd(&hist[(inverted >> shift) & 255u], 1u);
            }
            cluster.sync();
            if (tid < 32) {
                const Found f = find_digit(cluster, hist, ranks, cremaining, lane);
                if (lane == 0) {
                    s_prefix = cprefix | (f.digit << shift);
                    s_remaining = cremaining - f.above;
                }
            }
            __syncthreads();
            cprefix = s_prefix;
            cremaining = s_remaining;
            cmask |= 255u << shift;
        }
        last_tie_column = ~cprefix & 0x00FFFFFFu;
    }

    // ---- 3. collect in the first CTA, sort there, write -------------------------------------------------------
    {
        uint32_t* count0 = cluster.map_shared_rank(&s_collected, 0);
        u64* collected0 = cluster.map_shared_rank(collected, 0);
        for (uint32_t i = tid; i < mine; i += kThreads) {
            const uint32_t key = key_at(i), col = begin + i;
            if (key > kth || (key == kth && col <= last_tie_column)) {
                const uint32_t slot = atomicAdd(count0, 1u);
                if (slot < p.k_pad) collected0[slot] = ((u64)key << 32) | (uint32_t)~col;
            }
        }
    }
    cluster.sync();  // nobody touches another CTA's shared memory after this
    if (rank != 0) return;
    const uint32_t taken = min(s_collected, (uint32_t)p.k);  // == k
    for (uint32_t i = taken + tid; i < p.k_pad; i += kThreads) collected[i] = 0;
    __syncthreads();
    if (p.k_pad > 1) block_bitonic_sort(collected, (int)p.k_pad, /*descending=*/true);
    float* out_v = p.values + row_index * p.k;
    float* out_i = p.indices + row_index * p.k;
    for (uint32_t j = tid; j < taken; j += kThreads) {
        const uint32_t col = ~(uint32_t)collected[j];
        out_v[j] = row[col];
        out_i[j] = (float)col;
    }
}

}  // namespace

cudaError_t launch_topk_rows(const float* in, float* values, float* indices, size_t rows, size_t cols, size_t k,
                             bool largest, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    TopKParams p;
    p.in = in;
    p.values = values;
    p.indices = indices;
    p.cols = cols;
    p.k = k;
    p.largest = largest ? 1 : 0;
    p.cluster = cols <= 16384 ? 1 : cols <= 32768 ? 2 : cols <= 65536 ? 4 : 8;
    p.slice = (uint32_t)(((cols + p.cluster - 1) / p.cluster + 3) / 4 * 4);
    p.k_pad = 1;
    while (p.k_pad < k) p.k_pad <<= 1;
    // keys in shared memory when they fit beside the collecting array and the histograms
    p.in_shared = p.slice <= (uint32_t)kSliceMax && (size_t)p.k_pad * 8 + (size_t)p.slice * 4 + 8192 <= 227 * 1024 ? 1 : 0;
    const size_t shared = (size_t)p.k_pad * 8 + (p.in_shared ? (size_t)p.slice * 4 : 0);
    if (rows * (size_t)p.cluster > 0x7FFFFFFFull) return cudaErrorInvalidConfiguration;
    if (shared > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(topk_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)(rows * p.cluster));
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = (unsigned)p.cluster;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, topk_rows_kernel, p);
}

}  // namespace psx
