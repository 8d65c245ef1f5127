// top_k_rows: the k best entries of every row in rank order, with their columns as floats.
//
// A row belongs to a thread-block cluster of 1, 2, 4 or 8 CTAs (by its length), a slice of the
// row per CTA.  Entries are compared as order-preserving keys: NaN above every number,
// -0.0 == +0.0, `largest == 0` mirrors the order.
//
// The short way (k <= 256): two sweeps over the slice as floats, straight from global memory, the
// second one out of L2.  Sweep one notes every thread's best entry; the smallest over the warps of
// the kp-th best of those (kp = ceil(k / 8)) is a bound that k entries of the slice reach.  Sweep
// two lists what reaches the bound, usually k and a few; the list is put in rank order by
// counting, and with several CTAs per row the best k of each meet in the first CTA's shared memory
// (distributed shared memory, two cluster barriers), where they are sorted and written out.
//
// The long way (larger k, or a list that overflowed: thousands of ties): the slice becomes keys in
// shared memory (or is swept from global memory when it does not fit), and
//   1. a 4 x 8-bit radix select finds the k-th key: every CTA counts its slice's digits into a
//      histogram of its own, the cluster meets, and every CTA adds the cluster's histograms up
//      through distributed shared memory for itself;
//   2. when more entries tie with the k-th key than are wanted, a second radix select, over the
//      columns of the tying entries, finds the column up to which they are taken (the reference
//      keeps the lowest columns, src/top_k_math.hpp:19-47);
//   3. the entries above the k-th key and the chosen ties are collected in the first CTA's shared
//      memory (remote atomics and stores) and sorted there by (key, ~column) -- rank order, equal
//      values by ascending column.
// The values written are copied from the input, so that their bits (the sign of zero, NaN
// payloads) are the input's.  Pure selection: nothing is computed, so the result equals the host
// reference bit for bit.
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

// Three-input maximum / minimum in one instruction (sm_100); the .NaN forms return NaN when any
// operand is NaN, the plain forms pass NaN operands by.
__device__ __forceinline__ float max3_nan(float a, float b, float c) {
    float r;
    asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float min3(float a, float b, float c) {
    float r;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// The kp-th largest (1-based, kp <= 32) of the 32 lanes' keys: for small kp the maximum is taken
// away kp - 1 times, else a bitonic sort across the lanes.
__device__ __forceinline__ uint32_t warp_kth_largest_key(uint32_t key, int kp, int lane) {
    if (kp <= 6) {
        for (int i = 1; i < kp; ++i) {
            const uint32_t top = __reduce_max_sync(0xFFFFFFFFu, key);
            const uint32_t holders = __ballot_sync(0xFFFFFFFFu, key == top);
            if (lane == __ffs(holders) - 1) key = 0;
        }
        return __reduce_max_sync(0xFFFFFFFFu, key);
    }
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            const uint32_t other = __shfl_xor_sync(0xFFFFFFFFu, key, j);
            const bool descending_block = (lane & k) == 0, lower_lane = (lane & j) == 0;
            key = (lower_lane == descending_block) ? max(key, other) : min(key, other);
        }
    }
    return __shfl_sync(0xFFFFFFFFu, key, kp - 1);
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
    uint32_t list_cap;  // entries of a CTA's short list (0: no lists)
};

// The cluster's histograms of one pass, added up and scanned from the top by warp 0 of every CTA:
// the digit at which the count from the top reaches `remaining`, the count above that digit, and
// the count in it.  hist points at this CTA's 256 counters of the pass (the same address in every
// CTA of the cluster); the histograms of CTAs first_rank .. first_rank + ranks - 1 are added up.
struct Found {
    uint32_t digit, above, inside;
};
__device__ __forceinline__ Found find_digit(cg::cluster_group& cluster, uint32_t* hist, int first_rank, int ranks,
                                            uint32_t remaining, int lane) {
    // lane L owns digits 255-8L down to 248-8L
    uint32_t bins[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = first_rank; r < first_rank + ranks; ++r) {
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

template <bool kLargest>
__global__ void __launch_bounds__(kThreads, 4) topk_rows_kernel(const TopKParams p) {
    extern __shared__ __align__(16) unsigned char dyn[];
    // layout: [k_pad collected entries][list_cap listed entries][cluster * k_pad gathered entries], 8 bytes
    //         each, then [slice keys, 4 bytes each (when in_shared)]
    u64* collected = reinterpret_cast<u64*>(dyn);
    u64* list = collected + p.k_pad;
    u64* gathered = list + p.list_cap;
    uint32_t* keys = reinterpret_cast<uint32_t*>(gathered + (size_t)p.k_pad * (p.cluster > 1 && p.list_cap != 0 ? p.cluster : 0));
    // histograms of the long way, used in turn by its passes; a pass clears the one before it once the
    // cluster has met again (nobody reads it any more)
    __shared__ __align__(16) uint32_t s_hist[2][256];
    __shared__ uint32_t s_prefix, s_remaining, s_inside, s_collected, s_listed, s_overflow;

    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    int ranks = p.cluster;  // CTAs that take part in the steps below (1 once the lists are in the first CTA)
    const size_t row_index = blockIdx.x / (unsigned)p.cluster;
    constexpr bool largest = kLargest;
    const float* row = p.in + row_index * p.cols;
    const int tid = threadIdx.x, lane = tid & 31;
    const uint32_t n = (uint32_t)p.cols;
    const uint32_t begin = min(n, (uint32_t)rank * p.slice), end = min(n, begin + p.slice);
    const uint32_t mine = end - begin;
    const bool in_shared = p.in_shared != 0;
    // The cluster's barrier costs about a microsecond; one CTA on its own meets with the block barrier.
    auto meet = [&]() {
        if (ranks > 1) cluster.sync(); else __syncthreads();
    };

    for (int i = tid; i < 2 * 256; i += kThreads) (&s_hist[0][0])[i] = 0;
    if (tid == 0) {
        s_collected = 0;
        s_listed = 0;
        s_overflow = 0;
    }
    __syncthreads();
    float* out_v = p.values + row_index * p.k;
    float* out_i = p.indices + row_index * p.k;

    // ---- 0. the short way (k <= 256): two sweeps over the slice as floats, the second one out of L2.
    //      Sweep one notes every thread's best entry; a bound that k of those reach is a lower bound of
    //      the slice's k-th best.  Sweep two lists what reaches the bound, usually k and a few; the list
    //      is put in rank order by counting, and the best k of every CTA meet in the first CTA. ----------
    if (p.list_cap != 0) {  // uniform over the cluster
        __shared__ uint32_t s_warp_bound[kThreads / 32];
        const float* src = row + begin;
        const uint32_t head = min(mine, (uint32_t)((4 - ((reinterpret_cast<uintptr_t>(src) >> 2) & 3)) & 3));
        const uint32_t vectors = (mine - head) / 4;
        const float4* src4 = reinterpret_cast<const float4*>(src + head);
        constexpr int kBatch = 8;  // loads in flight per thread
        // sweep one: the extreme entry this thread sees.  With the largest wanted a NaN is the best
        // there is, and the maximum that returns NaN for a NaN operand finds it; with the smallest
        // wanted a NaN is the worst, and the plain minimum passes it by.
        float extreme = largest ? -INFINITY : INFINITY;
        auto note = [&](float x) { extreme = largest ? max3_nan(extreme, x, x) : fminf(extreme, x); };
        auto note4 = [&](const float4& d) {
            extreme = largest ? max3_nan(max3_nan(d.x, d.y, d.z), d.w, extreme) : min3(min3(d.x, d.y, d.z), d.w, extreme);
        };
        for (uint32_t i = tid; i < head; i += kThreads) note(src[i]);
        for (uint32_t v0 = tid; v0 < vectors; v0 += kBatch * kThreads) {
            float4 d[kBatch];
#pragma unroll
            for (int q = 0; q < kBatch; ++q) {
                const uint32_t v = v0 + q * kThreads;
                d[q] = v < vectors ? __ldg(src4 + v) : make_float4(extreme, extreme, extreme, extreme);
            }
#pragma unroll
            for (int q = 0; q < kBatch; ++q) note4(d[q]);
        }
        for (uint32_t i = head + 4 * vectors + tid; i < mine; i += kThreads) note(src[i]);
        // The thread's best key, never overstated: a thread that saw nothing offers 0, and so does one
        // whose minimum is still +inf when the smallest are wanted (it may have seen nothing but NaN).
        const bool saw_any = (uint32_t)tid < head || (uint32_t)tid < vectors || head + 4 * vectors + tid < mine;
        uint32_t thread_max = saw_any ? rank_key(extreme, largest) : 0u;
        if (!largest && extreme == INFINITY) thread_max = 0;

        uint32_t bound = 0;
        if (mine > p.k) {  // else everything is listed
            // every warp's kp-th largest thread maximum, kp = ceil(k / 8): the smallest of the eight is
            // reached by 8 * kp >= k thread maxima (mine > k and k <= 256: enough threads hold an entry)
            const int kp = ((int)p.k + kThreads / 32 - 1) / (kThreads / 32);
            const uint32_t warp_bound = warp_kth_largest_key(thread_max, kp, lane);
            if (lane == 0) s_warp_bound[tid >> 5] = warp_bound;
            __syncthreads();
            bound = s_warp_bound[0];
#pragma unroll
            for (int w = 1; w < kThreads / 32; ++w) bound = min(bound, s_warp_bound[w]);
        }
        // sweep two: key >= bound, decided on the float itself: with the largest wanted, x is NaN or
        // x >= the bound's float; with the smallest wanted, x <= the mirrored bound's float.  A bound of
        // 0 lists everything; a bound that only NaN reaches is left to the long way.
        const bool everything = bound == 0, only_nan = largest && bound == 0xFFFFFFFFu;
        const float edge = largest ? from_ordered_key(bound) : from_ordered_key(~bound);
        auto reaches = [&](float x) { return largest ? !(x < edge) : x <= edge; };
        auto put = [&](float x, uint32_t col) {
            const uint32_t slot = atomicAdd(&s_listed, 1u);
            if (slot < p.list_cap) list[slot] = ((u64)rank_key(x, largest) << 32) | (uint32_t)~col;
        };
        if (everything) {
            if (mine <= p.list_cap) {
                for (uint32_t i = tid; i < mine; i += kThreads) put(src[i], begin + i);
            } else if (tid == 0) {
                s_listed = p.list_cap + 1;  // does not fit
            }
        } else if (only_nan) {
            if (tid == 0) s_listed = p.list_cap + 1;
        } else {
            for (uint32_t i = tid; i < head; i += kThreads) {
                if (reaches(src[i])) put(src[i], begin + i);
            }
            for (uint32_t v0 = tid; v0 < vectors; v0 += kBatch * kThreads) {
                float4 d[kBatch];
#pragma unroll
                for (int q = 0; q < kBatch; ++q) {
                    const uint32_t v = v0 + q * kThreads;
                    // beyond the slice: a value that does not reach the bound
                    d[q] = v < vectors ? __ldg(src4 + v) : (largest ? make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY)
                                                                   : make_float4(INFINITY, INFINITY, INFINITY, INFINITY));
                }
#pragma unroll
                for (int q = 0; q < kBatch; ++q) {
                    // (a NaN among the four makes best4 NaN when the largest are wanted, and NaN reaches)
                    const float best4 = largest ? max3_nan(max3_nan(d[q].x, d[q].y, d[q].z), d[q].w, d[q].w)
                                                : min3(min3(d[q].x, d[q].y, d[q].z), d[q].w, d[q].w);
                    if (reaches(best4) && v0 + q * kThreads < vectors) {  // rare
                        const uint32_t col = begin + head + 4 * (v0 + q * kThreads);
                        if (reaches(d[q].x)) put(d[q].x, col);
                        if (reaches(d[q].y)) put(d[q].y, col + 1);
                        if (reaches(d[q].z)) put(d[q].z, col + 2);
                        if (reaches(d[q].w)) put(d[q].w, col + 3);
                    }
                }
            }
            for (uint32_t i = head + 4 * vectors + tid; i < mine; i += kThreads) {
                if (reaches(src[i])) put(src[i], begin + i);
            }
        }
        __syncthreads();
        const uint32_t on_list = s_listed;
        const bool fits = on_list <= p.list_cap;
        const uint32_t best = min(on_list, (uint32_t)p.k);  // entries of this CTA that can be among the row's k best
        // Where the best entries go: straight out (one CTA), or into this CTA's k_pad slots of the
        // first CTA's array.  An entry's place is the number of entries that rank before it.
        u64* gathered0 = ranks > 1 ? cluster.map_shared_rank(gathered, 0) + (size_t)rank * p.k_pad : nullptr;
        if (fits) {
            if (on_list > (uint32_t)kThreads) {  // a long list: sort it
                uint32_t n_pad = 2;
                while (n_pad < on_list) n_pad <<= 1;
                for (uint32_t i = on_list + tid; i < n_pad; i += kThreads) list[i] = 0;
                __syncthreads();
                block_bitonic_sort(list, (int)n_pad, /*descending=*/true);
            }
            for (uint32_t i = tid; i < on_list; i += kThreads) {
                const u64 entry = list[i];
                uint32_t place = i;
                if (on_list <= (uint32_t)kThreads) {
                    place = 0;
                    for (uint32_t j = 0; j < on_list; ++j) place += list[j] > entry ? 1u : 0u;
                }
                if (place < best) {
                    if (ranks == 1) {
                        const uint32_t col = ~(uint32_t)entry;
                        out_v[place] = row[col];
                        out_i[place] = (float)col;
                    } else {
                        gathered0[place] = entry;
                    }
                }
            }
            if (ranks == 1) return;
            for (uint32_t j = best + tid; j < p.k_pad; j += kThreads) gathered0[j] = 0;
        }
        if (ranks > 1) {
            if (tid == 0) s_overflow = fits ? 0u : 1u;
            cluster.sync();
            uint32_t overflow = 0;
            for (int r = 0; r < ranks; ++r) overflow |= *cluster.map_shared_rank(&s_overflow, r);
            if (overflow == 0) {  // uniform over the cluster
                cluster.sync();   // everybody has read everybody's verdict: CTAs may leave
                if (rank != 0) return;
                block_bitonic_sort(gathered, (int)(p.k_pad * (uint32_t)ranks), /*descending=*/true);
                for (uint32_t j = tid; j < (uint32_t)p.k; j += kThreads) {
                    const uint32_t col = ~(uint32_t)gathered[j];
                    out_v[j] = row[col];
                    out_i[j] = (float)col;
                }
                return;
            }
        }
        if (tid == 0) s_listed = 0;
        __syncthreads();
    }

    // ---- the slice as keys in shared memory, for the long way ----------------------------------------------
    if (in_shared) {
        const float* src = row + begin;
        const uint32_t head = min(mine, (uint32_t)((4 - ((reinterpret_cast<uintptr_t>(src) >> 2) & 3)) & 3));
        // keys[head] on a 16-byte boundary, like src[head]: the array starts up to three words in
        keys = reinterpret_cast<uint32_t*>((reinterpret_cast<uintptr_t>(keys) + 15) & ~uintptr_t(15)) + ((4 - head) & 3);
        for (uint32_t i = tid; i < head; i += kThreads) keys[i] = rank_key(src[i], largest);
        const uint32_t vectors = (mine - head) / 4;
        const float4* src4 = reinterpret_cast<const float4*>(src + head);
        uint4* keys4 = reinterpret_cast<uint4*>(keys + head);
        constexpr int kBatch = 8;  // loads in flight per thread
        for (uint32_t v0 = tid; v0 < vectors; v0 += kBatch * kThreads) {
            float4 d[kBatch];
#pragma unroll
            for (int q = 0; q < kBatch; ++q) {
                const uint32_t v = v0 + q * kThreads;
                d[q] = v < vectors ? __ldg(src4 + v) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int q = 0; q < kBatch; ++q) {
                const uint32_t v = v0 + q * kThreads;
                if (v < vectors) {
                    keys4[v] = make_uint4(rank_key(d[q].x, largest), rank_key(d[q].y, largest), rank_key(d[q].z, largest),
                                          rank_key(d[q].w, largest));
                }
            }
        }
        for (uint32_t i = head + 4 * vectors + tid; i < mine; i += kThreads) keys[i] = rank_key(src[i], largest);
    }
    __syncthreads();
    auto slice_key = [&](uint32_t i) { return in_shared ? keys[i] : rank_key(row[begin + i], largest); };

    // ---- the long way (k > 256, keys not in shared memory, or a list that overflowed: ties in the thousands):
    //      the whole cluster, over the slices ------------------------------------------------------------------
    const uint32_t count = mine;
    auto key_at = [&](uint32_t i) { return slice_key(i); };
    auto col_at = [&](uint32_t i) { return begin + i; };
    const int first_rank = 0;

    // ---- 1. radix select of the k-th key ---------------------------------------------------------------
    uint32_t prefix = 0, mask = 0, remaining = (uint32_t)p.k, inside = 0;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        uint32_t* hist = s_hist[pass & 1];
        for (uint32_t i = tid; i < count; i += kThreads) {
            const uint32_t key = key_at(i);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        meet();
        if (pass > 0) s_hist[(pass - 1) & 1][tid] = 0;  // kThreads == 256 bins
        if (tid < 32) {
            const Found f = find_digit(cluster, hist, first_rank, ranks, remaining, lane);
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
            uint32_t* hist = s_hist[pass & 1];  // the key's four passes left [0] cleared and [1] to clear
            for (uint32_t i = tid; i < count; i += kThreads) {
                if (key_at(i) != kth) continue;
                const uint32_t inverted = ~col_at(i) & 0x00FFFFFFu;  // lower columns rank higher; columns are below 2^24
                if ((inverted & cmask) == cprefix) atomicAdd(&hist[(inverted >> shift) & 255u], 1u);
            }
            meet();
            s_hist[(pass + 1) & 1][tid] = 0;
            if (tid < 32) {
                const Found f = find_digit(cluster, hist, first_rank, ranks, cremaining, lane);
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
        uint32_t* count0 = cluster.map_shared_rank(&s_collected, first_rank);
        u64* collected0 = cluster.map_shared_rank(collected, first_rank);
        for (uint32_t i = tid; i < count; i += kThreads) {
            const uint32_t key = key_at(i), col = col_at(i);
            if (key > kth || (key == kth && col <= last_tie_column)) {
                const uint32_t slot = atomicAdd(count0, 1u);
                if (slot < p.k_pad) collected0[slot] = ((u64)key << 32) | (uint32_t)~col;
            }
        }
    }
    meet();  // nobody touches another CTA's shared memory after this
    if (rank != 0) return;
    const uint32_t taken = min(s_collected, (uint32_t)p.k);  // == k
    for (uint32_t i = taken + tid; i < p.k_pad; i += kThreads) collected[i] = 0;
    __syncthreads();
    if (p.k_pad > 1) block_bitonic_sort(collected, (int)p.k_pad, /*descending=*/true);
    for (uint32_t j = tid; j < taken; j += kThreads) {
        const uint32_t col = ~(uint32_t)collected[j];
        out_v[j] = row[col];
        out_i[j] = (float)col;
    }
}

// ---- k beyond what one CTA's shared memory sorts: the whole row is sorted in global memory -----------
// One CTA of 1024 threads per row: the row becomes 64-bit keys (rank key, ~column), padded to a power
// of two with keys below every real one, in scratch memory; a bitonic network sorts them, descending --
// steps that reach across more than 4096 keys run over global memory, all the others over one tile of
// 4096 keys at a time in shared memory --, and the first k keys are the answer, in rank order: equal
// values keep the lower column first because ~column is part of the key.
constexpr int kSortThreads = 1024;
constexpr int kSortTile = 4096;

__device__ __forceinline__ void tile_steps(u64* tile, uint32_t tile_base, uint32_t k2, uint32_t j_from) {
    for (uint32_t j = j_from; j > 0; j >>= 1) {
        for (uint32_t q = threadIdx.x; q < kSortTile / 2; q += kSortThreads) {
            const uint32_t i = ((q & ~(j - 1)) << 1) | (q & (j - 1)), l = i | j;
            const bool descending = ((tile_base + i) & k2) == 0;
            const u64 a = tile[i], b = tile[l];
            if (descending ? a < b : a > b) {
                tile[i] = b;
                tile[l] = a;
            }
        }
        __syncthreads();
    }
}

template <bool kLargest>
__global__ void __launch_bounds__(kSortThreads) sort_rows_kernel(const float* __restrict__ in, float* values, float* indices,
                                                                 u64* scratch, size_t cols, size_t k, uint32_t n_pad,
                                                                 size_t first_row) {
    __shared__ u64 tile[kSortTile];
    const size_t row = first_row + blockIdx.x;
    const float* x = in + row * cols;
    u64* keys = scratch + (size_t)blockIdx.x * n_pad;
    const uint32_t tile_len = min((uint32_t)kSortTile, n_pad);
    // every tile on its own: keys from the row, all steps up to the tile's length
    for (uint32_t base = 0; base < n_pad; base += kSortTile) {
        for (uint32_t t = threadIdx.x; t < tile_len; t += kSortThreads) {
            const size_t i = (size_t)base + t;
            tile[t] = i < cols ? (((u64)rank_key(x[i], kLargest) << 32) | (uint32_t)~(uint32_t)i) : 0ull;
        }
        __syncthreads();
        for (uint32_t k2 = 2; k2 <= tile_len; k2 <<= 1) {
            for (uint32_t j = k2 >> 1; j > 0; j >>= 1) {
                for (uint32_t q = threadIdx.x; q < tile_len / 2; q += kSortThreads) {
                    const uint32_t i = ((q & ~(j - 1)) << 1) | (q & (j - 1)), l = i | j;
                    const bool descending = ((base + i) & k2) == 0;
                    const u64 a = tile[i], b = tile[l];
                    if (descending ? a < b : a > b) {
                        tile[i] = b;
                        tile[l] = a;
                    }
                }
                __syncthreads();
            }
        }
        for (uint32_t t = threadIdx.x; t < tile_len; t += kSortThreads) keys[base + t] = tile[t];
        __syncthreads();
    }
    // the longer steps over global memory, the rest of each merge over the tiles again
    for (uint32_t k2 = 2 * kSortTile; k2 <= n_pad && k2 != 0; k2 <<= 1) {
        for (uint32_t j = k2 >> 1; j >= (uint32_t)kSortTile; j >>= 1) {
            for (uint32_t q = threadIdx.x; q < n_pad / 2; q += kSortThreads) {
                const uint32_t i = ((q & ~(j - 1)) << 1) | (q & (j - 1)), l = i | j;
                const bool descending = (i & k2) == 0;
                const u64 a = keys[i], b = keys[l];
                if (descending ? a < b : a > b) {
                    keys[i] = b;
                    keys[l] = a;
                }
            }
            __syncthreads();  // (orders this block's global writes before its next reads)
        }
        for (uint32_t base = 0; base < n_pad; base += kSortTile) {
            for (uint32_t t = threadIdx.x; t < kSortTile; t += kSortThreads) tile[t] = keys[base + t];
            __syncthreads();
            tile_steps(tile, base, k2, kSortTile / 2);
            for (uint32_t t = threadIdx.x; t < kSortTile; t += kSortThreads) keys[base + t] = tile[t];
            __syncthreads();
        }
    }
    for (size_t jj = threadIdx.x; jj < k; jj += kSortThreads) {
        const uint32_t col = ~(uint32_t)keys[jj];
        values[row * k + jj] = x[col];
        indices[row * k + jj] = (float)col;
    }
}

}  // namespace

size_t sort_rows_scratch_bytes(size_t rows, size_t cols, size_t* rows_per_launch) {
    size_t n_pad = 1;
    while (n_pad < cols) n_pad <<= 1;
    const size_t budget = (size_t)256 << 20;  // scratch of one launch
    size_t batch = budget / (n_pad * 8);
    batch = batch < 1 ? 1 : batch > rows ? rows : batch;
    if (rows_per_launch) *rows_per_launch = batch;
    return batch * n_pad * 8;
}

cudaError_t launch_sort_rows(const float* in, float* values, float* indices, size_t rows, size_t cols, size_t k, bool largest,
                             void* scratch, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    size_t batch = 0;
    sort_rows_scratch_bytes(rows, cols, &batch);
    uint32_t n_pad = 1;
    while (n_pad < cols) n_pad <<= 1;
    for (size_t first = 0; first < rows; first += batch) {
        const unsigned blocks = (unsigned)(rows - first < batch ? rows - first : batch);
        if (largest) {
            sort_rows_kernel<true><<<blocks, kSortThreads, 0, stream>>>(in, values, indices, static_cast<u64*>(scratch), cols, k,
                                                                       n_pad, first);
        } else {
            sort_rows_kernel<false><<<blocks, kSortThreads, 0, stream>>>(in, values, indices, static_cast<u64*>(scratch), cols, k,
                                                                        n_pad, first);
        }
        if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

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
    // The short way (k <= 256) needs no keys in shared memory; if one of its lists overflows, the
    // long way sweeps global memory.  Otherwise the keys are kept when they fit.
    p.list_cap = k <= (size_t)kThreads ? 4 * (p.k_pad < 64 ? 64 : p.k_pad) : 0;
    const size_t entries = p.k_pad + p.list_cap + (p.cluster > 1 && p.list_cap != 0 ? (size_t)p.cluster * p.k_pad : 0);
    p.in_shared = p.list_cap == 0 && p.slice <= (uint32_t)kSliceMax &&
                  entries * 8 + (size_t)p.slice * 4 + 4096 <= 227 * 1024 ? 1 : 0;
    const size_t shared = entries * 8 + (p.in_shared ? (size_t)p.slice * 4 + 32 : 0);
    if (rows * (size_t)p.cluster > 0x7FFFFFFFull) return cudaErrorInvalidConfiguration;
    if (shared > 48 * 1024) {
        // Once per device and direction (the call sets the same value every time, so two host threads
        // that both find the flag clear do no harm).
        static bool lifted[2][64] = {};
        int device = 0;
        if (cudaError_t e = cudaGetDevice(&device); e != cudaSuccess) return e;
        bool& done = lifted[largest ? 1 : 0][device & 63];
        if (!done) {
            const cudaError_t e = largest ? allow_all_dynamic_shared(topk_rows_kernel<true>)
                                          : allow_all_dynamic_shared(topk_rows_kernel<false>);
            if (e != cudaSuccess) return e;
            done = true;
        }
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
    config.numAttrs = p.cluster > 1 ? 1 : 0;  // a row of one CTA is an ordinary launch
    return largest ? cudaLaunchKernelEx(&config, topk_rows_kernel<true>, p) : cudaLaunchKernelEx(&config, topk_rows_kernel<false>, p);
}

}  // namespace psx
