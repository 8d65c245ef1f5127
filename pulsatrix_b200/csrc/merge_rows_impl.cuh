// The survivor stage as device code, shared by the kernels that run it: one row per CTA.
#pragma once

#include "../../include/psx_b200.h"
#include "merge_rows.cuh"

#ifndef PSX_MERGE_STAGE
#define PSX_MERGE_STAGE(i) do {} while (0)
#endif

namespace psx {
namespace survivor {

using u64 = unsigned long long;

struct Decision {
    long long token;
    int status;
    int survivors;
    double draw_margin;
    double top_p_margin;
};

__device__ __forceinline__ uint32_t key_ord(u64 k) { return (uint32_t)(k >> 32); }
__device__ __forceinline__ uint32_t key_col(u64 k) { return ~(uint32_t)k; }

// Step 3, by one thread, in the reference's summation order.  keyA: the ns survivors of top-k by
// (value desc, column asc); keyB: (column << 32 | position in keyA) ascending; ex[pos] =
// exp(x'[pos] - x'max).  `rest` is the processed mass (relative to x'max) of everything that is
// not in keyA and still alive, `rest_bound` an upper bound on any such entry's ex.
__device__ inline void decide(const MergeParams& p, const u64* keyA, const u64* keyB, const double* ex, uint8_t* alive,
                       int ns, bool rest_alive, double rest, double rest_bound, double u, Decision& out) {
    out.status = PSX_ROW_OK;
    out.token = -1;
    out.draw_margin = INFINITY;
    out.top_p_margin = INFINITY;
    out.survivors = 0;
    const bool sample = p.do_sample != 0;

    if (sample && p.top_p < 1.0f) {  // src/generation.cpp:89-103
        const double limit = 1.0 - (double)p.top_p;
        double sum = rest_alive ? rest : 0.0;
        for (int j = 0; j < ns; ++j) sum += ex[(uint32_t)keyB[j]];
        double cumulative = 0.0;
        if (rest_alive) {
            // Everything outside the list is smaller than everything in it, so it leads the
            // ascending walk; it must fall below the cut as a whole.
            cumulative = rest / sum;
            out.top_p_margin = fabs(cumulative - limit);
            if (!(cumulative <= limit)) { out.status = PSX_ROW_TOO_WIDE; return; }
            rest_alive = false;
        }
        bool crossed = false;
        int group_end = ns;
        while (group_end > 0 && !crossed) {
            const uint32_t ord = key_ord(keyA[group_end - 1]);
            int group_begin = group_end - 1;
            while (group_begin > 0 && key_ord(keyA[group_begin - 1]) == ord) --group_begin;
            for (int pos = group_begin; pos < group_end; ++pos) {  // equal values: lower column first
                if (group_begin == 0 && pos == group_end - 1) break;  // the last of the walk always stays
                cumulative += ex[pos] / sum;
                const double dist = fabs(cumulative - limit);
                if (dist < out.top_p_margin) out.top_p_margin = dist;
                if (cumulative <= limit) {
                    alive[pos] = 0;
                } else {
                    crossed = true;
                    break;
                }
            }
            group_end = group_begin;
        }
    }

    if (sample && p.min_p > 0.0f) {  // src/generation.cpp:104-111
        double sum = rest_alive ? rest : 0.0;
        for (int j = 0; j < ns; ++j) {
            const uint32_t pos = (uint32_t)keyB[j];
            if (alive[pos]) sum += ex[pos];
        }
        const double top = ex[0] / sum;  // position 0 is the first maximum and is never removed
        const double floor_p = p.min_p * top;
        for (int pos = 1; pos < ns; ++pos) {
            if (alive[pos] && ex[pos] / sum < floor_p) alive[pos] = 0;
        }
        if (rest_alive) {
            if (rest_bound / sum < floor_p) rest_alive = false;
            else { out.status = PSX_ROW_TOO_WIDE; return; }
        }
    }

    int survivors = 0;
    for (int pos = 0; pos < ns; ++pos) survivors += alive[pos];
    out.survivors = survivors;

    long long chosen = key_col(keyA[0]);  // src/generation.cpp:135 first maximum: lower column wins
    if (sample) {                         // src/generation.cpp:140-152
        if (rest_alive) { out.status = PSX_ROW_TOO_WIDE; return; }
        double sum = 0.0;
        for (int j = 0; j < ns; ++j) {
            const uint32_t pos = (uint32_t)keyB[j];
            if (alive[pos]) sum += ex[pos];
        }
        double cumulative = 0.0, before = 0.0;
        for (int j = 0; j < ns; ++j) {
            const uint32_t pos = (uint32_t)keyB[j];
            if (!alive[pos]) continue;
            const double pr = ex[pos] / sum;
            if (pr == 0.0) continue;
            before = cumulative;
            cumulative += pr;
            chosen = (long long)(keyB[j] >> 32);
            if (u < cumulative) break;
        }
        const double lo = fabs(u - before), hi = fabs(u - cumulative);
        out.draw_margin = before == 0.0 ? hi : fmin(lo, hi);
    }
    out.token = chosen;
}

// Sorts n <= blockDim.x distinct 64-bit keys in shared memory by counting, one key per thread:
// a key's place is the number of keys that come before it.  Starts and ends with a barrier.
__device__ __forceinline__ void block_rank_sort(u64* keys, int n, bool descending) {
    __syncthreads();
    const int i = threadIdx.x;
    u64 mine = 0;
    int place = 0;
    if (i < n) {
        mine = keys[i];
        for (int j = 0; j < n; ++j) {
            const u64 other = keys[j];
            place += (descending ? other > mine : other < mine) ? 1 : 0;
        }
    }
    __syncthreads();
    if (i < n) keys[place] = mine;
    __syncthreads();
}

// Step 3 of the survivor stage for a SHORT list (n <= blockDim.x, the usual case after a top-k or
// for greedy): thread i owns entry i of the unsorted keys.  Places in the three orders the
// reference walks (value descending, column ascending, and the top-p walk: value ascending then
// column ascending) come from counting, so nothing is sorted; every thread drops what it
// contributes into the slot of its place, so the additions, whose order the reference fixes, are
// one thread running down a contiguous array, and the per-entry divisions by the softmax sums
// run in parallel (src/generation.cpp:80-152).  Exact: same operations, same order, same precision.
struct SmallScratch {
    uint32_t* order_b;   // entry of the j-th survivor by ascending column
    uint32_t* cols;      // column of the j-th entry by (value descending, column ascending)
    double* ex;          // exp(x - x_max) of the j-th survivor by ascending column (0 once a filter removed it)
    double* pr;          // probabilities, in the order of the walk that reads them
    uint8_t* alive;      // per entry: what survived (the min-p filter and the survivor export read it)
    uint32_t* shared;    // a few broadcast words
    double* sum;         // one broadcast double
};

// Eight doubles from index j of v (zero beyond n), by one thread; the loads are independent.
__device__ __forceinline__ void load8(const double* __restrict__ v, int j, int n, double (&x)[8]) {
#pragma unroll
    for (int q = 0; q < 8; ++q) x[q] = j + q < n ? v[j + q] : 0.0;
}

// sum of v[0..n) in index order by one thread: the next eight loads are in flight while eight
// additions, each waiting for the one before, are made.
__device__ __forceinline__ double ordered_sum(const double* __restrict__ v, int n, double start) {
    double sum = start;
    double x[8], y[8];
    load8(v, 0, n, x);
    for (int j = 0; j < n; j += 8) {
        load8(v, j + 8, n, y);
#pragma unroll
        for (int q = 0; q < 8; ++q) sum += x[q];  // adding the zeros beyond n changes nothing
#pragma unroll
        for (int q = 0; q < 8; ++q) x[q] = y[q];
    }
    return sum;
}

// The reference's running-sum walks (src/generation.cpp:96-102 and :144-151) by one thread: adds
// v[0], v[1], ... to `start` in index order and stops at the first index whose sum is above
// `level` (kStrict: level < sum; else: !(sum <= level)).  Eight sums are formed before they are
// compared, so the comparisons do not sit in the chain of additions.
struct WalkEnd {
    int index;      // where the sum first went above the level; n when it never did
    double before;  // the sum before that index's own share (the final sum when index == n)
    double upto;    // the sum including it (the final sum when index == n)
    int last;       // when index == n: the last index with a share that is not zero; -1 when none
};
template <bool kStrict>
__device__ __forceinline__ WalkEnd ordered_walk(const double* __restrict__ v, int n, double start, double level) {
    WalkEnd end;
    end.index = n;
    end.last = -1;
    double carried = start;  // the sum before index j
    double x[8], y[8];
    load8(v, 0, n, x);
    for (int j = 0; j < n; j += 8) {
        load8(v, j + 8, n, y);
        double run[8];
        double sum = carried;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            sum += x[q];
            run[q] = sum;
        }
        uint32_t above = 0, some = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const bool over = kStrict ? level < run[q] : !(run[q] <= level);
            above |= (over && j + q < n ? 1u : 0u) << q;
            some |= (x[q] != 0.0 ? 1u : 0u) << q;
        }
        if (above != 0) {
            const int q = __ffs(above) - 1;
            end.index = j + q;
            end.before = carried;
            end.upto = run[0];
#pragma unroll
            for (int r = 1; r < 8; ++r) {
                if (r <= q) { end.before = run[r - 1]; end.upto = run[r]; }
            }
            return end;
        }
        if (some != 0) end.last = j + 31 - __clz(some);
        carried = sum;
#pragma unroll
        for (int q = 0; q < 8; ++q) x[q] = y[q];
    }
    end.before = carried;
    end.upto = carried;
    return end;
}

__device__ inline void decide_small(const MergeParams& p, const u64* keyA, int n, bool top_k_on, bool rest_in_play,
                             double rest, float keep_from_x, double u, const SmallScratch& w, Decision* result) {
    const int tid = threadIdx.x;
    const bool sample = p.do_sample != 0;
    // T threads (a power of two, neighbours in a warp) share the counting loop of one entry.
    int n_pad = 8;
    while (n_pad < n) n_pad <<= 1;
    const int T = kMergeThreads / n_pad, shift_t = __ffs(T) - 1;
    const int e = tid >> shift_t, slice = tid & (T - 1);
    const bool in_range = e < n;
    const bool have = in_range && slice == 0;  // the thread that owns entry e from here on
    const u64 mine = in_range ? keyA[e] : 0;
    const uint32_t my_ord = key_ord(mine), my_col = key_col(mine);
    const bool cut_k = top_k_on && n >= p.top_k;

    // Among all n: how many come before mine by (value desc, column asc) -- the keys compare that
    // way as integers --, how many of those share my value, how many share my value at all, and
    // how many sit at lower columns.
    uint32_t counts = 0, lower = 0;  // three 10-bit fields; one count
    if (in_range) {
        for (int j = slice; j < n; j += T) {
            const u64 other = keyA[j];
            const uint32_t before = other > mine ? 1u : 0u, same = key_ord(other) == my_ord ? 1u : 0u;
            counts += before + ((before & same) << 10) + (same << 20);
            lower += key_col(other) < my_col ? 1u : 0u;
        }
    }
    for (int o = T >> 1; o > 0; o >>= 1) {
        counts += __shfl_xor_sync(0xFFFFFFFFu, counts, o);
        lower += __shfl_xor_sync(0xFFFFFFFFu, lower, o);
    }
    const int place = (int)(counts & 1023u), same_before = (int)((counts >> 10) & 1023u), same = (int)(counts >> 20);
    if (have) {
        if (place == 0) { w.shared[0] = my_ord; w.shared[1] = (uint32_t)e; }  // the first maximum
        if (cut_k && place == (int)p.top_k - 1) w.shared[2] = my_ord;        // the k-th value
    }
    if (tid == 0 && !cut_k) w.shared[2] = 0;
    __syncthreads();
    PSX_MERGE_STAGE(10);
    const uint32_t top_ord = w.shared[0], best = w.shared[1], kth = w.shared[2];
    const bool survivor = have && my_ord >= kth;  // src/generation.cpp:85: ties at the k-th value stay
    if (have) w.cols[place] = my_col;             // the survivors are exactly the first ns places
    const int ns = __syncthreads_count(survivor ? 1 : 0);
    bool rest_alive = !top_k_on && sample && rest_in_play;

    // Place by ascending column among the survivors, and in the top-p walk (value ascending, then
    // column ascending): the survivors below my value, plus those of my value at lower columns.
    // Place by ascending column: the lower columns among all n, less those of the few entries
    // beyond the survivors.
    int place_b = (int)lower;
    const int place_w = ns - (place - same_before) - same + same_before;
    double my_ex = 0.0;
    if (survivor) {
        for (int j = ns; j < n; ++j) place_b -= w.cols[j] < my_col ? 1 : 0;
        my_ex = exp((double)from_ordered_key(my_ord) - (double)from_ordered_key(top_ord));  // src/generation.cpp:46
        w.order_b[place_b] = (uint32_t)e;
        w.ex[place_b] = my_ex;
        if (e == (int)best) w.shared[5] = (uint32_t)place_b;
    }
    PSX_MERGE_STAGE(11);
    bool alive = survivor;
    Decision d;
    d.status = PSX_ROW_OK;
    d.token = -1;
    d.survivors = 0;
    d.draw_margin = INFINITY;
    d.top_p_margin = INFINITY;
    __syncthreads();

    if (sample && p.top_p < 1.0f) {  // src/generation.cpp:89-103
        if (tid == 0) *w.sum = ordered_sum(w.ex, ns, rest_alive ? rest : 0.0);  // column order, as the reference sums
        __syncthreads();
        if (survivor) w.pr[place_w] = my_ex / *w.sum;
        __syncthreads();
        if (tid == 0) {
            const double limit = 1.0 - (double)p.top_p;
            double start = 0.0;
            if (rest_alive) {  // everything outside the list leads the ascending walk and must fall as a whole
                start = rest / *w.sum;
                if (!(start <= limit)) d.status = PSX_ROW_TOO_WIDE;
            }
            int cut = 0;  // places of the walk below `cut` are removed; the last of the walk always stays
            if (d.status == PSX_ROW_OK) {
                const WalkEnd end = ordered_walk<false>(w.pr, ns - 1, start, limit);
                cut = end.index;
                // The running sum only grows, so of all the sums compared with the limit the nearest
                // are the last one at or below it and the first one above it.
                if (cut > 0 || rest_alive) d.top_p_margin = fabs(end.before - limit);
                if (cut < ns - 1) d.top_p_margin = fmin(d.top_p_margin, fabs(end.upto - limit));
            } else {
                d.top_p_margin = fabs(start - limit);
            }
            w.shared[4] = (uint32_t)cut;
        }
        rest_alive = false;
        __syncthreads();
        alive = survivor && place_w >= (int)w.shared[4];
    }
    PSX_MERGE_STAGE(12);

    if (sample && p.min_p > 0.0f) {  // src/generation.cpp:104-111 (rare: left to one thread)
        if (have) w.alive[e] = alive ? 1 : 0;
        __syncthreads();
        if (tid == 0 && d.status == PSX_ROW_OK) {
            double sum = rest_alive ? rest : 0.0;
            for (int j = 0; j < ns; ++j) {
                if (w.alive[w.order_b[j]]) sum += w.ex[j];
            }
            const double floor_p = p.min_p * (w.ex[w.shared[5]] / sum);
            for (int j = 0; j < ns; ++j) {
                const uint32_t o = w.order_b[j];
                if (w.alive[o] && o != best && w.ex[j] / sum < floor_p) w.alive[o] = 0;
            }
            if (rest_alive) {
                const double bound = exp((double)keep_from_x - (double)from_ordered_key(top_ord));
                if (bound / sum < floor_p) w.shared[3] = 0; else d.status = PSX_ROW_TOO_WIDE;
            }
        }
        if (tid == 0) w.shared[3] = (rest_alive && d.status == PSX_ROW_OK && w.shared[3] != 0) ? 1u : 0u;
        __syncthreads();
        rest_alive = rest_alive && w.shared[3] != 0;
        alive = have && w.alive[e] != 0;
    }
    PSX_MERGE_STAGE(13);

    if (sample) {  // src/generation.cpp:140-152
        if (survivor) w.ex[place_b] = alive ? my_ex : 0.0;  // adding 0.0 leaves the sum as skipping does
        const int alive_count = __syncthreads_count(alive ? 1 : 0);
        if (tid == 0) {
            *w.sum = ordered_sum(w.ex, ns, 0.0);
            d.survivors = alive_count;
            if (rest_alive && d.status == PSX_ROW_OK) d.status = PSX_ROW_TOO_WIDE;
        }
        __syncthreads();
        if (survivor) w.pr[place_b] = alive ? my_ex / *w.sum : 0.0;
        __syncthreads();
        if (tid == 0 && d.status == PSX_ROW_OK) {
            // The first place whose running sum exceeds u; a probability of zero (removed, or
            // underflowed) leaves the sum where it was and is never the first.  If u is not
            // below the last sum either, the last place with a probability is drawn.
            const WalkEnd end = ordered_walk<true>(w.pr, ns, 0.0, u);
            const int chosen = end.index < ns ? end.index : end.last;
            if (end.index < ns) {
                const double lo = fabs(u - end.before), hi = fabs(u - end.upto);
                d.draw_margin = end.before == 0.0 ? hi : fmin(lo, hi);
            } else {
                d.draw_margin = fabs(u - end.upto);
            }
            d.token = key_col(keyA[chosen >= 0 ? w.order_b[chosen] : best]);
        }
    } else if (tid == 0) {
        d.survivors = ns;
        d.token = key_col(keyA[best]);  // src/generation.cpp:135: the first maximum, lower column wins
    }
    PSX_MERGE_STAGE(14);
    if (have) w.alive[e] = alive ? 1 : 0;  // what survived, for a caller that wants the set itself
    if (tid == 0) *result = d;
    __syncthreads();
}

// Block-wide sum in a fixed order (same result in every thread); scratch holds one double per warp.
__device__ __forceinline__ double block_sum_fixed(double v, double* scratch) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    double r = 0.0;
#pragma unroll
    for (int w = 0; w < kMergeThreads / 32; ++w) r += scratch[w];
    return r;
}

// Block-wide maximum / minimum of 32-bit keys and minimum of doubles (same result in every thread).
__device__ __forceinline__ uint32_t block_max_u32(uint32_t v, double* scratch) {
    v = __reduce_max_sync(0xFFFFFFFFu, v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = (double)v;  // exact: 32-bit integers fit a double
    __syncthreads();
    double r = 0.0;
#pragma unroll
    for (int w = 0; w < kMergeThreads / 32; ++w) r = fmax(r, scratch[w]);
    return (uint32_t)r;
}
__device__ __forceinline__ uint32_t block_min_u32(uint32_t v, double* scratch) {
    return ~block_max_u32(~v, scratch);
}
__device__ __forceinline__ double block_min_f64(double v, double* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmin(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    double r = scratch[0];
#pragma unroll
    for (int w = 1; w < kMergeThreads / 32; ++w) r = fmin(r, scratch[w]);
    return r;
}

// Steps 3 of the survivor stage for a LONG list (sampling without a top-k: hundreds to thousands
// of entries), by the whole block and without sorting.  The reference's decisions are threshold
// decisions on monotone cumulative sums -- the top-p cut along ascending (value, column), the
// min-p floor, the CDF crossing along ascending column -- so each is found by a bisection whose
// probes are block-wide masked sums of exp in a fixed order.  Those sums differ from the
// reference's sequential ones by rounding only (~n * 1e-16), so whenever a decision comes closer
// than kExactMargin to its boundary the function gives up (returns false) and the caller takes the
// sorted, sequential replay instead.  keyA: n unsorted keys (ordered value << 32 | ~column);
// ex[i] = exp(x_i - x_max); alive[i] is set here.
constexpr double kExactMargin = 1e-9;
constexpr int kMassPasses = 8;  // histograms decide_wide needs: four passes over the value, four over the column

// Along ascending key (key_of(i) over the entries with in_play(i)), the first key K at which the
// running mass start + sum of ex over keys <= K rises above `target`; 8-bit radix passes from
// bit `top_shift` down, one barrier each: every pass adds the masses of the keys that still match
// into its own 256-bin histogram (hist: (top_shift / 8 + 1) * 768 words, all zero on entry) and
// every warp scans the bins for itself.  below = start + mass of the keys < K; at =
// mass of K.  When the mass never rises above the target, K is the largest key in play.
// Masses (all in [0, 1]) are added as fixed-point numbers of 2^-44, in three pieces of 15 bits,
// each piece into its own 32-bit bin: integer additions give the same sums in any order, native
// 32-bit shared-memory atomics do not mind many keys in one bin, and 2^15 entries cannot overflow
// a piece.  What the rounding to 2^-44 loses, at most n * 2.9e-14 in all, is far inside
// kExactMargin.
constexpr double kMassUnit = 17592186044416.0;  // 2^44
// `known` holds the digits above `top_shift + 8` that every key in play shares (0 when top_shift
// is the keys' top digit): the passes over them are skipped.
template <class KeyOf, class InPlay, class MassOf>
__device__ inline void mass_select(KeyOf key_of, InPlay in_play, MassOf mass_of, int n, int top_shift, uint32_t known,
                                   double start, double target, uint32_t* hist, uint32_t& K, double& below, double& at) {
    const int tid = threadIdx.x, lane = tid & 31;
    uint32_t mask = top_shift >= 24 ? 0u : ~((1u << (top_shift + 8)) - 1u);
    uint32_t prefix = known & mask;
    // the running mass is compared as an integer: units of 2^-44 above `start`
    const double room = (target - start) * kMassUnit;
    const u64 target_units = room <= 0.0 ? 0ull : room >= 1.8e19 ? ~0ull : (u64)room;
    const bool already_above = !(start <= target);
    u64 carried = 0;  // units below the current prefix
    u64 at_units = 0;
#pragma unroll 1
    for (int shift = top_shift; shift >= 0; shift -= 8) {
        uint32_t* h = hist + 768 * (shift >> 3);
        for (int i = tid; i < n; i += kMergeThreads) {
            if (!in_play(i)) continue;
            const uint32_t key = key_of(i);
            if ((key & mask) != prefix) continue;
            const u64 units = (u64)__double2ull_rn(mass_of(i) * kMassUnit);  // at most 2^44
            uint32_t* bin = h + ((key >> shift) & 255u);
            atomicAdd(bin, (uint32_t)units & 0x7FFFu);
            atomicAdd(bin + 256, (uint32_t)(units >> 15) & 0x7FFFu);
            atomicAdd(bin + 512, (uint32_t)(units >> 30));
        }
        __syncthreads();
        // lane L owns bins 8L .. 8L+7, ascending
        u64 run[8];
        u64 local = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int at_bin = 8 * lane + q;
            local += (u64)h[at_bin] + ((u64)h[at_bin + 256] << 15) + ((u64)h[at_bin + 512] << 30);
            run[q] = local;
        }
        u64 incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const u64 up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += up;
        }
        const u64 before_mine = carried + (incl - local);
        int first = 8, last = -1;  // first bin of mine that rises above the target; last bin of mine that holds mass
#pragma unroll
        for (int q = 7; q >= 0; --q) {
            if (already_above ? run[q] != (q ? run[q - 1] : 0ull) : before_mine + run[q] > target_units) first = q;
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            if (run[q] != (q ? run[q - 1] : 0ull)) last = q;
        }
        const uint32_t crossing = __ballot_sync(0xFFFFFFFFu, first < 8), holding = __ballot_sync(0xFFFFFFFFu, last >= 0);
        int src, q_src;
        if (crossing != 0) {
            src = __ffs(crossing) - 1;
            q_src = __shfl_sync(0xFFFFFFFFu, first, src);
        } else {  // never above the target: the largest key in play (holding != 0 while anything is in play)
            src = holding != 0 ? 31 - __clz(holding) : 0;
            q_src = max(0, __shfl_sync(0xFFFFFFFFu, last, src));
        }
        u64 below_bin = before_mine, mass_bin = run[0];
#pragma unroll
        for (int q = 1; q < 8; ++q) {
            if (q <= q_src) { below_bin = before_mine + run[q - 1]; mass_bin = run[q] - run[q - 1]; }
        }
        carried = __shfl_sync(0xFFFFFFFFu, below_bin, src);
        at_units = __shfl_sync(0xFFFFFFFFu, mass_bin, src);
        prefix |= (uint32_t)(8 * src + q_src) << shift;
        mask |= 255u << shift;
    }
    K = prefix;
    below = start + (double)carried / kMassUnit;
    at = (double)at_units / kMassUnit;
}

// Called by the whole block with ex[i] = exp(x_i - x_top) and alive[i] = 1 for the n entries of the list,
// list_sum their sum in block_sum_fixed's order, top_key the largest value key and `differing` the
// bits in which the value keys of the list are not all the same; `hist` is kWideWords words, the
// first kMassPasses * 768 of them zero.
constexpr int kCompactCap = 1024;                     // survivors that are drawn from a list of their own
constexpr int kWideWords = kMassPasses * 768 + 8;
__device__ inline bool decide_wide(const MergeParams& p, const u64* keyA, const double* ex, uint8_t* alive, int n,
                            bool rest_alive, double rest, double rest_bound, double u, double* scratch, uint32_t* hist,
                            uint32_t top_key, uint32_t differing, double list_sum, Decision& out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    out.status = PSX_ROW_OK;
    out.token = -1;
    out.draw_margin = INFINITY;
    out.top_p_margin = INFINITY;
    out.survivors = 0;
    auto masked_sum = [&](auto keep) {
        double v = 0.0;
        for (int i = tid; i < n; i += kMergeThreads) {
            if (keep(i)) v += ex[i];
        }
        return block_sum_fixed(v, scratch);
    };

    if (p.top_p < 1.0f) {  // src/generation.cpp:89-103
        const double limit = 1.0 - (double)p.top_p;
        const double base = rest_alive ? rest : 0.0;
        const double sum = base + list_sum;
        double margin = INFINITY;
        if (rest_alive) {
            const double lead = base / sum;  // everything outside the list leads the ascending walk
            margin = fabs(lead - limit);
            if (!(lead <= limit)) { out.status = PSX_ROW_TOO_WIDE; return true; }
            rest_alive = false;
        }
        // Smallest value key whose entries push the cumulative mass past the limit.
        if (limit >= 1.0 - 1e-12) return false;
        uint32_t cut;
        double mass_below, mass_at;
        // (neighbouring floats share their leading digits: a pass over a digit that all share would only
        // queue every entry at one bin)
        const int value_shift = differing >> 24 ? 24 : differing >> 16 ? 16 : differing >> 8 ? 8 : 0;
        mass_select([&](int i) { return key_ord(keyA[i]); }, [&](int) { return true; }, [&](int i) { return ex[i]; }, n,
                    value_shift, top_key, base, limit * sum, hist, cut, mass_below, mass_at);
        const double below = mass_below / sum;
        margin = fmin(margin, fabs(below - limit));
        // Entries equal to the cut value go in ascending column order, one probability each.
        double ties = 0.0;
        for (int i = tid; i < n; i += kMergeThreads) ties += key_ord(keyA[i]) == cut ? 1.0 : 0.0;
        const int group = (int)block_sum_fixed(ties, scratch);
        const double each = exp((double)from_ordered_key(cut) - (double)from_ordered_key(top_key)) / sum;
        double cumulative = below;
        int removed = 0;
        for (int j = 0; j < group; ++j) {
            cumulative += each;
            margin = fmin(margin, fabs(cumulative - limit));
            if (cumulative <= limit) ++removed; else break;
        }
        if (cut == top_key && removed >= group) removed = group - 1;  // the last of the walk always stays
        out.top_p_margin = margin;
        if (margin < kExactMargin) return false;
        for (int i = tid; i < n; i += kMergeThreads) {
            const uint32_t k = key_ord(keyA[i]);
            if (k < cut) {
                alive[i] = 0;
            } else if (k == cut && removed > 0) {
                const uint32_t col = key_col(keyA[i]);
                int before = 0;  // ties with a lower column
                for (int j = 0; j < n; ++j) before += (key_ord(keyA[j]) == cut && key_col(keyA[j]) < col) ? 1 : 0;
                if (before < removed) alive[i] = 0;
            }
        }
        __syncthreads();
    }

    if (p.min_p > 0.0f) {  // src/generation.cpp:104-111
        const double sum = (rest_alive ? rest : 0.0) + masked_sum([&](int i) { return alive[i] != 0; });
        const double floor_p = p.min_p * (1.0 / sum);  // the most likely entry has exp(0) = 1
        uint32_t best = 0xFFFFFFFFu;  // the first maximum: lowest column among the top values
        for (int i = tid; i < n; i += kMergeThreads) {
            if (key_ord(keyA[i]) == top_key) best = min(best, key_col(keyA[i]));
        }
        best = block_min_u32(best, scratch);
        double closest = INFINITY;
        for (int i = tid; i < n; i += kMergeThreads) {
            if (!alive[i] || (key_ord(keyA[i]) == top_key && key_col(keyA[i]) == best)) continue;
            const double pr = ex[i] / sum;
            closest = fmin(closest, fabs(pr - floor_p) / floor_p);
            if (pr < floor_p) alive[i] = 0;
        }
        closest = block_min_f64(closest, scratch);  // its barriers also publish the alive flags
        if (closest < 1e-12) return false;
        if (rest_alive) {
            if (rest_bound / sum < floor_p) rest_alive = false;
            else { out.status = PSX_ROW_TOO_WIDE; return true; }
        }
    }

    // The survivors, counted warp after warp in list order; when few are left of a long list they move
    // to a list of their own (over the histograms of the value selection, done with by now), in that
    // same order, and the draw looks at nothing else.
    constexpr int kWarps = kMergeThreads / 32;
    uint32_t* warp_counts = hist + kMassPasses * 768;
    uint32_t* small_cols = hist;
    double* small_ex = reinterpret_cast<double*>(hist + kCompactCap);
    const int chunk = ((n + kMergeThreads - 1) / kMergeThreads) * 32;  // entries of one warp
    const int chunk_begin = warp * chunk, chunk_end = min(n, chunk_begin + chunk);
    int mine = 0;
    for (int i = chunk_begin + lane; i < chunk_begin + chunk; i += 32) {
        mine += __popc(__ballot_sync(0xFFFFFFFFu, i < chunk_end && alive[i] != 0));
    }
    if (lane == 0) warp_counts[warp] = (uint32_t)mine;
    __syncthreads();
    int before_mine = 0, survivors = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        const int c = (int)warp_counts[w];
        before_mine += w < warp ? c : 0;
        survivors += c;
    }
    out.survivors = survivors;

    // src/generation.cpp:140-152: the first column whose cumulative probability exceeds u.
    if (rest_alive) { out.status = PSX_ROW_TOO_WIDE; return true; }
    const bool on_their_own = survivors <= kCompactCap;
    if (on_their_own) {
        int at = before_mine;
        for (int i = chunk_begin + lane; i < chunk_begin + chunk; i += 32) {
            const bool stays = i < chunk_end && alive[i] != 0;
            const uint32_t staying = __ballot_sync(0xFFFFFFFFu, stays);
            if (stays) {
                const int slot = at + __popc(staying & ((1u << lane) - 1u));
                small_cols[slot] = key_col(keyA[i]);
                small_ex[slot] = ex[i];
            }
            at += __popc(staying);
        }
        __syncthreads();
    }
    double sum;
    if (on_their_own) {
        double v = 0.0;
        for (int i = tid; i < survivors; i += kMergeThreads) v += small_ex[i];
        sum = block_sum_fixed(v, scratch);
    } else {
        sum = masked_sum([&](int i) { return alive[i] != 0; });
    }
    // The first column at which the running mass rises above u * sum.
    uint32_t hi;
    double mass_before, mass_at;
    const int column_shift = p.vocab <= (1 << 16) ? 8 : p.vocab <= (1 << 24) ? 16 : 24;
    if (on_their_own) {
        mass_select([&](int i) { return small_cols[i]; }, [&](int) { return true; }, [&](int i) { return small_ex[i]; }, survivors,
                    column_shift, 0u, 0.0, u * sum, hist + 4 * 768, hi, mass_before, mass_at);
    } else {
        mass_select([&](int i) { return key_col(keyA[i]); }, [&](int i) { return alive[i] != 0; }, [&](int i) { return ex[i]; }, n,
                    column_shift, 0u, 0.0, u * sum, hist + 4 * 768, hi, mass_before, mass_at);
    }
    const double before = mass_before / sum, upto = (mass_before + mass_at) / sum;
    out.draw_margin = before == 0.0 ? fabs(u - upto) : fmin(fabs(u - before), fabs(u - upto));
    if (out.draw_margin < kExactMargin) return false;
    out.token = (long long)hi;
    return true;
}

// The k-th largest (1-based, k <= m) of m 32-bit keys (key_at(i), i < m): four 8-bit radix
// passes, most significant digit first, one barrier each -- every pass has its own 256-bin
// histogram (hist: 1024 words, all zero on entry, not zero on exit), and every warp scans the
// bins for itself instead of waiting for one warp's answer.  Called by the whole block.
template <class KeyAt>
__device__ inline uint32_t block_select_kth(KeyAt key_at, int m, uint32_t k, uint32_t* hist) {
    const int tid = threadIdx.x, lane = tid & 31;
    uint32_t prefix = 0, mask = 0, remaining = k;
#pragma unroll 1
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        uint32_t* h = hist + 256 * pass;
        for (int i = tid; i < m; i += kMergeThreads) {
            // (Keys that share a digit -- the leading digits of neighbouring floats, or plain ties -- queue at
            // one bin; letting one lane count for all of them with match.any cost more than the queue.)
            const uint32_t key = key_at(i);
            if ((key & mask) == prefix) atomicAdd(&h[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        // lane L owns digits 255-8L down to 248-8L; find where the count from the top reaches `remaining`
        const uint4 lo4 = reinterpret_cast<const uint4*>(h)[62 - 2 * lane], hi4 = reinterpret_cast<const uint4*>(h)[63 - 2 * lane];
        const uint32_t bins[8] = {hi4.w, hi4.z, hi4.y, hi4.x, lo4.w, lo4.z, lo4.y, lo4.x};  // digit 255-8L first
        uint32_t local = 0;
#pragma unroll
        for (int b2 = 0; b2 < 8; ++b2) local += bins[b2];
        uint32_t incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += up;
        }
        const uint32_t excl = incl - local;
        const bool here = excl < remaining && remaining <= incl;
        uint32_t digit = 0, left = 0;
        if (here) {
            uint32_t above = excl;
            int b2 = 0;
#pragma unroll
            for (int q = 0; q < 7; ++q) {
                if (b2 == q && above + bins[q] < remaining) { above += bins[q]; b2 = q + 1; }
            }
            digit = (uint32_t)(255 - 8 * lane - b2);
            left = remaining - above;
        }
        const int src = __ffs(__ballot_sync(0xFFFFFFFFu, here)) - 1;  // exactly one lane while k <= m
        prefix |= __shfl_sync(0xFFFFFFFFu, digit, src < 0 ? 0 : src) << shift;
        remaining = __shfl_sync(0xFFFFFFFFu, left, src < 0 ? 0 : src);
        mask |= 255u << shift;
    }
    return prefix;
}

// What the parts of a row say together, and how many candidates the row has.
struct Joined {
    float raw_max, y_max, thr;
    uint32_t bad_bits;  // bit 0: a non-finite logit; bit 1: a copy that timed out; bit 2: a list that overflowed
    double alive_tail;
    int total;          // candidates of the row (they are in shared memory when it is <= gather_capacity)
};

// Step 1 of the survivor stage: joins the parts' records and brings every candidate of the row
// into shared memory, back to back in a fixed order.  The first 2^slot_shift slots of every
// part's list are fetched together with the counts (the slots exist whatever the count), so the
// usual row costs one trip to memory, not two; N such slots per thread.  What a longer list holds
// beyond them is appended afterwards.
template <int N>
__device__ __forceinline__ Joined join_and_gather(const MergeParams& p, const char* stats_row, const char* counts_row,
                                                  const char* cands_row, uint32_t* cand_l, uint32_t* cand_c,
                                                  float (*s_f)[kMergeThreads / 32], double (*s_d)[kMergeThreads / 32],
                                                  uint32_t (*s_u)[kMergeThreads / 32]) {
    constexpr int kWarps = kMergeThreads / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int shift = p.slot_shift, slots_per_part = 1 << shift, slots = p.parts << shift;
    uint2 fetched[N];
    uint32_t count_of[N];
#pragma unroll
    for (int q = 0; q < N; ++q) {
        const int i = q * kMergeThreads + tid;
        count_of[q] = 0;
        fetched[q] = make_uint2(0, 0);
        if (i < slots) {
            const int part = i >> shift, slot = i & (slots_per_part - 1);
            count_of[q] = min(*reinterpret_cast<const uint32_t*>(counts_row + part * p.count_part_stride), (uint32_t)p.part_cap);
            fetched[q] = reinterpret_cast<const uint2*>(cands_row + part * p.cand_part_stride)[slot];
        }
    }
    float raw_max = -FLT_MAX, y_max = -INFINITY, thr = -INFINITY;
    uint32_t bad = 0;  // bit 0: a non-finite logit; bit 1: a copy that timed out; bit 2: a list that overflowed
    double alive_tail = 0.0;
    for (int i = tid; i < p.parts; i += kMergeThreads) {
        const PartStats s = *reinterpret_cast<const PartStats*>(stats_row + i * p.stats_part_stride);
        raw_max = fmaxf(raw_max, s.raw_max);
        y_max = fmaxf(y_max, s.y_max);
        thr = fmaxf(thr, s.thr);
        bad |= (s.nonfinite & 3u) | (s.overflow ? 4u : 0u);
        alive_tail += (double)s.alive_tail;
    }
    uint32_t warp_total = 0, beyond = 0;
#pragma unroll
    for (int q = 0; q < N; ++q) {
        const uint32_t slot = (uint32_t)(q * kMergeThreads + tid) & (uint32_t)(slots_per_part - 1);
        warp_total += __popc(__ballot_sync(0xFFFFFFFFu, slot < count_of[q]));
        if (slot == 0 && count_of[q] > (uint32_t)slots_per_part) beyond += count_of[q] - (uint32_t)slots_per_part;
    }
    beyond = __reduce_add_sync(0xFFFFFFFFu, beyond);
    {   // one barrier for all the reductions
        raw_max = warp_max(raw_max);
        y_max = warp_max(y_max);
        thr = warp_max(thr);
        bad = __reduce_or_sync(0xFFFFFFFFu, bad);
        alive_tail = warp_sum(alive_tail);
        if (lane == 0) {
            s_f[0][warp] = raw_max; s_f[1][warp] = y_max; s_f[2][warp] = thr;
            s_d[1][warp] = alive_tail;
            s_u[0][warp] = warp_total; s_u[1][warp] = beyond; s_u[2][warp] = bad;
        }
        __syncthreads();
        raw_max = s_f[0][0]; y_max = s_f[1][0]; thr = s_f[2][0];
        bad = 0; alive_tail = 0.0;
        warp_total = 0; beyond = 0;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            raw_max = fmaxf(raw_max, s_f[0][w]);
            y_max = fmaxf(y_max, s_f[1][w]);
            thr = fmaxf(thr, s_f[2][w]);
            bad |= s_u[2][w];
            alive_tail += s_d[1][w];
            beyond += s_u[1][w];
        }
    }
    uint32_t running = 0, fetched_total = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        const uint32_t c = s_u[0][w];
        running += w < warp ? c : 0u;
        fetched_total += c;
    }
    Joined j;
    j.raw_max = raw_max; j.y_max = y_max; j.thr = thr;
    j.bad_bits = bad;
    j.alive_tail = alive_tail;
    j.total = (int)(fetched_total + beyond);
    if (j.bad_bits != 0 || j.total > p.gather_capacity) return j;
#pragma unroll
    for (int q = 0; q < N; ++q) {  // warp after warp, then fetch by fetch, then lane by lane
        const uint32_t slot = (uint32_t)(q * kMergeThreads + tid) & (uint32_t)(slots_per_part - 1);
        const bool valid = slot < count_of[q];
        const uint32_t voters = __ballot_sync(0xFFFFFFFFu, valid);
        if (valid) {
            const uint32_t at = running + __popc(voters & ((1u << lane) - 1u));
            cand_l[at] = fetched[q].x;
            cand_c[at] = fetched[q].y;
        }
        running += __popc(voters);
    }
    if (beyond != 0) {  // rare: the rest of the long lists, part after part
        uint32_t at = fetched_total;
        for (int part = 0; part < p.parts; ++part) {
            const uint32_t count = min(*reinterpret_cast<const uint32_t*>(counts_row + part * p.count_part_stride), (uint32_t)p.part_cap);
            if (count <= (uint32_t)slots_per_part) continue;
            for (uint32_t i = (uint32_t)slots_per_part + tid; i < count; i += kMergeThreads) {
                const uint2 c = reinterpret_cast<const uint2*>(cands_row + part * p.cand_part_stride)[i];
                cand_l[at + i - slots_per_part] = c.x;
                cand_c[at + i - slots_per_part] = c.y;
            }
            at += count - (uint32_t)slots_per_part;
        }
    }
    __syncthreads();
    return j;
}

// One row of the survivor stage, by a whole block of kMergeThreads threads; `dyn` is the block's
// dynamic shared memory (merge_rows_shared_bytes(...) bytes, 8-byte aligned).
__device__ __forceinline__ void merge_row(const MergeParams& p, const int64_t row, u64* dyn) {
    const int cap = p.sort_capacity, gcap = p.gather_capacity;
    u64* keyA = dyn;
    u64* keyB = keyA + cap;
    double* ex = reinterpret_cast<double*>(keyB + cap);
    uint8_t* alive = reinterpret_cast<uint8_t*>(ex + cap);
    // raw logit bits of every candidate; with `overlay` they lie over keyB / ex / alive, which nothing
    // touches before the list in keyA is complete, and are not looked at afterwards
    const bool overlay = p.overlay != 0 && p.logits != nullptr && !(p.do_sample && p.top_k > 0 && p.top_k < p.vocab);
    uint32_t* cand_l = overlay ? reinterpret_cast<uint32_t*>(keyB) : reinterpret_cast<uint32_t*>(alive + cap);
    uint32_t* cand_c = cand_l + gcap;                             // column | flags
    uint32_t* ykeys = reinterpret_cast<uint32_t*>(dyn);           // scratch over the (still unused) sort arrays
    uint32_t* xkeys = reinterpret_cast<uint32_t*>(keyB);          // likewise, clear of the list itself: 4 * cap words

    __shared__ float s_f[3][kMergeThreads / 32];
    __shared__ double s_d[3][kMergeThreads / 32];
    __shared__ uint32_t s_u[3][kMergeThreads / 32];
    __shared__ int s_count;
    __shared__ int s_ns;
    __shared__ uint32_t s_chosen_raw;
    __shared__ Decision s_dec;
    __shared__ __align__(16) uint32_t s_hist[4 * 256];  // the selection's histograms, one per pass

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool apply_t = p.apply_temperature != 0;
    const char* stats_row = static_cast<const char*>(p.stats) + row * p.stats_row_stride;
    const char* counts_row = static_cast<const char*>(p.part_counts) + row * p.count_row_stride;
    const char* cands_row = static_cast<const char*>(p.candidates) + row * p.cand_row_stride;
    auto part_stats = [&](int i) { return *reinterpret_cast<const PartStats*>(stats_row + i * p.stats_part_stride); };

    PSX_MERGE_STAGE(0);
    const double u_row = (p.do_sample && p.uniforms) ? p.uniforms[row] : 0.5;
    if (tid == 0) s_count = 0;
    reinterpret_cast<uint4*>(s_hist)[tid] = make_uint4(0, 0, 0, 0);  // published by the barrier of step 1
    bool hist_clean = true;

    // ---- 1. join the parts; every candidate of the row into shared memory ----------------------------
    Joined joined;
    {
        const int per_thread = ((p.parts << p.slot_shift) + kMergeThreads - 1) / kMergeThreads;
        if (per_thread <= 2) joined = join_and_gather<2>(p, stats_row, counts_row, cands_row, cand_l, cand_c, s_f, s_d, s_u);
        else if (per_thread <= 4) joined = join_and_gather<4>(p, stats_row, counts_row, cands_row, cand_l, cand_c, s_f, s_d, s_u);
        else if (per_thread <= 8) joined = join_and_gather<8>(p, stats_row, counts_row, cands_row, cand_l, cand_c, s_f, s_d, s_u);
        else joined = join_and_gather<16>(p, stats_row, counts_row, cands_row, cand_l, cand_c, s_f, s_d, s_u);
    }
    const float raw_max = joined.raw_max, y_max = joined.y_max, thr = joined.thr;
    const double alive_tail = joined.alive_tail;
    const int total = joined.total;
    if (joined.bad_bits != 0 || total > gcap) {
        if (tid == 0) {
            p.tokens[row] = -1;
            p.log_probs[row] = 0.0f;
            p.row_status[row] = (joined.bad_bits & 2u) ? PSX_ROW_DEVICE_TIMEOUT
                                : (joined.bad_bits & 1u) ? PSX_ROW_NON_FINITE : PSX_ROW_TOO_WIDE;
            if (p.diag) p.diag[row] = psx_row_diag{total, 0, INFINITY, INFINITY};
        }
        return;
    }

    PSX_MERGE_STAGE(3);
    float keep_from = relax_threshold(thr, apply_t, p.temperature);
    const float x_max = temper(y_max, apply_t, p.temperature);
    const bool top_k_on = p.do_sample && p.top_k > 0 && p.top_k < p.vocab;  // src/generation.cpp:80

    // Greedy keeps the maximum and its ties.  With a top-k, the largest part threshold is already a
    // lower bound of the row's k-th largest (that part alone has k logits at or above it), and
    // what reaches it is usually short enough for the one-entry-per-thread path, which finds the
    // k-th value itself; only a longer list pays for an exact selection first (below).
    if (!p.do_sample) keep_from = fmaxf(y_max, -FLT_MAX);

    PSX_MERGE_STAGE(4);
    // ---- 2. raw sum-exp over everything; the list of those that can survive ------------------------
    double z_raw = 0.0, z_rest = 0.0, dropped = 0.0;
    for (int i = tid; i < p.parts; i += kMergeThreads) {
        const PartStats s = part_stats(i);
        z_raw += s.raw_tail * exp((double)s.raw_max - (double)raw_max);
        if (s.y_max > -INFINITY && s.proc_tail > 0.0) {
            z_rest += s.proc_tail * exp((double)temper(s.y_max, apply_t, p.temperature) - (double)x_max);
        }
    }
    // With a top-k, what reaches the largest part threshold is still several times k (every part
    // handed on its own k).  One histogram over the values from that threshold to the row's
    // maximum, 256 equal bins, finds a bin edge with at least k values above it: only those go on
    // the list, usually k and a handful, and the exact k-th value is found among them later.
    // (Any map from value to bin that never decreases as the value falls would do.)
    const bool narrow = top_k_on && total > p.top_k;
    const float x_low = temper(keep_from, apply_t, p.temperature);
    const uint32_t low_key = ordered_key(x_low);
    float bin_scale = 0.0f;  // 0: one bin, nothing is cut here
    if (narrow && x_max - x_low > 0.0f && x_max - x_low < INFINITY) bin_scale = __fdiv_rn(255.0f, x_max - x_low);
    auto bin_of = [&](uint32_t key) {
        return (uint32_t)max(0, min(255, (int)__fmul_rn(__fsub_rn(x_max, from_ordered_key(key)), bin_scale)));
    };
    if (narrow) {
        for (int i = tid; i < total; i += kMergeThreads) {
            const float l = __uint_as_float(cand_l[i]);
            const uint32_t cf = cand_c[i];
            z_raw += exp((double)l - (double)raw_max);
            const float y = processed_before_temperature(l, cf, p.penalty);
            const uint32_t key = ordered_key(temper(y, apply_t, p.temperature));
            const bool listed = y > -INFINITY && key >= low_key;
            xkeys[i] = listed ? key : 0u;  // 0 is below every key of a number
            if (listed) atomicAdd(&s_hist[bin_of(key)], 1u);
        }
        hist_clean = false;
        z_raw = warp_sum(z_raw);
        if (lane == 0) s_d[0][warp] = z_raw;
        __syncthreads();
        z_raw = 0.0;
#pragma unroll
        for (int w = 0; w < kMergeThreads / 32; ++w) z_raw += s_d[0][w];
        // lane L owns bins 8L .. 8L+7, the highest values first; where does the count reach k?
        const uint4 a4 = reinterpret_cast<const uint4*>(s_hist)[2 * lane], b4 = reinterpret_cast<const uint4*>(s_hist)[2 * lane + 1];
        const uint32_t bins[8] = {a4.x, a4.y, a4.z, a4.w, b4.x, b4.y, b4.z, b4.w};
        uint32_t local = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) local += bins[q];
        uint32_t incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += up;
        }
        const uint32_t need = (uint32_t)p.top_k, excl = incl - local;
        const bool here = excl < need && need <= incl;
        int my_bin = 8 * lane;
        if (here) {
            uint32_t above = excl;
#pragma unroll
            for (int q = 0; q < 7; ++q) {
                if (my_bin == 8 * lane + q && above + bins[q] < need) { above += bins[q]; ++my_bin; }
            }
        }
        const int src = __ffs(__ballot_sync(0xFFFFFFFFu, here)) - 1;
        const uint32_t cut_bin = src < 0 ? 255u : (uint32_t)__shfl_sync(0xFFFFFFFFu, my_bin, src);  // fewer than k: all stay
        for (int i = tid; i < total; i += kMergeThreads) {
            const uint32_t key = xkeys[i];
            if (key != 0u && bin_of(key) <= cut_bin) {
                const int slot = atomicAdd(&s_count, 1);
                if (slot < cap) keyA[slot] = ((u64)key << 32) | (uint32_t)~(cand_c[i] & kColumnMask);
            }
        }
        __syncthreads();
    } else {
        // (a warp takes its places on the list with one addition: without a top-k thousands are listed,
        // and one addition each would queue at the counter)
        for (int base = 0; base < total; base += kMergeThreads) {
            const int i = base + tid;
            bool listed = false;
            float y = 0.0f;
            uint32_t cf = 0;
            if (i < total) {
                const float l = __uint_as_float(cand_l[i]);
                cf = cand_c[i];
                z_raw += exp((double)l - (double)raw_max);
                y = processed_before_temperature(l, cf, p.penalty);
                listed = y >= keep_from;
            }
            const uint32_t takers = __ballot_sync(0xFFFFFFFFu, listed);
            int first_slot = 0;
            if (takers != 0 && lane == 0) first_slot = atomicAdd(&s_count, __popc(takers));
            first_slot = __shfl_sync(0xFFFFFFFFu, first_slot, 0);
            if (listed) {
                const float x = temper(y, apply_t, p.temperature);
                const int slot = first_slot + __popc(takers & ((1u << lane) - 1u));
                if (slot < cap) keyA[slot] = ((u64)ordered_key(x) << 32) | (uint32_t)~(cf & kColumnMask);
            } else if (i < total && y > -INFINITY && !top_k_on) {
                z_rest += exp((double)temper(y, apply_t, p.temperature) - (double)x_max);
                dropped += 1.0;
            }
        }
        // three sums, one barrier (which also makes s_count final); fixed order
        z_raw = warp_sum(z_raw);
        z_rest = warp_sum(z_rest);
        dropped = warp_sum(dropped);
        if (lane == 0) { s_d[0][warp] = z_raw; s_d[1][warp] = z_rest; s_d[2][warp] = dropped; }
        __syncthreads();
        z_raw = 0.0; z_rest = 0.0; dropped = 0.0;
#pragma unroll
        for (int w = 0; w < kMergeThreads / 32; ++w) {
            z_raw += s_d[0][w];
            z_rest += s_d[1][w];
            dropped += s_d[2][w];
        }
    }
    PSX_MERGE_STAGE(5);
    int n = s_count;
    if (top_k_on && total > p.top_k && n > cap) {
        // Too many reach the largest part threshold for the list.  Every part handed on at least
        // k logits, so together they hold the k that a top-k keeps: the k-th largest of everything
        // collected IS the row's k-th largest.  Select it; only it and what ties with it after the
        // temperature divide go on the list.
        for (int i = tid; i < total; i += kMergeThreads) {
            ykeys[i] = ordered_key(processed_before_temperature(__uint_as_float(cand_l[i]), cand_c[i], p.penalty));
        }
        if (!hist_clean) {
            for (int i = tid; i < 4 * 256; i += kMergeThreads) s_hist[i] = 0;
        }
        if (tid == 0) s_count = 0;
        __syncthreads();
        const uint32_t kth = block_select_kth([&](int i) { return ykeys[i]; }, total, (uint32_t)p.top_k, s_hist);
        hist_clean = false;
        keep_from = fmaxf(keep_from, relax_threshold(from_ordered_key(kth), apply_t, p.temperature));
        __syncthreads();  // ykeys lies over the list that is written next
        for (int i = tid; i < total; i += kMergeThreads) {
            const uint32_t cf = cand_c[i];
            const float y = processed_before_temperature(__uint_as_float(cand_l[i]), cf, p.penalty);
            if (y >= keep_from) {
                const int slot = atomicAdd(&s_count, 1);
                if (slot < cap) {
                    keyA[slot] = ((u64)ordered_key(temper(y, apply_t, p.temperature)) << 32) | (uint32_t)~(cf & kColumnMask);
                }
            }
        }
        __syncthreads();
        n = s_count;
    }
    if (n > cap || n == 0) {
        if (tid == 0) {
            p.tokens[row] = -1;
            p.log_probs[row] = 0.0f;
            p.row_status[row] = n == 0 ? PSX_ROW_ALL_REMOVED : PSX_ROW_TOO_WIDE;
            if (p.diag) p.diag[row] = psx_row_diag{n, 0, INFINITY, INFINITY};
        }
        return;
    }

    constexpr int kCountDirectly = 64;  // up to here the one-entry-per-thread path finds the k-th value by counting
    if (top_k_on && n > kCountDirectly && n > p.top_k) {
        // A top-k over a longer list: the k-th largest value by radix selection, then only it, its
        // ties and what lies above stay (src/generation.cpp:80-87).
        if (!hist_clean) {
            for (int i = tid; i < 4 * 256; i += kMergeThreads) s_hist[i] = 0;
        }
        if (tid == 0) s_ns = 0;
        __syncthreads();
        const uint32_t kth = block_select_kth([&](int i) { return key_ord(keyA[i]); }, n, (uint32_t)p.top_k, s_hist);
        u64* kept = reinterpret_cast<u64*>(ex);
        for (int i = tid; i < n; i += kMergeThreads) {
            const u64 key = keyA[i];
            if (key_ord(key) >= kth) kept[atomicAdd(&s_ns, 1)] = key;
        }
        __syncthreads();
        n = s_ns;
        for (int i = tid; i < n; i += kMergeThreads) keyA[i] = kept[i];
        __syncthreads();
    }
    PSX_MERGE_STAGE(6);
    // ---- 3'. a long list without a top-k: decided by the whole block, without sorting --------------
    bool decided = false;
    if (p.do_sample && !top_k_on && n > kMergeThreads) {
        // the largest value key, and the bits in which the value keys differ: one barrier for the three
        uint32_t top_key = 0, in_all = ~0u, in_any = 0u;
        for (int i = tid; i < n; i += kMergeThreads) {
            const uint32_t k = key_ord(keyA[i]);
            top_key = max(top_key, k);
            in_all &= k;
            in_any |= k;
        }
        top_key = __reduce_max_sync(0xFFFFFFFFu, top_key);
        in_all = __reduce_and_sync(0xFFFFFFFFu, in_all);
        in_any = __reduce_or_sync(0xFFFFFFFFu, in_any);
        if (lane == 0) { s_u[0][warp] = top_key; s_u[1][warp] = in_all; s_u[2][warp] = in_any; }
        __syncthreads();
#pragma unroll
        for (int w = 0; w < kMergeThreads / 32; ++w) {
            top_key = max(top_key, s_u[0][w]);
            in_all &= s_u[1][w];
            in_any |= s_u[2][w];
        }
        const float x_top = from_ordered_key(top_key);
        // (the histograms lie over the second sort array, idle on this path)
        const bool room = cap * 8 >= kWideWords * 4;
        if (room) {
            for (int i = tid; i < kMassPasses * 768 / 4; i += kMergeThreads) reinterpret_cast<uint4*>(keyB)[i] = make_uint4(0, 0, 0, 0);
        }
        double list_sum = 0.0;
        for (int i = tid; i < n; i += kMergeThreads) {
            const double e = exp((double)from_ordered_key(key_ord(keyA[i])) - (double)x_top);  // src/generation.cpp:46
            ex[i] = e;
            alive[i] = 1;
            list_sum += e;
        }
        list_sum = block_sum_fixed(list_sum, s_d[0]);  // its barriers publish the arrays too
        const bool rest_in_play = (alive_tail + dropped) > 0.0;
        const double bound = exp((double)temper(keep_from, apply_t, p.temperature) - (double)x_top);
        Decision wide;
        decided = room && decide_wide(p, keyA, ex, alive, n, rest_in_play, z_rest, bound, u_row, s_d[0],
                                      reinterpret_cast<uint32_t*>(keyB), top_key, in_all ^ in_any, list_sum, wide);
        __syncthreads();
        if (decided && tid == 0) {
            s_dec = wide;
            s_chosen_raw = 0;
        }
    }

    if (!decided && n <= kMergeThreads) {
        // ---- 3''. a short list (the usual case): one entry per thread, nothing sorted ---------------
        SmallScratch w;  // over the second sort array and the exp array, both idle on this path
        w.order_b = reinterpret_cast<uint32_t*>(keyB);
        w.cols = w.order_b + kMergeThreads;
        w.shared = w.cols + kMergeThreads;             // 8 words
        w.pr = reinterpret_cast<double*>(w.shared + 8);
        w.ex = ex;
        w.alive = alive;
        w.sum = &s_d[0][0];
        if (tid < 8) w.shared[tid] = 1;
        __syncthreads();
        decide_small(p, keyA, n, top_k_on, (alive_tail + dropped) > 0.0, z_rest,
                     temper(keep_from, apply_t, p.temperature),
                     u_row, w, &s_dec);
        if (tid == 0) s_chosen_raw = 0;
        decided = true;
    }

    if (!decided) {
    // ---- 3. sort by (value desc, column asc); top-k keeps the k-th value and its ties -----------
    {
        int n_pad = 2;
        while (n_pad < n) n_pad <<= 1;
        for (int i = n + tid; i < n_pad; i += kMergeThreads) keyA[i] = 0;
        __syncthreads();
        block_bitonic_sort(keyA, n_pad, /*descending=*/true);
    }

    if (tid == 0) s_ns = 0;
    __syncthreads();
    bool rest_alive = false;
    if (top_k_on && n >= p.top_k) {
        const uint32_t kth = key_ord(keyA[p.top_k - 1]);
        int count = 0;
        for (int i = tid; i < n; i += kMergeThreads) count += key_ord(keyA[i]) >= kth ? 1 : 0;
        if (count) atomicAdd(&s_ns, count);
    } else {
        if (tid == 0) s_ns = n;
        // Without a top-k the rest of the vocabulary is still in play.
        rest_alive = !top_k_on && p.do_sample && (alive_tail + dropped) > 0.0;
    }
    __syncthreads();
    const int ns = s_ns;
    const float x_first = from_ordered_key(key_ord(keyA[0]));
    const double rest_bound = exp((double)temper(keep_from, apply_t, p.temperature) - (double)x_first);
    for (int i = tid; i < n; i += kMergeThreads) {
        if (i >= ns) { alive[i] = 0; continue; }
        const float x = from_ordered_key(key_ord(keyA[i]));
        ex[i] = exp((double)x - (double)x_first);  // src/generation.cpp:46
        alive[i] = 1;
        keyB[i] = ((u64)key_col(keyA[i]) << 32) | (uint32_t)i;
    }
    if (ns <= kMergeThreads) {
        block_rank_sort(keyB, ns, /*descending=*/false);
    } else {
        int ns_pad = 2;
        while (ns_pad < ns) ns_pad <<= 1;
        for (int i = ns + tid; i < ns_pad; i += kMergeThreads) keyB[i] = ~0ull;
        __syncthreads();
        block_bitonic_sort(keyB, ns_pad, /*descending=*/false);
    }

    // ---- 4. the reference's walk, by one thread ------------------------------------------------------
    if (tid == 0) {
        decide(p, keyA, keyB, ex, alive, ns, rest_alive, z_rest, rest_bound, u_row, s_dec);
        s_chosen_raw = 0;
    }
    }  // !decided
    __syncthreads();
    PSX_MERGE_STAGE(7);
    Decision dec = s_dec;
    if (p.survivor_cols != nullptr && dec.status == PSX_ROW_OK) {  // hand the surviving set itself out
        if (tid == 0) s_count = 0;
        __syncthreads();
        for (int i = tid; i < n; i += kMergeThreads) {
            if (!alive[i]) continue;
            const int slot = atomicAdd(&s_count, 1);
            if (slot < p.survivor_cap) {
                p.survivor_cols[row * p.survivor_cap + slot] = key_col(keyA[i]);
                p.survivor_vals[row * p.survivor_cap + slot] = from_ordered_key(key_ord(keyA[i]));
            }
        }
        __syncthreads();
        if (s_count > p.survivor_cap) dec.status = PSX_ROW_TOO_WIDE;
        if (tid == 0) p.survivor_counts[row] = (uint32_t)min(s_count, p.survivor_cap);
    }
    PSX_MERGE_STAGE(8);
    if (dec.status == PSX_ROW_OK) {
        if (overlay) {  // the chosen column's raw logit, from the logits themselves
            if (tid == 0) s_chosen_raw = __float_as_uint(p.logits[row * p.logits_row_stride + (dec.token - p.logits_col_begin)]);
        } else {        // it sits among the candidates
            for (int i = tid; i < total; i += kMergeThreads) {
                if ((long long)(cand_c[i] & kColumnMask) == dec.token) s_chosen_raw = cand_l[i];
            }
        }
    }
    __syncthreads();
    if (tid == 0) {
        p.row_status[row] = dec.status;
        p.tokens[row] = dec.status == PSX_ROW_OK ? dec.token : -1;
        float lp = 0.0f;
        if (dec.status == PSX_ROW_OK) {
            const double l = (double)__uint_as_float(s_chosen_raw);
            lp = (float)log(exp(l - (double)raw_max) / z_raw);  // src/generation.cpp:156
        }
        p.log_probs[row] = lp;
        if (p.diag) p.diag[row] = psx_row_diag{n, dec.survivors, dec.draw_margin, dec.top_p_margin};
    }
    PSX_MERGE_STAGE(9);
}


}  // namespace survivor
}  // namespace psx
