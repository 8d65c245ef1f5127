// The survivor stage with one WARP per row, for the plans whose lists are short: greedy, and sampling
// under a top-k of at most 64.  The same decisions as merge_row (merge_rows_impl.cuh), made the same
// way -- places in the reference's three orders by counting, the sums and walks whose order the
// reference fixes by one lane running down a contiguous array (src/generation.cpp:80-152) -- but
// without a block's barriers and without seven more warps issuing the same bookkeeping: eight rows
// share a CTA, a few KB of shared memory each.  A row that does not fit (more entries at or above the
// threshold than the warp's list holds, a part whose list overflowed) is left marked kRowUndecided
// for the block-per-row kernel that follows.
#pragma once

#include "merge_rows_impl.cuh"

namespace psx {
namespace survivor {

constexpr int kRowsPerCta = kMergeThreads / 32;
constexpr int kWarpEntries = 4;  // list entries a lane owns at most (list capacity 128)

// Shared memory of one warp's row: the list (keys, raw logit bits), the arrays of decide_small.
__host__ __device__ inline size_t warp_arena_bytes(int cap) {
    return ((size_t)cap * (8 + 8 + 8 + 4 + 4 + 4 + 1) + 8 * 4 + 8 + 15) & ~(size_t)15;
}

constexpr float kWarpLog2e = 1.4426950408889634f;

template <int N>
__device__ __forceinline__ void warp_merge_row(const MergeParams& p, const int64_t row, unsigned char* arena) {
    const int lane = threadIdx.x & 31;
    const uint32_t lanes_below = (1u << lane) - 1u;
    const int cap = p.warp_list_cap;
    u64* keyA = reinterpret_cast<u64*>(arena);
    double* ex = reinterpret_cast<double*>(keyA + cap);
    double* pr = ex + cap;
    double* sum = pr + cap;
    uint32_t* raw = reinterpret_cast<uint32_t*>(sum + 1);
    uint32_t* cols = raw + cap;
    uint32_t* order_b = cols + cap;
    uint32_t* shared = order_b + cap;  // 8 broadcast words
    uint8_t* alive_of = reinterpret_cast<uint8_t*>(shared + 8);

    const bool sample = p.do_sample != 0, apply_t = p.apply_temperature != 0;
    const bool top_k_on = sample && p.top_k > 0 && p.top_k < p.vocab;  // src/generation.cpp:80
    const char* stats_row = static_cast<const char*>(p.stats) + row * p.stats_row_stride;
    const char* counts_row = static_cast<const char*>(p.part_counts) + row * p.count_row_stride;
    const char* cands_row = static_cast<const char*>(p.candidates) + row * p.cand_row_stride;
    auto count_of_part = [&](int part) {
        return min(*reinterpret_cast<const uint32_t*>(counts_row + part * p.count_part_stride), (uint32_t)p.part_cap);
    };
    auto list_of_part = [&](int part) { return reinterpret_cast<const uint2*>(cands_row + part * p.cand_part_stride); };

    // ---- 1. the first 2^shift slots of every part's list, fetched together with the counts -------------
    const int shift = p.warp_slot_shift, slots_per_part = 1 << shift, slots = p.parts << shift;
    uint2 fetched[N];
    uint32_t count_of[N];
#pragma unroll
    for (int q = 0; q < N; ++q) {
        const int i = q * 32 + lane;
        count_of[q] = 0;
        fetched[q] = make_uint2(0, 0);
        if (i < slots) {
            const int part = i >> shift;
            count_of[q] = count_of_part(part);
            fetched[q] = list_of_part(part)[i & (slots_per_part - 1)];
        }
    }
    const double u_row = (sample && p.uniforms) ? p.uniforms[row] : 0.5;

    // ---- the parts' records -------------------------------------------------------------------------------
    float raw_max = -FLT_MAX, y_max = -INFINITY, thr = -INFINITY;
    uint32_t bad = 0, total = 0;
    bool longer = false;  // a list that goes on beyond the fetched slots
    for (int i = lane; i < p.parts; i += 32) {
        const PartStats s = *reinterpret_cast<const PartStats*>(stats_row + i * p.stats_part_stride);
        raw_max = fmaxf(raw_max, s.raw_max);
        y_max = fmaxf(y_max, s.y_max);
        thr = fmaxf(thr, s.thr);
        bad |= (s.nonfinite & 3u) | (s.overflow ? 4u : 0u);
        const uint32_t c = count_of_part(i);
        total += c;
        longer |= c > (uint32_t)slots_per_part;
    }
    raw_max = warp_max(raw_max);
    y_max = warp_max(y_max);
    thr = warp_max(thr);
    bad = __reduce_or_sync(0xFFFFFFFFu, bad);
    total = __reduce_add_sync(0xFFFFFFFFu, total);
    longer = __any_sync(0xFFFFFFFFu, longer);
    if ((bad & 3u) != 0) {  // as merge_row: a time-out first, then a non-finite logit
        if (lane == 0) {
            p.tokens[row] = -1;
            p.log_probs[row] = 0.0f;
            p.row_status[row] = (bad & 2u) ? PSX_ROW_DEVICE_TIMEOUT : PSX_ROW_NON_FINITE;
            if (p.diag) p.diag[row] = psx_row_diag{(int)total, 0, INFINITY, INFINITY};
        }
        return;
    }
    if ((bad & 4u) != 0) {  // an overflowed list: the block kernel reports it or decides from the row itself
        if (lane == 0) p.row_status[row] = kRowUndecided;
        return;
    }

    // ---- 2. raw sum-exp over everything; the list of those that can survive ---------------------------------
    float keep_from = sample ? relax_threshold(thr, apply_t, p.temperature) : fmaxf(y_max, -FLT_MAX);
    double z_raw = 0.0;
    for (int i = lane; i < p.parts; i += 32) {
        const PartStats s = *reinterpret_cast<const PartStats*>(stats_row + i * p.stats_part_stride);
        z_raw += s.raw_tail * exp((double)s.raw_max - (double)raw_max);
    }
    // A candidate below the threshold belongs to the tail like the logits the row pass left behind, and its
    // exponential is taken the same way: ex2 in float against the rounded exponent of the maximum, the
    // rounding put back once for the whole sum.  What may be drawn gets its exponential in double.
    const float c_l2 = __fmul_rn(raw_max, kWarpLog2e);
    const float c_res = __fmaf_rn(raw_max, kWarpLog2e, -c_l2);
    float tail = 0.0f;
    int n = 0;
    // The processed value of every fetched candidate, once (a penalised one costs a divide).
    float y_of[N];
#pragma unroll
    for (int q = 0; q < N; ++q) {
        const uint32_t slot = (uint32_t)(q * 32 + lane) & (uint32_t)(slots_per_part - 1);
        y_of[q] = slot < count_of[q] ? processed_before_temperature(__uint_as_float(fetched[q].x), fetched[q].y, p.penalty) : -INFINITY;
    }
    // With a top-k, what reaches the largest part threshold is still several times k (every part handed on
    // its own k).  One 32-bin histogram over the values from that threshold up to the row's maximum finds
    // the bin in which the count reaches k; what falls into later bins is below k candidates and leaves.
    // A candidate is listed by the bin of its value RAISED by what the temperature divide can merge (twice
    // relax_threshold's margin): one that is not listed then lies below the relaxed value of k counted
    // candidates, so its quotient is strictly below theirs and it is no tie of the k-th
    // (src/generation.cpp:80-87).  Candidates beyond the fetched slots are not counted, which can only move
    // the cut to a later bin.
    int cut = 32;  // 32: nothing is cut here
    float bin_scale = 0.0f;
    auto bin_of = [&](float v) { return min(31, max(0, (int)__fmul_rn(__fsub_rn(y_max, v), bin_scale))); };
    auto raised = [&](float y) {
        return apply_t ? __fadd_rn(y, __fmaf_rn(fabsf(y), 0x1p-20f, __fmul_rn(p.temperature, 0x1p-146f))) : y;
    };
    if (top_k_on && (long long)total > p.top_k && y_max - keep_from > 0.0f && y_max - keep_from < INFINITY) {
        bin_scale = __fdiv_rn(31.5f, y_max - keep_from);
        uint32_t* hist = order_b;  // (idle until the places are known)
        hist[lane] = 0;
        __syncwarp();
#pragma unroll
        for (int q = 0; q < N; ++q) {
            if (y_of[q] >= keep_from) atomicAdd(&hist[bin_of(y_of[q])], 1u);  // (an empty slot holds -inf)
        }
        __syncwarp();
        uint32_t incl = hist[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += up;
        }
        const uint32_t reached = __ballot_sync(0xFFFFFFFFu, (long long)incl >= p.top_k);
        cut = reached != 0 ? __ffs(reached) - 1 : 31;
        __syncwarp();
    }
    auto consume = [&](bool valid, uint32_t l_bits, uint32_t cf, float y) {  // by the whole warp; appends in lane order
        const float l = __uint_as_float(l_bits);
        const bool listed = valid && y >= keep_from && (cut >= 32 || bin_of(raised(y)) <= cut);
        if (valid && !listed) tail += ex2_approx(__fmaf_rn(l, kWarpLog2e, -c_l2));
        const uint32_t voters = __ballot_sync(0xFFFFFFFFu, listed);
        if (listed) {
            const int at = n + __popc(voters & lanes_below);
            if (at < cap) {  // (the value still before the temperature: the divide waits until the list is complete)
                keyA[at] = ((u64)__float_as_uint(y) << 32) | (uint32_t)~(cf & kColumnMask);
                raw[at] = l_bits;
            }
        }
        n += __popc(voters);
    };
#pragma unroll
    for (int q = 0; q < N; ++q) {
        const uint32_t slot = (uint32_t)(q * 32 + lane) & (uint32_t)(slots_per_part - 1);
        consume(slot < count_of[q], fetched[q].x, fetched[q].y, y_of[q]);
    }
    if (longer) {  // the rest of the long lists, part after part
        for (int part = 0; part < p.parts; ++part) {
            const uint32_t count = count_of_part(part);
            for (uint32_t i0 = (uint32_t)slots_per_part; i0 < count; i0 += 32) {
                const uint32_t i = i0 + lane;
                const uint2 c = i < count ? list_of_part(part)[i] : make_uint2(0, 0);
                consume(i < count, c.x, c.y, processed_before_temperature(__uint_as_float(c.x), c.y, p.penalty));
            }
        }
    }
    if (n > cap) {
        if (lane == 0) p.row_status[row] = kRowUndecided;
        return;
    }
    __syncwarp();
    // What is listed may be drawn: its exponential in double and its temperature divide, one entry per lane
    // and round.
    for (int e = lane; e < n; e += 32) {
        z_raw += exp((double)__uint_as_float(raw[e]) - (double)raw_max);
        const u64 k = keyA[e];
        keyA[e] = ((u64)ordered_key(temper(__uint_as_float((uint32_t)(k >> 32)), apply_t, p.temperature)) << 32) | (uint32_t)k;
    }
    z_raw += (double)tail * exp2_of_minus_small(c_res);
    z_raw = warp_sum(z_raw);
    if (n == 0) {
        if (lane == 0) {
            p.tokens[row] = -1;
            p.log_probs[row] = 0.0f;
            p.row_status[row] = PSX_ROW_ALL_REMOVED;
            if (p.diag) p.diag[row] = psx_row_diag{0, 0, INFINITY, INFINITY};
        }
        return;
    }
    __syncwarp();

    // ---- 3. the decisions on the list (decide_small, with up to four entries per lane) ----------------------
    u64 mine[kWarpEntries];
    uint32_t counts[kWarpEntries], lower[kWarpEntries];
#pragma unroll
    for (int j = 0; j < kWarpEntries; ++j) {
        const int e = lane + 32 * j;
        mine[j] = e < n ? keyA[e] : 0;
        counts[j] = 0;
        lower[j] = 0;
    }
    // Among all n: how many come before mine by (value desc, column asc), how many of those share my value,
    // how many share it at all, how many sit at lower columns.
    const int rounds = (n + 31) >> 5;  // entries per lane that exist at all (warp-uniform)
    for (int o = 0; o < n; ++o) {
        const u64 other = keyA[o];
#pragma unroll
        for (int j = 0; j < kWarpEntries; ++j) {
            if (j >= rounds) break;
            const uint32_t before = other > mine[j] ? 1u : 0u, same = key_ord(other) == key_ord(mine[j]) ? 1u : 0u;
            counts[j] += before + ((before & same) << 10) + (same << 20);
            lower[j] += key_col(other) < key_col(mine[j]) ? 1u : 0u;
        }
    }
    const bool cut_k = top_k_on && n >= p.top_k;
    if (lane == 0 && !cut_k) shared[2] = 0;
#pragma unroll
    for (int j = 0; j < kWarpEntries; ++j) {
        const int e = lane + 32 * j;
        if (e < n) {
            const int place = (int)(counts[j] & 1023u);
            if (place == 0) { shared[0] = key_ord(mine[j]); shared[1] = (uint32_t)e; }  // the first maximum
            if (cut_k && place == (int)p.top_k - 1) shared[2] = key_ord(mine[j]);       // the k-th value
            cols[place] = key_col(mine[j]);
        }
    }
    __syncwarp();
    const uint32_t top_ord = shared[0], best = shared[1], kth = shared[2];
    bool survivor[kWarpEntries], alive[kWarpEntries];
    int ns = 0;
#pragma unroll
    for (int j = 0; j < kWarpEntries; ++j) {
        survivor[j] = lane + 32 * j < n && key_ord(mine[j]) >= kth;  // src/generation.cpp:85: ties at the k-th value stay
        ns += __popc(__ballot_sync(0xFFFFFFFFu, survivor[j]));
    }
    int place_b[kWarpEntries], place_w[kWarpEntries];
    double my_ex[kWarpEntries];
#pragma unroll
    for (int j = 0; j < kWarpEntries; ++j) {
        place_b[j] = 0; place_w[j] = 0; my_ex[j] = 0.0;
        alive[j] = survivor[j];
        if (survivor[j]) {
            const int place = (int)(counts[j] & 1023u), same_before = (int)((counts[j] >> 10) & 1023u), same = (int)(counts[j] >> 20);
            int b = (int)lower[j];
            for (int t = ns; t < n; ++t) b -= cols[t] < key_col(mine[j]) ? 1 : 0;
            place_b[j] = b;
            place_w[j] = ns - (place - same_before) - same + same_before;
            my_ex[j] = exp((double)from_ordered_key(key_ord(mine[j])) - (double)from_ordered_key(top_ord));  // src/generation.cpp:46
            order_b[b] = (uint32_t)(lane + 32 * j);
            ex[b] = my_ex[j];
            if (lane + 32 * j == (int)best) shared[5] = (uint32_t)b;
        }
    }
    Decision d;
    d.status = PSX_ROW_OK;
    d.token = -1;
    d.survivors = 0;
    d.draw_margin = INFINITY;
    d.top_p_margin = INFINITY;
    int chosen_entry = (int)best;
    __syncwarp();

    if (sample && p.top_p < 1.0f) {  // src/generation.cpp:89-103 (nothing outside the list is in play under a top-k)
        if (lane == 0) *sum = ordered_sum(ex, ns, 0.0);  // column order, as the reference sums
        __syncwarp();
        const double total_ex = *sum;
#pragma unroll
        for (int j = 0; j < kWarpEntries; ++j) {
            if (survivor[j]) pr[place_w[j]] = my_ex[j] / total_ex;
        }
        __syncwarp();
        if (lane == 0) {
            const double limit = 1.0 - (double)p.top_p;
            const WalkEnd end = ordered_walk<false>(pr, ns - 1, 0.0, limit);  // the last of the walk always stays
            const int cut = end.index;
            if (cut > 0) d.top_p_margin = fabs(end.before - limit);
            if (cut < ns - 1) d.top_p_margin = fmin(d.top_p_margin, fabs(end.upto - limit));
            shared[4] = (uint32_t)cut;
        }
        __syncwarp();
        const int cut = (int)shared[4];
#pragma unroll
        for (int j = 0; j < kWarpEntries; ++j) alive[j] = survivor[j] && place_w[j] >= cut;
    }

    if (sample && p.min_p > 0.0f) {  // src/generation.cpp:104-111 (rare: left to one lane)
#pragma unroll
        for (int j = 0; j < kWarpEntries; ++j) {
            if (lane + 32 * j < n) alive_of[lane + 32 * j] = alive[j] ? 1 : 0;
        }
        __syncwarp();
        if (lane == 0) {
            double s = 0.0;
            for (int t = 0; t < ns; ++t) {
                if (alive_of[order_b[t]]) s += ex[t];
            }
            const double floor_p = p.min_p * (ex[shared[5]] / s);
            for (int t = 0; t < ns; ++t) {
                const uint32_t o = order_b[t];
                if (alive_of[o] && o != best && ex[t] / s < floor_p) alive_of[o] = 0;
            }
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < kWarpEntries; ++j) alive[j] = lane + 32 * j < n && alive_of[lane + 32 * j] != 0;
    }

    if (sample) {  // src/generation.cpp:140-152
        int alive_count = 0;
        __syncwarp();
#pragma unroll
        for (int j = 0; j < kWarpEntries; ++j) {
            if (survivor[j]) ex[place_b[j]] = alive[j] ? my_ex[j] : 0.0;  // adding 0.0 leaves the sum as skipping does
            alive_count += __popc(__ballot_sync(0xFFFFFFFFu, alive[j]));
        }
        __syncwarp();
        if (lane == 0) *sum = ordered_sum(ex, ns, 0.0);
        __syncwarp();
        const double total_ex = *sum;
#pragma unroll
        for (int j = 0; j < kWarpEntries; ++j) {
            if (survivor[j]) pr[place_b[j]] = alive[j] ? my_ex[j] / total_ex : 0.0;
        }
        __syncwarp();
        d.survivors = alive_count;
        if (lane == 0) {
            // The first place whose running sum exceeds u; a probability of zero (removed, or
            // underflowed) leaves the sum where it was and is never the first.  If u is not
            // below the last sum either, the last place with a probability is drawn.
            const WalkEnd end = ordered_walk<true>(pr, ns, 0.0, u_row);
            const int chosen = end.index < ns ? end.index : end.last;
            if (end.index < ns) {
                const double lo = fabs(u_row - end.before), hi = fabs(u_row - end.upto);
                d.draw_margin = end.before == 0.0 ? hi : fmin(lo, hi);
            } else {
                d.draw_margin = fabs(u_row - end.upto);
            }
            chosen_entry = chosen >= 0 ? (int)order_b[chosen] : (int)best;
        }
    } else {
        d.survivors = ns;  // src/generation.cpp:135: the first maximum, lower column wins
    }

    // ---- 4. the row's results -----------------------------------------------------------------------------------
    if (lane == 0) {
        const long long token = key_col(keyA[chosen_entry]);
        const double l = (double)__uint_as_float(raw[chosen_entry]);
        p.row_status[row] = PSX_ROW_OK;
        p.tokens[row] = token;
        p.log_probs[row] = (float)log(exp(l - (double)raw_max) / z_raw);  // src/generation.cpp:156
        if (p.diag) p.diag[row] = psx_row_diag{n, d.survivors, d.draw_margin, d.top_p_margin};
    }
}

}  // namespace survivor
}  // namespace psx
