// general_row: one row of src/generation.cpp:55-156 decided from the row itself, by one CTA.
//
// The survivor stage normally works on the few candidates the row pass hands on.  Some rows do not
// fit that scheme: sampling with no filter at all (every token survives), a top-p or min-p whose
// kept set is wider than the candidate lists, a top-k beyond what a part can bound, thousands of
// exact ties at a cut.  The reference answers all of them, so this path does too: the CTA walks
// the whole row again (it has just been read, so mostly out of L2), a dozen or so times, and
// replays the reference with block-wide primitives --
//   - processed logits on the fly (a bitmap of the history in shared memory; penalty, EOS ban and
//     temperature with the reference's float operations);
//   - top-k: the k-th largest key by radix selection, ties kept (:80-88);
//   - top-p: the cut of the ascending (value, index) walk by a radix descent over mass histograms;
//     ties at the cut value go in index order (:89-103);
//   - min-p against the first maximum (:104-111);
//   - the inverse-CDF walk in index order by a radix descent over the index (:140-152);
//   - the unprocessed log-softmax of the chosen token (:133,156).
// Sums over the vocabulary are made of fixed-point terms (2^-44), so they do not depend on the
// order of the additions: the same input gives the same bits.  They differ from the reference's
// sequential double sums by at most about vocab * 3e-14; a decision closer than that to its
// boundary may differ from the reference's, and the distances are reported per row (draw_margin,
// top_p_margin) so that a caller can tell.  Slow (a hundred microseconds or so per row) and rare.
#pragma once

#include "merge_rows_impl.cuh"

namespace psx {
namespace survivor {

__device__ __forceinline__ u64 block_max_u64(u64 v, double* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const u64 other = __shfl_xor_sync(0xFFFFFFFFu, v, o);
        v = other > v ? other : v;
    }
    __syncthreads();
    u64* slots = reinterpret_cast<u64*>(scratch);
    if ((threadIdx.x & 31) == 0) slots[threadIdx.x >> 5] = v;
    __syncthreads();
    u64 r = 0;
#pragma unroll
    for (int w = 0; w < kMergeThreads / 32; ++w) r = slots[w] > r ? slots[w] : r;
    __syncthreads();
    return r;
}

// Block-wide sum of 64-bit integers (the same in every thread, whatever the order).
__device__ __forceinline__ u64 block_sum_u64(u64 v, double* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    __syncthreads();
    u64* slots = reinterpret_cast<u64*>(scratch);
    if ((threadIdx.x & 31) == 0) slots[threadIdx.x >> 5] = v;
    __syncthreads();
    u64 r = 0;
#pragma unroll
    for (int w = 0; w < kMergeThreads / 32; ++w) r += slots[w];
    __syncthreads();
    return r;
}
// ... of masses in [0, 1] given as fixed-point integers of 2^-44 (up to 2^19 of them fit).
__device__ __forceinline__ double block_mass_sum(u64 units, double* scratch) {
    return (double)block_sum_u64(units, scratch) / kMassUnit;
}

// mass_select for a whole row: the same radix descent, with one 64-bit bin per digit (a bin may
// collect hundreds of thousands of masses).  hist: (top_shift / 8 + 1) * 256 64-bit words, zero on entry.
template <class KeyOf, class InPlay, class MassOf>
__device__ inline void row_mass_select(KeyOf key_of, InPlay in_play, MassOf mass_of, int n, int top_shift, double target,
                                       u64* hist, uint32_t& K, double& below, double& at) {
    const int tid = threadIdx.x, lane = tid & 31;
    uint32_t prefix = 0, mask = 0;
    const double room = target * kMassUnit;
    const u64 target_units = room <= 0.0 ? 0ull : room >= 1.8e19 ? ~0ull : (u64)room;
    u64 carried = 0, at_units = 0;  // units below the current prefix; units of the digit chosen last
#pragma unroll 1
    for (int shift = top_shift; shift >= 0; shift -= 8) {
        u64* h = hist + 256 * (shift >> 3);
        for (int i = tid; i < n; i += kMergeThreads) {
            if (!in_play(i)) continue;
            const uint32_t key = key_of(i);
            if ((key & mask) != prefix) continue;
            atomicAdd(reinterpret_cast<unsigned long long*>(h + ((key >> shift) & 255u)),
                      (unsigned long long)__double2ull_rn(mass_of(i) * kMassUnit));
        }
        __syncthreads();
        u64 run[8];  // lane L owns bins 8L .. 8L+7, ascending
        u64 local = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            local += h[8 * lane + q];
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
            if (before_mine + run[q] > target_units) first = q;
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
        } else {  // never above the target: the largest key in play
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
    below = (double)carried / kMassUnit;
    at = (double)at_units / kMassUnit;
}

// (MergeParams by value: the copy is made where the call is, not on entry to the kernel.)
__device__ __noinline__ void general_row(const MergeParams p, const int64_t row, u64* dyn) {
    __shared__ double s_scratch[kMergeThreads / 32];
    const int tid = threadIdx.x;
    const int V = (int)p.vocab;
    const float* x = p.logits + row * p.logits_row_stride;
    const bool sample = p.do_sample != 0, apply_t = p.apply_temperature != 0;
    const bool top_k_on = sample && p.top_k > 0 && p.top_k < p.vocab;
    const bool penalise = p.history_ids != nullptr && p.penalty != 1.0f;
    const bool use_flags = penalise || p.num_banned > 0;
    const bool process = p.process_out != nullptr;

    // shared memory: the history bitmap, then the histograms of one selection at a time (1024 counters
    // of 32 bits, or 4 x 256 masses of 64)
    const int words = ((V + 31) / 32 + 3) & ~3;
    uint32_t* bits = reinterpret_cast<uint32_t*>(dyn);
    uint32_t* hist = bits + words;
    constexpr int kHistWords = 4 * 256 * 2;
    auto give_up = [&](int status) {
        if (tid == 0) {
            p.row_status[row] = status;
            if (!process) {
                p.tokens[row] = -1;
                p.log_probs[row] = 0.0f;
            }
            if (p.diag) p.diag[row] = psx_row_diag{V, 0, INFINITY, INFINITY};
        }
    };
    if ((size_t)(words + kHistWords) * 4 > (size_t)p.dyn_bytes || p.logits_col_begin != 0) {
        give_up(PSX_ROW_TOO_WIDE);  // a vocabulary whose bitmap does not fit beside the histograms
        return;
    }
    auto clear_hist = [&]() {
        __syncthreads();
        for (int i = tid; i < kHistWords; i += kMergeThreads) hist[i] = 0;
        __syncthreads();
    };
    if (use_flags) {
        for (int i = tid; i < words; i += kMergeThreads) bits[i] = 0;
        __syncthreads();
        if (penalise) {
            for (int64_t i = p.history_offsets[row] + tid; i < p.history_offsets[row + 1]; i += kMergeThreads) {
                const int64_t id = p.history_ids[i];
                if (id >= 0 && id < p.vocab) atomicOr(&bits[id >> 5], 1u << (id & 31));  // src/generation.cpp:62
            }
        }
        for (int i = tid; i < p.num_banned; i += kMergeThreads) {
            const int64_t id = p.banned_ids[i];
            if (id >= 0 && id < p.vocab) atomicOr(&bits[id >> 5], 1u << (id & 31));
        }
        __syncthreads();
    }
    // the processed logit of column i (src/generation.cpp:59-79)
    auto processed = [&](int i) {
        float y = x[i];
        if (use_flags && ((bits[i >> 5] >> (i & 31)) & 1u)) {
            bool banned = false;
            for (int b = 0; b < p.num_banned; ++b) banned |= p.banned_ids[b] == (int64_t)i;
            y = banned ? -INFINITY : penalize(y, p.penalty);
        }
        return sample ? temper(y, apply_t, p.temperature) : y;
    };
    auto key_of = [&](int i) { return ordered_key(processed(i)); };

    // ---- the maxima: raw, and processed with the lowest column among equals (:135); finite check (:128-132) ----
    float raw_max = -FLT_MAX;
    bool finite = true;
    u64 best = 0;  // (key << 32) | ~column: the largest is the first maximum
    for (int i = tid; i < V; i += kMergeThreads) {
        const float l = x[i];
        finite = finite && (fabsf(l) < INFINITY);
        raw_max = fmaxf(raw_max, l);
        const u64 k = ((u64)key_of(i) << 32) | (uint32_t)~(uint32_t)i;
        best = k > best ? k : best;
    }
    best = block_max_u64(best, s_scratch);
    raw_max = from_ordered_key(block_max_u32(ordered_key(raw_max), s_scratch));
    const bool all_finite = __syncthreads_and(finite ? 1 : 0) != 0;
    if (!all_finite && !process) {  // (like the reference's ProcessLogits, process mode does not look)
        give_up(PSX_ROW_NON_FINITE);
        return;
    }
    const uint32_t top_key = (uint32_t)(best >> 32);
    const int best_col = (int)~(uint32_t)best;
    const float x_top = from_ordered_key(top_key);
    if (!(x_top > -INFINITY)) {  // every token was removed (:136-138)
        if (process) {
            float* out = p.process_out + row * p.logits_row_stride;
            for (int i = tid; i < V; i += kMergeThreads) out[i] = -INFINITY;
            if (tid == 0) p.row_status[row] = kRowDoneInPlace;
        } else {
            give_up(PSX_ROW_ALL_REMOVED);
        }
        return;
    }
    auto ex_of = [&](int i) { return exp((double)processed(i) - (double)x_top); };  // (:46; -inf gives 0)
    auto units_of = [&](double mass) { return (u64)__double2ull_rn(mass * kMassUnit); };

    // ---- top-k: the k-th largest of the processed row, ties kept (:80-88) ----
    uint32_t kth_key = 0;
    if (top_k_on) {
        clear_hist();
        kth_key = block_select_kth(key_of, V, (uint32_t)p.top_k, hist);
        __syncthreads();
    }
    // ---- top-p: the ascending walk's cut (:89-103) ----
    uint32_t cut_key = 0;   // keys below it are removed
    int tie_cut = -1;       // columns of the cut key up to this one are removed as well
    double top_p_margin = INFINITY, draw_margin = INFINITY;
    if (sample && p.top_p < 1.0f) {
        const double limit = 1.0 - (double)p.top_p;
        u64 units = 0;
        for (int i = tid; i < V; i += kMergeThreads) {
            if (key_of(i) >= kth_key) units += units_of(ex_of(i));
        }
        const double sum = block_mass_sum(units, s_scratch);
        clear_hist();
        double mass_below, mass_at;
        row_mass_select(key_of, [&](int i) { return key_of(i) >= kth_key && processed(i) > -INFINITY; }, ex_of, V, 24,
                        limit * sum, reinterpret_cast<u64*>(hist), cut_key, mass_below, mass_at);
        __syncthreads();
        const double below = mass_below / sum;
        top_p_margin = fabs(below - limit);
        // Entries equal to the cut value go in ascending column order, one probability each.
        int ties = 0;
        for (int i = tid; i < V; i += kMergeThreads) ties += key_of(i) == cut_key ? 1 : 0;
        const int group = (int)block_sum_u64((u64)ties, s_scratch);
        const double each = exp((double)from_ordered_key(cut_key) - (double)x_top) / sum;
        double cumulative = below;
        int removed = 0;
        for (int j = 0; j < group; ++j) {
            cumulative += each;
            top_p_margin = fmin(top_p_margin, fabs(cumulative - limit));
            if (cumulative <= limit) ++removed; else break;
        }
        if (cut_key == top_key && removed >= group) removed = group - 1;  // the last of the walk always stays
        if (removed >= group) {
            tie_cut = V;
        } else if (removed > 0) {  // the `removed` lowest columns among the ties: select by column
            clear_hist();
            const uint32_t pick = block_select_kth(
                [&](int i) { return key_of(i) == cut_key ? 0x7FFFFFFFu - (uint32_t)i : 0u; }, V, (uint32_t)removed, hist);
            __syncthreads();
            tie_cut = (int)(0x7FFFFFFFu - pick);
        }
    }
    auto alive_p = [&](int i) {
        const uint32_t k = key_of(i);
        if (k < kth_key || !(processed(i) > -INFINITY)) return false;
        if (sample && p.top_p < 1.0f) return k > cut_key || (k == cut_key && i > tie_cut);
        return true;
    };
    // ---- min-p against the first maximum (:104-111) ----
    double min_p_sum = 0.0;
    const bool min_p_on = sample && p.min_p > 0.0f;
    if (min_p_on) {
        u64 units = 0;
        for (int i = tid; i < V; i += kMergeThreads) {
            if (alive_p(i)) units += units_of(ex_of(i));
        }
        min_p_sum = block_mass_sum(units, s_scratch);
    }
    auto alive = [&](int i) {
        if (!alive_p(i)) return false;
        if (!min_p_on || i == best_col) return true;
        return !(ex_of(i) / min_p_sum < (double)p.min_p * (1.0 / min_p_sum));  // the maximum has exp(0) = 1
    };

    if (process) {  // ProcessLogits: the row as the filters leave it, in place
        float* out = p.process_out + row * p.logits_row_stride;
        for (int i = tid; i < V; i += kMergeThreads) {
            const float value = alive(i) ? processed(i) : -INFINITY;  // (reads column i before it writes it)
            out[i] = value;
        }
        if (tid == 0) p.row_status[row] = kRowDoneInPlace;
        return;
    }

    // ---- the draw (:140-152), or the first maximum ----
    int chosen = best_col, survivors = 1;
    if (sample) {
        u64 units = 0;
        int count = 0;
        for (int i = tid; i < V; i += kMergeThreads) {
            if (alive(i)) {
                units += units_of(ex_of(i));
                ++count;
            }
        }
        const double sum = block_mass_sum(units, s_scratch);
        survivors = (int)block_sum_u64((u64)count, s_scratch);
        const double u = p.uniforms[row];
        clear_hist();
        uint32_t hit;
        double mass_before, mass_at;
        const int column_shift = V <= (1 << 16) ? 8 : V <= (1 << 24) ? 16 : 24;
        row_mass_select([&](int i) { return (uint32_t)i; }, [&](int i) { return alive(i) && ex_of(i) / sum != 0.0; }, ex_of, V,
                        column_shift, u * sum, reinterpret_cast<u64*>(hist), hit, mass_before, mass_at);
        __syncthreads();
        const double before = mass_before / sum, upto = (mass_before + mass_at) / sum;
        draw_margin = before == 0.0 ? fabs(u - upto) : fmin(fabs(u - before), fabs(u - upto));
        chosen = (int)hit;
    }
    // ---- the chosen token's log-probability under the unprocessed logits (:133,156) ----
    double z = 0.0;
    {
        u64 units = 0;
        for (int i = tid; i < V; i += kMergeThreads) units += units_of(exp((double)x[i] - (double)raw_max));
        z = block_mass_sum(units, s_scratch);
    }
    if (tid == 0) {
        p.row_status[row] = PSX_ROW_OK;
        p.tokens[row] = chosen;
        p.log_probs[row] = (float)log(exp((double)x[chosen] - (double)raw_max) / z);
        if (p.diag) p.diag[row] = psx_row_diag{V, survivors, draw_margin, top_p_margin};
    }
}

}  // namespace survivor
}  // namespace psx
