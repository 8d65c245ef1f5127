// How one sampling call is laid out over the two kernels: parts per row, what every part must hand
// on, the survivor stage's capacities.  One definition for every entry point that launches the
// pair (the context-based calls and the allocation-free one), so that they cannot drift apart.
#pragma once

#include <algorithm>
#include <cstdlib>

#include "../../include/psx_b200.h"
#include "merge_rows.cuh"
#include "scan_rows.cuh"

namespace psx {

struct Plan {
    int parts = 1;
    int vecs_per_part = 1;
    int k_need = 1;
    bool nucleus = false;  // sampling without a top-k: the processed tail mass is needed too
    bool apply_temperature = false;
    int sort_capacity = 1024;
    int gather_capacity = 4096;
    int slot_shift = 0;    // the survivor stage fetches 2^slot_shift slots of every part's list at once
    bool lists_cannot_bound = false;  // no candidate list can hold what may survive: rows are decided from the row itself
};

constexpr int kNucleusNeed = 160;  // logits every part hands on when no top-k bounds the survivors

// rows x cols logits on this GPU (cols == vocab unless the vocabulary is sharded).
inline Plan make_plan(const float* logits, int64_t cols, int64_t row_stride, int64_t vocab, const psx_sampling_config* c) {
    Plan plan;
    const bool aligned = (reinterpret_cast<uintptr_t>(logits) % 16 == 0) && (row_stride % 4 == 0);
    const int64_t vectors = (cols + 3 + (aligned ? 0 : 3)) / 4;  // most float4 a row can span
    static const int part_vecs = [] {  // tuning knob, read once: vectors per CTA, 256..4096
        const char* env = std::getenv("PSX_B200_PART_VECS");
        return env ? std::max(256, std::min(kPartVecs, std::atoi(env))) : kPartVecs;
    }();
    plan.parts = (int)((vectors + part_vecs - 1) / part_vecs);
    plan.vecs_per_part = (int)((vectors + plan.parts - 1) / plan.parts);
    const bool sample = c->do_sample != 0;
    const bool top_k_on = sample && c->top_k > 0 && c->top_k < vocab;
    plan.apply_temperature = sample && c->temperature != 1.0f;  // src/generation.cpp:77
    plan.nucleus = sample && !top_k_on;
    if (!sample) plan.k_need = 1;
    else if (top_k_on) plan.k_need = (int)std::min<int64_t>(c->top_k, 1 << 20);
    else plan.k_need = kNucleusNeed;
    // A row of at most 256 vectors fits a part's candidate list whole (1024 logits): hand
    // everything on, and every filter is exact whatever the settings.
    if (vectors * 4 <= kPartCap) plan.k_need = 1 << 30;
    // Sampling with no filter at all keeps every token, and a part can bound a top-k of at most one
    // logit per thread: such rows skip the row pass and are decided from the row itself.
    plan.lists_cannot_bound = vectors * 4 > kPartCap &&
                              ((plan.nucleus && !(c->top_p < 1.0f) && !(c->min_p > 0.0f)) || (top_k_on && plan.k_need > kScanThreads));
    plan.sort_capacity = plan.nucleus ? 4096 : 1024;
    plan.gather_capacity = plan.nucleus ? 8192 : 4096;
    if (!plan.nucleus && plan.k_need < kPartCap) {
        // A large k over many parts: a part whose threshold is a warp's 25th of 32 thread maxima hands
        // on about twice k, and the row's candidates no longer fit 4096 slots.
        const int64_t estimate = (int64_t)plan.parts * (2 * plan.k_need + 32) + 256;
        if (estimate > 3500) {
            plan.sort_capacity = 2048;
            plan.gather_capacity = estimate > 5600 ? 8192 : 6144;
        }
    }
    // A part usually hands on a little over k_need logits, plus the few its share of the history flags.
    const int expected = plan.k_need >= kPartCap ? kPartCap
                         : plan.k_need > 64      ? 2 * plan.k_need + 24
                                                 : plan.k_need + plan.k_need / 4 + 24;
    plan.slot_shift = merge_slot_shift(plan.parts, kPartCap, expected);
    return plan;
}

// The part of ScanParams that follows from the settings (not the pointers, not the banned ids).
inline void fill_scan_settings(ScanParams& sp, const psx_sampling_config* c, const Plan& plan) {
    sp.apply_penalty = c->repetition_penalty != 1.0f ? 1 : 0;  // src/generation.cpp:59
    sp.penalty = c->repetition_penalty;
    sp.apply_temperature = plan.apply_temperature ? 1 : 0;
    sp.temperature = c->temperature;
    const double log2e = 1.4426950408889634073599246810019;
    sp.log2e_over_t = (float)(plan.apply_temperature ? log2e / (double)c->temperature : log2e);
    sp.k_need = plan.k_need;
    sp.parts = plan.parts;
    sp.vecs_per_part = plan.vecs_per_part;
    sp.wait_limit_ns = kDefaultWaitLimitNs;
    sp.test_short_copy = 0;
    sp.wait_before_writes = 1;
    sp.num_banned = 0;
    sp.banned_ids = nullptr;
}

// The survivor stage over what a row pass with `sp` leaves behind.  `logits` (with its stride) lets a
// plan without a top-k overlay its shared-memory arrays, and lets any plan decide from the row itself
// the rows its candidate lists cannot; pass nullptr when the whole row is not on this GPU.
inline void fill_merge_params(MergeParams& mp, const ScanParams& sp, const Plan& plan, const psx_sampling_config* c,
                              int64_t rows, int64_t vocab, const double* uniforms, int64_t* tokens, float* log_probs,
                              int32_t* row_status, psx_row_diag* diag, const float* logits, int64_t row_stride) {
    mp.stats = sp.stats;
    mp.part_counts = sp.part_counts;
    mp.candidates = sp.candidates;
    mp.parts = plan.parts;
    mp.part_cap = kPartCap;
    mp.slot_shift = plan.slot_shift;
    mp.stats_part_stride = sizeof(PartStats);
    mp.stats_row_stride = mp.stats_part_stride * plan.parts;
    mp.count_part_stride = sizeof(uint32_t);
    mp.count_row_stride = mp.count_part_stride * plan.parts;
    mp.cand_part_stride = sizeof(uint2) * kPartCap;
    mp.cand_row_stride = mp.cand_part_stride * plan.parts;
    mp.rows = rows;
    mp.vocab = vocab;
    mp.do_sample = c->do_sample != 0;
    mp.apply_temperature = plan.apply_temperature ? 1 : 0;
    mp.temperature = c->temperature;
    mp.penalty = c->repetition_penalty;
    mp.top_k = c->top_k;
    mp.top_p = c->top_p;
    mp.min_p = c->min_p;
    mp.uniforms = uniforms;
    mp.tokens = tokens;
    mp.log_probs = log_probs;
    mp.row_status = row_status;
    mp.diag = diag;
    mp.sort_capacity = plan.sort_capacity;
    mp.gather_capacity = plan.gather_capacity;
    if (logits != nullptr) {
        mp.logits = logits;
        mp.logits_row_stride = row_stride;
        mp.logits_col_begin = 0;
        mp.overlay = plan.nucleus ? 1 : 0;  // the wide plan: candidates and sort arrays share their shared memory
        // what it takes to decide a row from the row itself, should the lists not do
        mp.history_ids = sp.apply_penalty ? sp.history_ids : nullptr;
        mp.history_offsets = sp.history_offsets;
        mp.banned_ids = sp.banned_ids;
        mp.num_banned = sp.num_banned;
        mp.general = plan.lists_cannot_bound ? 2 : 1;
        // Short lists straight from a row pass: one warp per row.  (The flagged logits of the history are
        // handed on whatever their value only when the penalty is below one.)
        if (!plan.nucleus) {
            const bool greedy = !mp.do_sample;
            const int flagged = (sp.apply_penalty && sp.penalty < 1.0f) ? 24 : 4;
            plan_merge_by_warp(mp, plan.k_need, greedy, greedy ? 2 : plan.k_need + plan.k_need / 2 + flagged);
        }
    }
}

}  // namespace psx
