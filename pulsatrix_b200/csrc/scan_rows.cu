// The row pass: the one kernel that reads the logits from HBM.
//
// Each CTA owns one "part" of one row: up to 4096 aligned float4 vectors (16384 logits, 64 KB).
// One thread asks the TMA unit for the whole part with four bulk asynchronous copies of 16 KB
// (cp.async.bulk global -> shared, each completing on an mbarrier of its own; no multicast), so the
// bytes stream from HBM into shared memory without passing through registers while the other
// threads turn the row's token history into a bitmap; a warp starts on a quarter of the part as
// soon as that quarter has landed.  Everything after that reads shared memory:
//   1. the few logits the history (repetition penalty, src/generation.cpp:59-68) or the EOS ban
//      (:69-73) names are handed on as candidates whatever their value, in a fixed order, and
//      blanked in shared memory, so the dense passes below never look at a flag;
//   2. pass one takes per-thread maxima; the smallest over the warps of the kp-th largest
//      per-thread maximum is a threshold that at least k_need logits of the part reach, found
//      without sorting the data;
//   3. pass two sums exp(l - max) over everything below the threshold (the unprocessed
//      log-softmax of src/generation.cpp:133,156 needs it) and hands on every logit at or above
//      it (raw value, column, flags), warp by warp in a fixed order, so the survivor stage is
//      reproducible bit for bit.
// Selection works on the logits BEFORE the temperature divide: dividing by a positive number is
// monotonic, so the k-th largest commutes with it, and the threshold is relaxed by the few ulps
// the divide can merge (relax_threshold).
//
// HBM bound: 4 bytes per logit, read once; what is written is a few hundred bytes per part.
#include "psx_async.cuh"
#include "scan_rows.cuh"

namespace psx {

namespace {

constexpr float kLog2e = 1.4426950408889634f;
// log2(e) = kLog2e * (1 + kLog2eRel): the part of log2(e) that the float constant drops.
constexpr float kLog2eRel = (float)(1.4426950408889634073599246810019 / (double)1.4426950408889634f - 1.0);
constexpr float kPad = -FLT_MAX;  // stands for "no logit here": finite, never above a real logit
constexpr int kBitmapWords = kPartVecs * 4 / 32;  // one bit per logit of a part
constexpr uint32_t kCopyChunk = 16384;            // bytes per bulk copy; every copy completes on a barrier of its own
constexpr int kCopies = kPartVecs * 16 / kCopyChunk;

// acc = max(acc, all four) in two three-input instructions.
__device__ __forceinline__ float max_into(float acc, const float4& v) { return fmax3(fmax3(v.x, v.y, v.z), v.w, acc); }
__device__ __forceinline__ float amax_into(float acc, const float4& v) {
    return fmax3(fmax3(fabsf(v.x), fabsf(v.y), fabsf(v.z)), fabsf(v.w), acc);
}

// Sets, in a bitmap with one bit per logit of this part, the columns that `ids` names (and the
// same bits in `also`, when given).  Every bit that was not set before adds one to the count of
// the warp that owns its word in the dense passes, so each warp's number of flagged logits is
// known without anybody looking at the bitmap again.
__device__ __forceinline__ void mark_ids(const int64_t* ids, int64_t begin, int64_t end, const ScanParams& p,
                                         int first_pos, int part_logits, uint32_t* bitmap, uint32_t* also,
                                         uint32_t* warp_counts) {
    // first_pos: position of this part's first slot in the row's aligned window, minus the
    // row's misalignment, i.e. the (possibly negative) local column of data[0].  The ids this part
    // cares about are one interval: its slots, cut to this GPU's columns [0, cols).  Those lie inside
    // the vocabulary (src/generation.cpp:62 ignores ids outside it), so one unsigned comparison
    // of the distance from the interval's first id decides.
    const int lo = max(first_pos, 0);
    const int64_t hi = min((int64_t)first_pos + part_logits, p.cols);
    const int64_t first_id = p.col_begin + lo;
    const uint64_t span = hi > lo ? (uint64_t)(hi - lo) : 0u;
    const uint32_t shift = (uint32_t)(lo - first_pos);
    for (int64_t i = begin + threadIdx.x; i < end; i += kScanThreads) {
        const uint64_t rel = (uint64_t)ids[i] - (uint64_t)first_id;  // wraps for ids before the interval
        if (rel < span) {
            const uint32_t e = (uint32_t)rel + shift;  // slot in this part
            const uint32_t word = e >> 5, bit = 1u << (e & 31);
            if (!(atomicOr(&bitmap[word], bit) & bit)) atomicAdd(&warp_counts[(word >> 2) & (kScanWarps - 1)], 1u);
            if (also) atomicOr(&also[word], bit);
        }
    }
}

constexpr int kPool = 64 / kScanWarps;  // per-thread maxima a warp can offer to the pooled threshold (64 in all)

}  // namespace

// Profiling build only (-DPSX_STAGE_CLOCKS): thread 0 of each CTA stamps the SM clock at the stage
// boundaries; the stamps of the first 4096 CTAs are kept for psx_debug_stage_clocks to read back.
#ifdef PSX_STAGE_CLOCKS
__device__ unsigned long long g_stage_clocks[4096 * 16];
#define STAGE(i) do { if (threadIdx.x == 0) clk[i] = clock64(); } while (0)
#else
#define STAGE(i) do {} while (0)
#endif

template <bool kNucleus>
__global__ void __launch_bounds__(kScanThreads, 3) scan_rows_kernel(const ScanParams p) {
#ifdef PSX_STAGE_CLOCKS
    unsigned long long clk[16];
    for (int i = 0; i < 16; ++i) clk[i] = 0;
    unsigned long long gt0; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt0));
    STAGE(0);
#endif
    extern __shared__ __align__(128) unsigned char dyn_smem[];
    float* data = reinterpret_cast<float*>(dyn_smem);
    const float4* data4 = reinterpret_cast<const float4*>(dyn_smem);

    __shared__ __align__(8) uint64_t s_bar[kCopies];
    __shared__ __align__(16) uint32_t s_bits[2 * kBitmapWords];
    uint32_t* const s_flag = s_bits;                 // penalised or banned
    uint32_t* const s_ban = s_bits + kBitmapWords;   // banned
    __shared__ float s_wraw[kScanWarps], s_wamax[kScanWarps], s_wymax[kScanWarps], s_wthr[kScanWarps];
    __shared__ uint32_t s_pool[kScanWarps * kPool];
    __shared__ double s_wtail[kScanWarps], s_wproc[kScanWarps];
    __shared__ uint32_t s_wfill[kScanWarps], s_wflag[kScanWarps];

    const int part = blockIdx.x;  // grid: (parts, rows in chunks of 65535, chunks)
    const int64_t row = (int64_t)blockIdx.z * 65535 + blockIdx.y;
    if (row >= p.rows) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t part_index = (size_t)row * p.parts + part;

    // ---- geometry: the row as aligned float4 vectors ------------------------------------------
    const float* row_ptr = p.logits + row * p.row_stride;
    const uint32_t misalign = (uint32_t)((reinterpret_cast<uintptr_t>(row_ptr) >> 2) & 3);
    const float4* vbase = reinterpret_cast<const float4*>(row_ptr - misalign);
    const int nv = (int)((misalign + p.cols + 3) >> 2);
    const int v0 = part * p.vecs_per_part;
    const int v1 = min(v0 + p.vecs_per_part, nv);
    const int nvec = v1 - v0;
    // The survivor stage that follows may be set up while this kernel runs.  This kernel reads only
    // its caller's inputs until it has something to hand on: when the caller has promised that they
    // are complete, it runs ahead of the kernel before it in the stream until its first write.
    grid_dependents_may_launch();
    if (!p.inputs_ready) grid_dependency_wait();
    if (nvec <= 0) {  // a part past the end of a row that starts on a 16-byte boundary: nothing to report
        grid_dependency_wait();
        if (tid == 0) {
            p.part_counts[part_index] = 0;
            PartStats s;
            s.raw_tail = 0.0; s.proc_tail = 0.0; s.raw_max = kPad; s.y_max = -INFINITY; s.thr = -INFINITY;
            s.nonfinite = 0; s.alive_tail = 0; s.overflow = 0;
            p.stats[part_index] = s;
        }
        return;
    }

    // ---- start the copy, and build the history bitmaps while it is in flight ----------------------
    if (tid == 0) {
        for (int i = 0; i < kCopies; ++i) barrier_init(&s_bar[i], 1);
        barrier_init_fence();
    }
    if (tid < kScanWarps) s_wflag[tid] = 0;
    static_assert(2 * kBitmapWords % 4 == 0, "the bitmaps are cleared 16 bytes at a time");
    for (int i = tid; i < 2 * kBitmapWords / 4; i += kScanThreads) reinterpret_cast<uint4*>(s_bits)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    STAGE(1);
    if (tid == 0) {
        const uint32_t bytes = (uint32_t)nvec * 16u;
        const char* src = reinterpret_cast<const char*>(vbase + v0);
        for (uint32_t off = 0, i = 0; off < bytes; off += kCopyChunk, ++i) {
            const uint32_t piece = min(kCopyChunk, bytes - off);
            // (test hook: announcing more bytes than the copy delivers leaves the barrier open with
            // nothing in flight, which is how the bounded wait is exercised)
            barrier_expect_bytes(&s_bar[i], piece + (p.test_short_copy ? 16u : 0u));
            bulk_copy_to_shared(dyn_smem + off, src + off, piece, &s_bar[i]);
        }
    }
    const bool use_flags = p.apply_penalty || p.num_banned > 0;
    const int first_pos = v0 * 4 - (int)misalign;
    if (p.apply_penalty) {
        mark_ids(p.history_ids, p.history_offsets[row], p.history_offsets[row + 1], p, first_pos, nvec * 4, s_flag, nullptr,
                 s_wflag);
    }
    if (p.num_banned > 0) mark_ids(p.banned_ids, 0, p.num_banned, p, first_pos, nvec * 4, s_flag, s_ban, s_wflag);
    __syncthreads();  // the bitmaps are complete
    STAGE(2);
    const int copies = (nvec * 16 + (int)kCopyChunk - 1) / (int)kCopyChunk;
    const int trips = (nvec + kScanThreads - 1) / kScanThreads;  // the part is padded to whole trips
    // Pad the part to whole 256-vector trips (at most one vector per thread).  The padding lies
    // behind the copied bytes, so it need not wait for them.
    {
        // Every shared-memory write from here on is made by the thread that owns the vector in the
        // dense passes (vector v belongs to thread v % kScanThreads) or by a thread of its warp, so
        // warp-level ordering is enough and the warps run on without meeting again until the
        // threshold.
        const int v = (trips - 1) * kScanThreads + tid;
        if (v >= nvec) reinterpret_cast<float4*>(dyn_smem)[v] = make_float4(kPad, kPad, kPad, kPad);
    }
    // The part's candidates form one list: first the flagged logits, warp after warp (each warp
    // knows every warp's count from the marking above), then what reaches the threshold.
    uint2* part_out = p.candidates + part_index * kPartCap;
    uint32_t flagged_total, seg_fill;  // warp-uniform: the next free slot of this warp's run
    {
        const uint32_t v = lane < kScanWarps ? s_wflag[lane] : 0u;
        flagged_total = __reduce_add_sync(0xFFFFFFFFu, v);
        seg_fill = __reduce_add_sync(0xFFFFFFFFu, lane < warp ? v : 0u);
    }
    const int col_base = (int)((int64_t)v0 * 4 - misalign + p.col_begin);  // global column of data[0]; fits 31 bits
    float f_raw = kPad, f_amax = 0.0f, f_y = -INFINITY;
    float m = kPad, amax = 0.0f;
    bool landed = true;  // (a wait that ran out is dealt with where the block meets next)

    // The part in two halves of 32 KB (two copies, eight trips each): a warp waits for a half itself
    // -- the wait also orders the copied bytes before the warp's reads --, hands on the half's
    // flagged logits and takes its maxima while the other half is still landing.
    constexpr int kWordsPerWarp = kBitmapWords / kScanWarps;
    static_assert(kCopies == 4 && kVecPerThread == 16 && kWordsPerWarp == 64, "two halves of two copies, eight trips, 32 bitmap words per warp");
    for (int half = 0; half < 2 && 2 * half < copies; ++half) {
        for (int i = 2 * half; i < min(copies, 2 * half + 2); ++i) {
            landed = barrier_wait_bounded(&s_bar[i], 0, p.wait_limit_ns) && landed;
        }
        // From here on the kernel writes scratch that an earlier survivor stage may still be reading.
        if (half == 0) grid_dependency_wait();
        // Components of the first and last vector that lie outside the row are blanked.
        if (half == 0 && v0 == 0 && tid == 0) {
            for (uint32_t c = 0; c < misalign; ++c) data[c] = kPad;
        }
        if (2 * half + 2 >= copies && v1 == nv && tid == ((nvec - 1) & (kScanThreads - 1))) {
            for (int64_t pos = (int64_t)misalign + p.cols; pos < (int64_t)nv * 4; ++pos) data[pos - (int64_t)v0 * 4] = kPad;
        }
        __syncwarp();
        STAGE(3);

        // ---- 1. flagged logits: handed on in bitmap order, then blanked -------------------------------
        if (use_flags) {
            // A warp takes the bitmap words of the logits its own threads own in the dense passes
            // (vector v belongs to thread v % kScanThreads), so a row that is handed on whole fills every
            // warp's segment with exactly its own 128 logits.  Lane L: trip 8 * half + L / 4, quarter L % 4.
            const int idx = half * 32 + lane;
            const int word = (kScanThreads / 8) * (idx >> 2) + 4 * warp + (idx & 3);
            const uint32_t banned_bits = s_ban[word];
            uint32_t bits = s_flag[word];
            const uint32_t count = __popc(bits);
            const uint32_t voters = __ballot_sync(0xFFFFFFFFu, count != 0);
            if (voters != 0) {
                // Slots in lane order.  Usually a lane flags one logit; otherwise scan the counts.
                uint32_t slot = seg_fill + __popc(voters & ((1u << lane) - 1u));
                uint32_t total = __popc(voters);
                if (__ballot_sync(0xFFFFFFFFu, count > 1) != 0) {
                    uint32_t incl = count;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                        if (lane >= o) incl += up;
                    }
                    slot = seg_fill + incl - count;
                    total = __shfl_sync(0xFFFFFFFFu, incl, 31);
                }
                seg_fill += total;
                while (bits) {
                    const int b = __ffs(bits) - 1;
                    bits &= bits - 1;
                    const uint32_t e = (uint32_t)word * 32u + (uint32_t)b;
                    const float l = data[e];
                    const bool banned = (banned_bits >> b) & 1u;
                    const float y = banned ? -INFINITY : penalize(l, p.penalty);
                    f_raw = fmaxf(f_raw, l);
                    f_amax = (l != l) ? INFINITY : fmaxf(f_amax, fabsf(l));
                    f_y = fmaxf(f_y, y);
                    if (slot < (uint32_t)kPartCap) {
                        part_out[slot] = make_uint2(__float_as_uint(l),
                                                   (uint32_t)(col_base + (int)e) | (banned ? kFlagBanned : kFlagPenalized));
                    }
                    ++slot;
                    data[e] = kPad;
                }
            }
            __syncwarp();
        }
        STAGE(4);

        // ---- 2. per-thread maxima (the part's raw max and selection threshold follow) ------------------
        const int t_end = min(trips, 8 * half + 8);
#pragma unroll 4
        for (int t = 8 * half; t < t_end; ++t) {
            const float4 d = data4[t * kScanThreads + tid];
            m = max_into(m, d);
            amax = amax_into(amax, d);
        }
    }
    amax = fmaxf(amax, f_amax);
    STAGE(5);
    const float m_alive = (m == kPad) ? -INFINITY : m;  // a thread without logits takes no part in the selection
    const int live_threads = min(kScanThreads, nvec);
    const int full_warps = live_threads >> 5;  // warps whose every thread owns a vector
    int kp = 33;  // > 32: no threshold, hand everything on
    if (full_warps == kScanWarps) kp = (p.k_need + kScanWarps - 1) / kScanWarps;  // the usual case: a shift
    else if (full_warps > 0) kp = (p.k_need + full_warps - 1) / full_warps;
    // Threshold: a value that at least k_need logits of the part reach (or everything, when the
    // part has fewer).  Greedy needs the part's maximum only.  Otherwise every full warp finds
    // its kp-th largest per-thread maximum, kp = ceil(k_need / full warps), and the smallest of
    // those is reached by kp maxima in every full warp.  When that would overshoot k_need by
    // only a few, the warps pool their kp largest instead and the overshoot is taken away from
    // the bottom of the pool, which gives exactly k_need.
    const bool single = p.k_need == 1;
    const bool pooled = !single && kp <= kPool && full_warps * kp - p.k_need <= 4;
    {
        const float wraw = warp_max_redux(fmaxf(m, f_raw)), wamax = warp_max_redux(amax);
        const float wymax = warp_max_redux(fmaxf(m_alive, f_y));
        float wthr = -INFINITY;
        if (single) {
            wthr = warp_max_redux(m_alive);
        } else if (pooled) {
            uint32_t offer = 0xFFFFFFFFu;  // lane i ends up with the warp's i-th largest; all ones: no entry
            if (warp < full_warps) {
                uint32_t key = monotone_key(m_alive);
                for (int i = 0; i < kp; ++i) {
                    const uint32_t top = __reduce_max_sync(0xFFFFFFFFu, key);
                    if (lane == i) offer = top;
                    const uint32_t holders = __ballot_sync(0xFFFFFFFFu, key == top);
                    if (lane == __ffs(holders) - 1) key = 0;
                }
            }
            if (lane < kPool) s_pool[warp * kPool + lane] = offer;
        } else if (kp <= 8) {
            wthr = warp_kth_largest_small(m_alive, kp, lane);
        } else if (kp <= 32) {
            wthr = warp_kth_largest(m_alive, kp, lane);
        }
        if (lane == 0) {
            s_wraw[warp] = wraw;
            s_wamax[warp] = wamax;
            s_wymax[warp] = wymax;
            s_wthr[warp] = wthr;
        }
    }
    if (__syncthreads_or(landed ? 0 : 1) != 0) {
        // A copy did not complete in time: report it, give the copies one more bounded chance to
        // drain (shared memory must not be handed to the next CTA under a copy in flight), and leave.
        if (tid == 0) {
            p.part_counts[part_index] = 0;
            PartStats s;
            s.raw_tail = 0.0; s.proc_tail = 0.0; s.raw_max = kPad; s.y_max = -INFINITY; s.thr = -INFINITY;
            s.nonfinite = 2; s.alive_tail = 0; s.overflow = 0;
            p.stats[part_index] = s;
        }
        if (warp == 0) {
            for (int i = 0; i < copies; ++i) barrier_wait_bounded(&s_bar[i], 0, p.wait_limit_ns);
        }
        return;
    }
    STAGE(6);

    // ---- every warp joins the warps' results and works out the part's constants for itself --------------
    const float cmax = warp_max_redux(lane < kScanWarps ? s_wraw[lane] : kPad);
    const float camax = warp_max_redux(lane < kScanWarps ? s_wamax[lane] : 0.0f);
    const float cymax = warp_max_redux(lane < kScanWarps ? s_wymax[lane] : -INFINITY);
    float thr = -INFINITY;
    if (single) {
        thr = warp_max_redux(lane < kScanWarps ? s_wthr[lane] : -INFINITY);
    } else if (pooled) {
        // Lane L holds pool entries L and L + 32; the smallest entries are dropped until k_need
        // are left, whose minimum is the threshold.
        static_assert(kPool * kScanWarps == 64, "two pool entries per lane");
        uint32_t a = s_pool[lane], b2 = s_pool[lane + 32];
        const int surplus = full_warps * kp - p.k_need;
        for (int i = 0; i < surplus; ++i) {
            const uint32_t mine = min(a, b2);
            const uint32_t low = __reduce_min_sync(0xFFFFFFFFu, mine);
            const uint32_t holders = __ballot_sync(0xFFFFFFFFu, mine == low);
            if (lane == __ffs(holders) - 1) {
                if (a == low) a = 0xFFFFFFFFu; else b2 = 0xFFFFFFFFu;
            }
        }
        thr = from_ordered_key(__reduce_min_sync(0xFFFFFFFFu, min(a, b2)));
    } else if (full_warps > 0 && kp <= 32) {
        const uint32_t key = lane < full_warps ? monotone_key(s_wthr[lane]) : 0xFFFFFFFFu;
        thr = from_ordered_key(__reduce_min_sync(0xFFFFFFFFu, key));
    }
    // Blanked slots hold kPad and must never pass: the threshold stays one step above it.
    const float tprime = fmaxf(relax_threshold(thr, p.apply_temperature != 0, p.temperature), -3.4028233e38f);
    const float c_l2 = __fmul_rn(cmax, kLog2e);
    const float c_res = __fmaf_rn(cmax, kLog2e, -c_l2);  // cmax*kLog2e = c_l2 + c_res exactly
    const float pc_l2 = __fmul_rn(cymax, p.log2e_over_t);
    const float pc_res = __fmaf_rn(cymax, p.log2e_over_t, -pc_l2);
    STAGE(7);

    // ---- 3. exp-sum of what stays behind, hand-off of what reaches the threshold -------------------------
    const bool second_exp = kNucleus && p.apply_temperature != 0;
    // Per-lane float sums of at most 16 four-element sums each; they go to double in the reduction.
    float tail = 0.0f, proc = 0.0f;

    // The part was padded to whole 256-vector trips and the loop is branch-free: a vector that
    // reaches the threshold (rare) is only noted, one bit per trip, and its sums are left out; after
    // the loop its components below the threshold are summed again and what reaches it is counted.
    uint32_t noted = 0;
    auto exps_of = [&](const float4& d, float& e0, float& e1, float& e2, float& e3, float& q0, float& q1, float& q2,
                       float& q3) {
        float x0 = __fmaf_rn(d.x, kLog2e, -c_l2), x1 = __fmaf_rn(d.y, kLog2e, -c_l2);
        float x2 = __fmaf_rn(d.z, kLog2e, -c_l2), x3 = __fmaf_rn(d.w, kLog2e, -c_l2);
        if (kNucleus) {
            x0 = __fmaf_rn(x0, kLog2eRel, x0); x1 = __fmaf_rn(x1, kLog2eRel, x1);
            x2 = __fmaf_rn(x2, kLog2eRel, x2); x3 = __fmaf_rn(x3, kLog2eRel, x3);
        }
        e0 = ex2_approx(x0); e1 = ex2_approx(x1); e2 = ex2_approx(x2); e3 = ex2_approx(x3);
        q0 = q1 = q2 = q3 = 0.0f;
        if (second_exp) {
            float y0 = __fmaf_rn(d.x, p.log2e_over_t, -pc_l2), y1 = __fmaf_rn(d.y, p.log2e_over_t, -pc_l2);
            float y2 = __fmaf_rn(d.z, p.log2e_over_t, -pc_l2), y3 = __fmaf_rn(d.w, p.log2e_over_t, -pc_l2);
            q0 = ex2_approx(__fmaf_rn(y0, kLog2eRel, y0)); q1 = ex2_approx(__fmaf_rn(y1, kLog2eRel, y1));
            q2 = ex2_approx(__fmaf_rn(y2, kLog2eRel, y2)); q3 = ex2_approx(__fmaf_rn(y3, kLog2eRel, y3));
        }
    };
#pragma unroll 4
    for (int t = 0; t < trips; ++t) {
        const float4 d = data4[t * kScanThreads + tid];
        float e0, e1, e2, e3, q0, q1, q2, q3;
        exps_of(d, e0, e1, e2, e3, q0, q1, q2, q3);
        const bool hit = fmax3(fmax3(d.x, d.y, d.z), d.w, kPad) >= tprime;
        const float s = (e0 + e1) + (e2 + e3);
        tail += hit ? 0.0f : s;
        if (second_exp) {
            const float q = (q0 + q1) + (q2 + q3);
            proc += hit ? 0.0f : q;
        }
        noted |= hit ? (1u << t) : 0u;
    }
    STAGE(8);
    // What reaches the threshold is counted now and handed on after the block has met (below): a
    // warp's run in the part's list starts where the runs of the warps before it end.  It leaves
    // the sums (its exp is taken in double by the survivor stage); its neighbours in the vector stay.
    uint32_t count = 0, before_mine = 0, warp_count = 0;
    const bool any_noted = __ballot_sync(0xFFFFFFFFu, noted != 0) != 0;
    if (any_noted) {
        for (uint32_t m2 = noted; m2; m2 &= m2 - 1) {
            const float4 d = data4[(__ffs(m2) - 1) * kScanThreads + tid];
            float e0, e1, e2, e3, q0, q1, q2, q3;
            exps_of(d, e0, e1, e2, e3, q0, q1, q2, q3);
            const bool h0 = d.x >= tprime, h1 = d.y >= tprime, h2 = d.z >= tprime, h3 = d.w >= tprime;
            count += (h0 ? 1u : 0u) + (h1 ? 1u : 0u) + (h2 ? 1u : 0u) + (h3 ? 1u : 0u);
            tail += ((h0 ? 0.0f : e0) + (h1 ? 0.0f : e1)) + ((h2 ? 0.0f : e2) + (h3 ? 0.0f : e3));
            if (second_exp) proc += ((h0 ? 0.0f : q0) + (h1 ? 0.0f : q1)) + ((h2 ? 0.0f : q2) + (h3 ? 0.0f : q3));
        }
        // Slots in lane order.  Usually a lane hands on one logit; otherwise scan the counts.
        const uint32_t voters = __ballot_sync(0xFFFFFFFFu, count != 0);
        before_mine = __popc(voters & ((1u << lane) - 1u));
        warp_count = __popc(voters);
        if (__ballot_sync(0xFFFFFFFFu, count > 1) != 0) {
            uint32_t incl = count;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (lane >= o) incl += up;
            }
            before_mine = incl - count;
            warp_count = __shfl_sync(0xFFFFFFFFu, incl, 31);
        }
    }

    STAGE(9);
    // ---- block reduction in a fixed order, then the hand-off and the part's record -----------------------
    {
        const double wt = warp_sum((double)tail), wp = second_exp ? warp_sum((double)proc) : 0.0;
        if (lane == 0) {
            s_wtail[warp] = wt;
            s_wproc[warp] = wp;
            s_wfill[warp] = warp_count;
        }
    }
    __syncthreads();
    STAGE(10);
    if (any_noted) {  // slots in warp order, then lane, trip, component -- a fixed order
        uint32_t slot = flagged_total + before_mine;
        for (int w = 0; w < warp; ++w) slot += s_wfill[w];
        for (uint32_t m2 = noted; m2; m2 &= m2 - 1) {
            const int v = (__ffs(m2) - 1) * kScanThreads + tid;
            const float4 d = data4[v];
            const float l[4] = {d.x, d.y, d.z, d.w};
            const uint32_t col = (uint32_t)(col_base + v * 4);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (l[c] >= tprime) {
                    if (slot < (uint32_t)kPartCap) part_out[slot] = make_uint2(__float_as_uint(l[c]), col + c);
                    ++slot;
                }
            }
        }
    }
    if (tid == 0) {
        double t = 0.0, q = 0.0;
        uint32_t handed_on = flagged_total;
#pragma unroll
        for (int w = 0; w < kScanWarps; ++w) {
            t += s_wtail[w];
            q += s_wproc[w];
            handed_on += s_wfill[w];
        }
        p.part_counts[part_index] = min(handed_on, (uint32_t)kPartCap);
        const int64_t first = max((int64_t)v0 * 4 - (int64_t)misalign, (int64_t)0);
        const int64_t last = min((int64_t)v1 * 4 - (int64_t)misalign, p.cols);
        const uint32_t logits_here = (uint32_t)(last - first);
        // The exponents used c_l2 where cmax*log2(e) was meant: put the dropped part back.
        const double raw_tail = t * exp2(-(double)c_res);
        PartStats s;
        s.raw_tail = raw_tail;
        s.proc_tail = 0.0;
        if (kNucleus && cymax > -INFINITY) {
            // What stays behind is unflagged, so its processed value is l / T; without a
            // temperature the processed tail is the raw one measured against the other maximum.
            s.proc_tail = second_exp ? q * exp2(-(double)pc_res) : raw_tail * exp((double)cmax - (double)cymax);
        }
        s.raw_max = cmax;
        s.y_max = cymax;
        s.thr = thr;
        s.nonfinite = (!(camax < INFINITY) || t != t || q != q) ? 1u : 0u;
        s.alive_tail = logits_here > handed_on ? logits_here - handed_on : 0u;
        s.overflow = handed_on > (uint32_t)kPartCap ? 1u : 0u;
        p.stats[part_index] = s;
    }
#ifdef PSX_STAGE_CLOCKS
    STAGE(11);
    if (tid == 0 && part_index < 4096) {
        unsigned long long gt1; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt1));
        unsigned sm; asm volatile("mov.u32 %0, %smid;" : "=r"(sm));
        clk[12] = gt0; clk[13] = gt1; clk[14] = sm;
        for (int i = 0; i < 16; ++i) g_stage_clocks[part_index * 16 + i] = clk[i];
    }
#endif
}

#ifdef PSX_STAGE_CLOCKS
extern "C" __attribute__((visibility("default"))) int psx_debug_stage_clocks(unsigned long long* out, int n) {
    return (int)cudaMemcpyFromSymbol(out, g_stage_clocks, sizeof(unsigned long long) * n);
}
#endif

cudaError_t configure_scan_rows() {
    const cudaError_t e = allow_all_dynamic_shared(scan_rows_kernel<true>);
    if (e != cudaSuccess) return e;
    return allow_all_dynamic_shared(scan_rows_kernel<false>);
}

cudaError_t launch_scan_rows(const ScanParams& p, bool nucleus, cudaStream_t stream) {
    if (p.rows <= 0 || p.parts <= 0) return cudaSuccess;
    if (p.vecs_per_part > kPartVecs || p.rows > 65535ll * 65535ll) return cudaErrorInvalidConfiguration;
    const size_t shared = (size_t)((p.vecs_per_part + kScanThreads - 1) / kScanThreads * kScanThreads) * 16;
    const dim3 grid((unsigned)p.parts, (unsigned)(p.rows < 65535 ? p.rows : 65535), (unsigned)((p.rows + 65534) / 65535));
    return launch_overlapping(nucleus ? scan_rows_kernel<true> : scan_rows_kernel<false>, grid, dim3(kScanThreads), shared,
                              stream, p);
}

}  // namespace psx
