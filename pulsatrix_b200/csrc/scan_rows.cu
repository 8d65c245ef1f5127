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
// the warp that owns its word in the dense passes (`warp_counts`, when given), so each warp's number
// of flagged logits is known without anybody looking at the bitmap again; `also_count`, when given,
// counts the bits newly set in `also`.
__device__ __forceinline__ void mark_ids(const int64_t* ids, int64_t begin, int64_t end, int64_t first_id_loaded,
                                         const ScanParams& p, int first_pos, int part_logits, uint32_t* bitmap,
                                         uint32_t* also, uint32_t* warp_counts, uint32_t* also_count) {
    // first_pos: position of this part's first slot in the row's aligned window, minus the
    // row's misalignment, i.e. the (possibly negative) local column of data[0].  The ids this part
    // cares about are one interval: its slots, cut to this GPU's columns [0, cols).  Those lie inside
    // the vocabulary (src/generation.cpp:62 ignores ids outside it), so one unsigned comparison
    // of the distance from the interval's first id decides.
    // first_id_loaded: ids[begin + threadIdx.x], read by the caller ahead of time (when there is one).
    const int lo = max(first_pos, 0);
    const int64_t hi = min((int64_t)first_pos + part_logits, p.cols);
    const int64_t first_id = p.col_begin + lo;
    const uint64_t span = hi > lo ? (uint64_t)(hi - lo) : 0u;
    const uint32_t shift = (uint32_t)(lo - first_pos);
    auto mark = [&](int64_t id) {
        const uint64_t rel = (uint64_t)id - (uint64_t)first_id;  // wraps for ids before the interval
        if (rel < span) {
            const uint32_t e = (uint32_t)rel + shift;  // slot in this part
            const uint32_t word = e >> 5, bit = 1u << (e & 31);
            const bool fresh = !(atomicOr(&bitmap[word], bit) & bit);
            if (warp_counts != nullptr && fresh) atomicAdd(&warp_counts[(word >> 2) & (kScanWarps - 1)], 1u);
            if (also != nullptr) {
                const bool fresh_also = !(atomicOr(&also[word], bit) & bit);
                if (also_count != nullptr && fresh_also) atomicAdd(also_count, 1u);
            }
        }
    };
    // A thread's ids four at a time: the three after the one in hand are asked for together, so a history
    // of a thousand ids costs one trip to memory here, not three one after another.
    int64_t id = first_id_loaded;
    if (end - begin <= kScanThreads) {  // at most the one id that the caller has already fetched
        if (begin + threadIdx.x < end) mark(id);
        return;
    }
    for (int64_t i = begin + threadIdx.x; i < end;) {
        int64_t next[3];
#pragma unroll
        for (int q = 0; q < 3; ++q) {
            const int64_t j = i + (int64_t)(q + 1) * kScanThreads;
            next[q] = j < end ? ids[j] : (int64_t)-1;  // (-1 lies before every interval)
        }
        mark(id);
#pragma unroll
        for (int q = 0; q < 3; ++q) mark(next[q]);
        i += 4 * kScanThreads;
        if (i < end) id = ids[i];
    }
}

constexpr int kPool = 64 / kScanWarps;  // per-thread maxima a warp can offer to the pooled threshold (64 in all)
constexpr uint32_t kKeyMinusInf = 0x007FFFFFu;  // monotone_key(-inf): the lowest key a threshold can have
constexpr uint32_t kKeyNone = 0xFFFFFFFFu;      // "no entry" in the pool (above every key of a number)

}  // namespace

// Profiling build only (-DPSX_STAGE_CLOCKS): thread 0 of each CTA stamps the SM clock at the stage
// boundaries; the stamps of the first 4096 CTAs are kept for psx_debug_stage_clocks to read back.
#ifdef PSX_STAGE_CLOCKS
__device__ unsigned long long g_stage_clocks[4096 * 24];
#define STAGE(i) do { if (threadIdx.x == 0) clk[i] = clock64(); } while (0)
#else
#define STAGE(i) do {} while (0)
#endif

// kNucleus: also accumulate the processed-domain tail (a top-p / min-p over the whole vocabulary).
// kRestore: how the logits that the history or the EOS ban names ("flagged") are dealt with.
//   false: every flagged logit is handed on as a candidate whatever its value, in a fixed order, and
//          blanked in shared memory, so the dense passes never look at a flag.
//   true:  flagged logits are blanked only while the maxima are taken (they must not take the places
//          of unflagged ones in the threshold) and put back before the sums; one that reaches the
//          threshold is handed on like any other logit, with its flag looked up in the bitmap.  Valid
//          when a flag can only lower a logit (penalty >= 1: l / p or l * p <= l; a ban gives -inf) and no
//          processed tail is wanted: a flagged logit whose processed value reaches the threshold then
//          reaches it raw as well, and the rest belong to the raw tail with their raw value.
// kAnnounce: raise ScanParams::row_ready when a part is written (a build of its own, so that the usual one
//   carries nothing for it).
template <bool kNucleus, bool kRestore, bool kAnnounce = false>
__global__ void __launch_bounds__(kScanThreads, 3) scan_rows_kernel(const ScanParams p) {
    static_assert(!(kNucleus && kRestore), "the processed tail needs the flagged logits out of the sums");
#ifdef PSX_STAGE_CLOCKS
    unsigned long long clk[24];
    for (int i = 0; i < 24; ++i) clk[i] = 0;
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
    __shared__ __align__(16) uint4 s_wkeys[kScanWarps];  // per warp: keys of its unflagged maximum, flagged raw maximum, flagged processed maximum
    __shared__ uint32_t s_pool[kScanWarps * kPool];
    __shared__ float s_wamax[kScanWarps];
    __shared__ double s_wtail[kScanWarps], s_wproc[kScanWarps];
    __shared__ uint32_t s_wfill[kScanWarps], s_wflag[kScanWarps], s_wban[kScanWarps];
    __shared__ uint32_t s_banned_here;

    const int part = blockIdx.x;  // grid: (parts, rows in chunks of 65535, chunks)
    const int64_t row = (int64_t)blockIdx.z * 65535 + blockIdx.y;
    // (see ScanParams::wait_before_writes: the last CTA of the grid keeps the kernel from finishing early)
    const bool ends_the_grid = !p.wait_before_writes && blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1 &&
                               blockIdx.z == gridDim.z - 1;
    if (row >= p.rows) {
        if (ends_the_grid) grid_dependency_wait();
        return;
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t part_index = (size_t)row * p.parts + part;
    auto announce_part = [&]() {  // (by the whole CTA, after its last write)
        if (kAnnounce && p.row_ready != nullptr) {
            __syncthreads();
            if (tid == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.row_ready + row) : "memory");
        }
    };

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
        if (p.wait_before_writes || ends_the_grid) grid_dependency_wait();
        if (tid == 0) {
            p.part_counts[part_index] = 0;
            PartStats s;
            s.raw_tail = 0.0; s.proc_tail = 0.0; s.raw_max = kPad; s.y_max = -INFINITY; s.thr = -INFINITY;
            s.nonfinite = 0; s.alive_tail = 0; s.overflow = 0;
            p.stats[part_index] = s;
        }
        announce_part();
        return;
    }

    // ---- start the copy at once, and build the history bitmaps while it is in flight ---------------
    const bool use_flags = p.apply_penalty || p.num_banned > 0;
    const int copies = (nvec * 16 + (int)kCopyChunk - 1) / (int)kCopyChunk;
    if (lane == 0 && warp < copies) {  // copy i is set up and issued by the first thread of warp i
        static_assert(kCopies <= kScanWarps, "one warp per copy");
        const uint32_t bytes = (uint32_t)nvec * 16u, off = (uint32_t)warp * kCopyChunk;
        const uint32_t piece = min(kCopyChunk, bytes - off);
        barrier_init(&s_bar[warp], 1);
        barrier_init_fence();
        // (test hook: announcing more bytes than the copy delivers leaves the barrier open with
        // nothing in flight, which is how the bounded wait is exercised)
        barrier_expect_bytes(&s_bar[warp], piece + (p.test_short_copy ? 16u : 0u));
        bulk_copy_to_shared(dyn_smem + off, reinterpret_cast<const char*>(vbase + v0) + off, piece, &s_bar[warp]);
    }
    // The history's bounds and every thread's first id are asked for now, ahead of the barrier below.
    int64_t h_begin = 0, h_end = 0, h_first = 0, b_first = 0;
    if (p.apply_penalty) {
        h_begin = p.history_offsets[row];
        h_end = p.history_offsets[row + 1];
        if (h_begin + tid < h_end) h_first = p.history_ids[h_begin + tid];
    }
    if (tid < p.num_banned) b_first = p.banned_ids[tid];
    if (use_flags) {
        if (tid < kScanWarps) s_wflag[tid] = 0;
        if (tid == 0) s_banned_here = 0;
        static_assert(2 * kBitmapWords % 4 == 0, "the bitmaps are cleared 16 bytes at a time");
        for (int i = tid; i < 2 * kBitmapWords / 4; i += kScanThreads) reinterpret_cast<uint4*>(s_bits)[i] = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();  // the barriers are set up (and the bitmaps empty)
    STAGE(1);
    const int first_pos = v0 * 4 - (int)misalign;
    if (use_flags) {
        if (p.apply_penalty) {
            mark_ids(p.history_ids, h_begin, h_end, h_first, p, first_pos, nvec * 4, s_flag, nullptr, kRestore ? nullptr : s_wflag,
                     nullptr);
        }
        if (p.num_banned > 0) {
            mark_ids(p.banned_ids, 0, p.num_banned, b_first, p, first_pos, nvec * 4, s_flag, s_ban, kRestore ? nullptr : s_wflag,
                     &s_banned_here);
        }
        __syncthreads();  // the bitmaps are complete
    }
    STAGE(2);
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
    uint2* part_out = p.candidates + part_index * kPartCap;
    // Without kRestore the part's candidates form one list: first the flagged logits, warp after warp
    // (each warp knows every warp's count from the marking above), then what reaches the threshold.
    uint32_t flagged_total = 0, seg_fill = 0;  // warp-uniform: the next free slot of this warp's run
    if (!kRestore && use_flags) {
        const uint32_t v = lane < kScanWarps ? s_wflag[lane] : 0u;
        flagged_total = __reduce_add_sync(0xFFFFFFFFu, v);
        seg_fill = __reduce_add_sync(0xFFFFFFFFu, lane < warp ? v : 0u);
    }
    const int col_base = (int)((int64_t)v0 * 4 - misalign + p.col_begin);  // global column of data[0]; fits 31 bits
    const float* const window = reinterpret_cast<const float*>(vbase + v0);  // the part in global memory, slot by slot
    // Of the flagged logits: the largest raw value, the largest magnitude, the largest raw value that is not banned
    // (the penalty never changes an order, so that one gives the largest penalised value).
    float f_raw = kPad, f_amax = 0.0f, f_pen = kPad;
    float m = kPad, amax = 0.0f;
    bool landed = true;  // (a wait that ran out is dealt with where the block meets next)

    // The part in two halves of 32 KB (two copies, eight trips each): a warp waits for a half itself
    // -- the wait also orders the copied bytes before the warp's reads --, deals with the half's
    // flagged logits and takes its maxima while the other half is still landing.
    constexpr int kWordsPerWarp = kBitmapWords / kScanWarps;
    static_assert(kCopies == 4 && kVecPerThread == 16 && kWordsPerWarp == 64, "two halves of two copies, eight trips, 32 bitmap words per warp");
    for (int half = 0; half < 2 && 2 * half < copies; ++half) {
        for (int i = 2 * half; i < min(copies, 2 * half + 2); ++i) {
            landed = barrier_wait_bounded(&s_bar[i], 0, p.wait_limit_ns) && landed;
        }
        STAGE(16 + half);
        // Without kRestore the kernel now writes scratch that an earlier survivor stage may still be reading.
        if (!kRestore && half == 0 && p.wait_before_writes) grid_dependency_wait();
        // Components of the first and last vector that lie outside the row are blanked.
        if (half == 0 && v0 == 0 && tid == 0) {
            for (uint32_t c = 0; c < misalign; ++c) data[c] = kPad;
        }
        if (2 * half + 2 >= copies && v1 == nv && tid == ((nvec - 1) & (kScanThreads - 1))) {
            for (int64_t pos = (int64_t)misalign + p.cols; pos < (int64_t)nv * 4; ++pos) data[pos - (int64_t)v0 * 4] = kPad;
        }
        __syncwarp();
        STAGE(3);

        // ---- 1. flagged logits -----------------------------------------------------------------------
        // A warp takes the bitmap words of the logits its own threads own in the dense passes
        // (vector v belongs to thread v % kScanThreads).  Lane L: trip 8 * half + L / 4, quarter L % 4.
        const int idx = half * 32 + lane;
        const int word = (kScanThreads / 8) * (idx >> 2) + 4 * warp + (idx & 3);
        uint32_t my_bits = 0;
        float first_raw = 0.0f;
        if (use_flags) {
            my_bits = s_flag[word];
            if (kRestore) {
                // Out of the maxima: blanked now, put back after this half's trips.  The first value of a
                // word stays in a register; a word with more (rare) reads the others again from the row.
                if (my_bits != 0) {
                    const uint32_t banned_bits = p.num_banned > 0 ? s_ban[word] : 0u;
                    first_raw = data[(uint32_t)word * 32u + (uint32_t)(__ffs(my_bits) - 1)];
                    uint32_t bits = my_bits;
                    do {
                        const int b = __ffs(bits) - 1;
                        bits &= bits - 1;
                        const uint32_t e = (uint32_t)word * 32u + (uint32_t)b;
                        const float l = data[e];
                        f_raw = fmaxf(f_raw, l);
                        f_amax = fmaxf(f_amax, fabsf(l));  // (a NaN comes back into the sums below and shows there)
                        if (!((banned_bits >> b) & 1u)) f_pen = fmaxf(f_pen, l);
                        data[e] = kPad;
                    } while (bits);
                }
            } else {
                const uint32_t banned_bits = s_ban[word];
                uint32_t bits = my_bits;
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
                        f_raw = fmaxf(f_raw, l);
                        f_amax = (l != l) ? INFINITY : fmaxf(f_amax, fabsf(l));
                        if (!banned) f_pen = fmaxf(f_pen, l);
                        if (slot < (uint32_t)kPartCap) {
                            part_out[slot] = make_uint2(__float_as_uint(l),
                                                       (uint32_t)(col_base + (int)e) | (banned ? kFlagBanned : kFlagPenalized));
                        }
                        ++slot;
                        data[e] = kPad;
                    }
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
        if (kRestore && use_flags) {
            __syncwarp();
            if (my_bits != 0) {
                data[(uint32_t)word * 32u + (uint32_t)(__ffs(my_bits) - 1)] = first_raw;
                for (uint32_t bits = my_bits & (my_bits - 1); bits; bits &= bits - 1) {
                    const uint32_t e = (uint32_t)word * 32u + (uint32_t)(__ffs(bits) - 1);
                    data[e] = window[e];
                }
            }
            __syncwarp();
        }
    }
    amax = fmaxf(amax, f_amax);
    STAGE(5);
    // Threshold: a value that at least k_need unflagged logits of the part reach (or everything, when
    // the part has fewer).  Every warp offers its kp largest per-thread maxima, kp = ceil(k_need / 8):
    // among the 8 kp offered there are k_need that are reached by k_need different threads' maxima, so
    // the block drops the smallest offers until k_need are left, and the smallest of those is the
    // threshold.  A warp takes its largest away one after the other; equal maxima go together, which can
    // only offer less, i.e. lower the threshold.  (A thread without logits offers the padding value:
    // such a part has fewer than 1024 logits and hands all of them on.)  Beyond 8 per warp a warp
    // offers its kp-th largest only, and beyond 32 there is no threshold.
    const bool single = p.k_need == 1;
    const int kp = (int)min(((int64_t)p.k_need + kScanWarps - 1) / kScanWarps, (int64_t)33);
    const bool pooled = kp <= kPool;
    {
        uint32_t key = monotone_key(m);
        const uint32_t top0 = __reduce_max_sync(0xFFFFFFFFu, key);  // the warp's unflagged maximum
        uint32_t offer = kKeyNone;
        if (pooled) {
            if (lane == 0) offer = top0;
            key = (key == top0) ? 0u : key;
            for (int i = 1; i < kp; ++i) {
                const uint32_t top = __reduce_max_sync(0xFFFFFFFFu, key);
                if (lane == i) offer = top;
                key = (key == top) ? 0u : key;
            }
        } else if (kp <= 32) {  // (the sort is a warp-wide exchange: every lane takes part)
            const float kth = warp_kth_largest(m, kp, lane);
            if (lane == 0) offer = monotone_key(kth);
        } else if (lane == 0) {
            offer = kKeyMinusInf;
        }
        // The low six bits of an offer give way to its slot number: offers become distinct (dropping the
        // smallest needs no tie-break) at the price of a threshold up to 63 steps lower.
        if (lane < kPool) s_pool[warp * kPool + lane] = offer == kKeyNone ? kKeyNone : ((offer & ~63u) | (uint32_t)(warp * kPool + lane));
        uint32_t fraw_key = 0u, fpen_key = 0u;
        if (use_flags) {
            fraw_key = __reduce_max_sync(0xFFFFFFFFu, monotone_key(f_raw));
            fpen_key = __reduce_max_sync(0xFFFFFFFFu, monotone_key(f_pen));
        }
        if (lane == 0) s_wkeys[warp] = make_uint4(top0, fraw_key, fpen_key, 0u);
    }
    if (__syncthreads_or(landed ? 0 : 1) != 0) {
        // A copy did not complete in time: report it, give the copies one more bounded chance to
        // drain (shared memory must not be handed to the next CTA under a copy in flight), and leave.
        if (p.wait_before_writes || ends_the_grid) grid_dependency_wait();
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
        announce_part();
        return;
    }
    STAGE(6);

    // ---- every warp joins the warps' results and works out the part's constants for itself --------------
    float cmax, cymax;
    uint32_t pen_key = monotone_key(kPad);  // key of the largest flagged raw logit that is not banned
    uint32_t pool_a = kKeyNone, pool_b = kKeyNone;  // lane L holds pool entries L and L + 32
    int surplus = 0;                                // offers still to be dropped, the smallest first
    auto drop_smallest_offer = [&]() {  // (offers are distinct)
        const uint32_t low = __reduce_min_sync(0xFFFFFFFFu, min(pool_a, pool_b));
        pool_a = pool_a == low ? kKeyNone : pool_a;
        pool_b = pool_b == low ? kKeyNone : pool_b;
    };
    auto threshold_of = [&](uint32_t key) {
        // (a key below -inf's stands for maxima that went with their equals; the low bits were a slot number)
        const float t = from_ordered_key(max(key & ~63u, kKeyMinusInf & ~63u));
        return (t != t || t <= kPad) ? -INFINITY : t;  // a thread without logits: everything is handed on
    };
    {
        const uint4 k4 = lane < kScanWarps ? s_wkeys[lane] : make_uint4(0u, 0u, 0u, 0u);
        const uint32_t unflagged = __reduce_max_sync(0xFFFFFFFFu, k4.x);
        uint32_t raw_key = unflagged, y_key = unflagged == monotone_key(kPad) ? kKeyMinusInf : unflagged;
        if (use_flags) {
            raw_key = max(raw_key, __reduce_max_sync(0xFFFFFFFFu, k4.y));
            pen_key = __reduce_max_sync(0xFFFFFFFFu, k4.z);
            // (its penalised value may be the part's processed maximum; only the processed tail needs that
            // before the sums, otherwise the divide waits for the part's record)
            if (kNucleus && pen_key != monotone_key(kPad)) {
                y_key = max(y_key, monotone_key(penalize(from_ordered_key(pen_key), p.penalty)));
            }
        }
        cmax = from_ordered_key(raw_key);
        cymax = from_ordered_key(y_key);
        static_assert(kPool * kScanWarps == 64, "two pool entries per lane");
        if (single) {
            pool_a = lane == 0 ? unflagged : kKeyNone;  // greedy needs the part's maximum only
        } else {
            pool_a = s_pool[lane];
            pool_b = s_pool[lane + 32];
            surplus = pooled ? kScanWarps * kp - p.k_need : 0;
        }
    }
    for (int i = 0; i < surplus; ++i) drop_smallest_offer();
    const float thr = threshold_of(__reduce_min_sync(0xFFFFFFFFu, min(pool_a, pool_b)));
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
    const float neg_c = -c_l2, neg_pc = -pc_l2;
    auto exps_of = [&](const float4& d, float& e0, float& e1, float& e2, float& e3, float& q0, float& q1, float& q2,
                       float& q3) {
        float x0, x1, x2, x3;
        fma_pair(x0, x1, d.x, d.y, kLog2e, kLog2e, neg_c, neg_c);
        fma_pair(x2, x3, d.z, d.w, kLog2e, kLog2e, neg_c, neg_c);
        if (kNucleus) {
            fma_pair(x0, x1, x0, x1, kLog2eRel, kLog2eRel, x0, x1);
            fma_pair(x2, x3, x2, x3, kLog2eRel, kLog2eRel, x2, x3);
        }
        e0 = ex2_approx(x0); e1 = ex2_approx(x1); e2 = ex2_approx(x2); e3 = ex2_approx(x3);
        q0 = q1 = q2 = q3 = 0.0f;
        if (second_exp) {
            float y0, y1, y2, y3;
            fma_pair(y0, y1, d.x, d.y, p.log2e_over_t, p.log2e_over_t, neg_pc, neg_pc);
            fma_pair(y2, y3, d.z, d.w, p.log2e_over_t, p.log2e_over_t, neg_pc, neg_pc);
            fma_pair(y0, y1, y0, y1, kLog2eRel, kLog2eRel, y0, y1);
            fma_pair(y2, y3, y2, y3, kLog2eRel, kLog2eRel, y2, y3);
            q0 = ex2_approx(y0); q1 = ex2_approx(y1); q2 = ex2_approx(y2); q3 = ex2_approx(y3);
        }
    };
    // A vector holds a logit at or above the threshold only if its four exponentials add up to at least
    // the threshold's own (less the approximation's few ulps on either side): one comparison on a sum that
    // is needed anyway.  A bound too small to be a normal number becomes zero, i.e. every vector is looked at
    // one logit at a time below.
    float e_bound;
    {
        float t0, t1, t2, t3, u0, u1, u2, u3;
        exps_of(make_float4(tprime, tprime, tprime, tprime), t0, t1, t2, t3, u0, u1, u2, u3);
        e_bound = __fmul_rn(t0, 1.0f - 0x1p-19f);
        if (!(e_bound >= 0x1p-120f)) e_bound = 0.0f;
    }
#pragma unroll 4
    for (int t = 0; t < trips; ++t) {
        const float4 d = data4[t * kScanThreads + tid];
        float e0, e1, e2, e3, q0, q1, q2, q3;
        exps_of(d, e0, e1, e2, e3, q0, q1, q2, q3);
        float s01, s23;
        add_pair(s01, s23, e0, e2, e1, e3);  // (e0 + e1), (e2 + e3)
        const float s = s01 + s23;
        const bool hit = s >= e_bound;
        tail += hit ? 0.0f : s;
        if (second_exp) {
            float q01, q23;
            add_pair(q01, q23, q0, q2, q1, q3);
            const float q = q01 + q23;
            proc += hit ? 0.0f : q;
        }
        noted |= hit ? (1u << t) : 0u;
    }
    STAGE(8);
    // What reaches the threshold is counted now and handed on after the block has met (below): a
    // warp's run in the part's list starts where the runs of the warps before it end.  It leaves
    // the sums (its exp is taken in double by the survivor stage); its neighbours in the vector stay.
    uint32_t count = 0, before_mine = 0, warp_count = 0, banned_hits = 0;
    const bool any_noted = __ballot_sync(0xFFFFFFFFu, noted != 0) != 0;
    if (any_noted) {
        for (uint32_t m2 = noted; m2; m2 &= m2 - 1) {
            const int v = (__ffs(m2) - 1) * kScanThreads + tid;
            const float4 d = data4[v];
            float e0, e1, e2, e3, q0, q1, q2, q3;
            exps_of(d, e0, e1, e2, e3, q0, q1, q2, q3);
            const bool h0 = d.x >= tprime, h1 = d.y >= tprime, h2 = d.z >= tprime, h3 = d.w >= tprime;
            count += (h0 ? 1u : 0u) + (h1 ? 1u : 0u) + (h2 ? 1u : 0u) + (h3 ? 1u : 0u);
            tail += ((h0 ? 0.0f : e0) + (h1 ? 0.0f : e1)) + ((h2 ? 0.0f : e2) + (h3 ? 0.0f : e3));
            if (second_exp) proc += ((h0 ? 0.0f : q0) + (h1 ? 0.0f : q1)) + ((h2 ? 0.0f : q2) + (h3 ? 0.0f : q3));
            if (kRestore && p.num_banned > 0) {  // banned logits that are handed on (the others are not alive)
                const uint32_t nib = (s_ban[v >> 3] >> ((v & 7) * 4)) & 15u;
                banned_hits += ((h0 ? nib : 0u) & 1u) + ((h1 ? nib >> 1 : 0u) & 1u) + ((h2 ? nib >> 2 : 0u) & 1u) + ((h3 ? nib >> 3 : 0u) & 1u);
            }
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
        const float wamax = from_ordered_key(__reduce_max_sync(0xFFFFFFFFu, monotone_key(amax)));  // (|x| or +inf: no NaN)
        uint32_t wban = 0;
        if (kRestore && p.num_banned > 0) wban = __reduce_add_sync(0xFFFFFFFFu, banned_hits);
        if (lane == 0) {
            s_wtail[warp] = wt;
            s_wproc[warp] = wp;
            s_wfill[warp] = warp_count;
            s_wamax[warp] = wamax;
            s_wban[warp] = wban;
        }
    }
    __syncthreads();
    STAGE(10);
    if (kRestore && p.wait_before_writes) grid_dependency_wait();  // the first write to scratch that the kernel before this one may still be reading
#ifdef PSX_STAGE_CLOCKS
    if (threadIdx.x == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); clk[15] = t_; }
#endif
    STAGE(18);
    // The part's record, by three warps side by side, each ahead of its share of the hand-off.
    PartStats* const record = p.stats + part_index;
    if (warp == 0) {
        // The warps' sums, joined in a fixed order by the first eight lanes: ((0+4)+(2+6)) + ((1+5)+(3+7)).
        double t = lane < kScanWarps ? s_wtail[lane] : 0.0, q = (second_exp && lane < kScanWarps) ? s_wproc[lane] : 0.0;
#pragma unroll
        for (int o = kScanWarps / 2; o > 0; o >>= 1) {
            t += __shfl_down_sync(0xFFFFFFFFu, t, o);
            if (second_exp) q += __shfl_down_sync(0xFFFFFFFFu, q, o);
        }
        const float camax = from_ordered_key(__reduce_max_sync(0xFFFFFFFFu, lane < kScanWarps ? monotone_key(s_wamax[lane]) : 0u));
        if (lane == 0) {
            // The exponents used c_l2 where cmax*log2(e) was meant: put the dropped part back.
            const double raw_tail = t * exp2_of_minus_small(c_res);
            double proc_tail = 0.0;
            if (kNucleus && cymax > -INFINITY) {
                // What stays behind is unflagged, so its processed value is l / T; without a
                // temperature the processed tail is the raw one measured against the other maximum.
                proc_tail = second_exp      ? q * exp2_of_minus_small(pc_res)
                            : cmax == cymax ? raw_tail
                                            : raw_tail * exp((double)cmax - (double)cymax);
            }
            record->raw_tail = raw_tail;
            record->proc_tail = proc_tail;
            record->raw_max = cmax;
            record->thr = thr;
            record->nonfinite = (!(camax < INFINITY) || t != t || q != q) ? 1u : 0u;
        }
    } else if (warp == 1) {
        if (lane == 0) {  // (the one divide of the kernel when no processed tail is wanted)
            if (!kNucleus && pen_key != monotone_key(kPad)) cymax = fmaxf(cymax, penalize(from_ordered_key(pen_key), p.penalty));
            record->y_max = cymax;
        }
    } else if (warp == 2) {
        const uint32_t handed_on = flagged_total + __reduce_add_sync(0xFFFFFFFFu, lane < kScanWarps ? s_wfill[lane] : 0u);
        const uint32_t banned_handed_on = __reduce_add_sync(0xFFFFFFFFu, lane < kScanWarps ? s_wban[lane] : 0u);
        if (lane == 0) {
            p.part_counts[part_index] = min(handed_on, (uint32_t)kPartCap);
            const int64_t first = max((int64_t)v0 * 4 - (int64_t)misalign, (int64_t)0);
            const int64_t last = min((int64_t)v1 * 4 - (int64_t)misalign, p.cols);
            const uint32_t logits_here = (uint32_t)(last - first);
            // alive: neither handed on nor banned (with kRestore a banned logit below the threshold stays behind)
            const uint32_t not_alive = handed_on + ((kRestore && p.num_banned > 0) ? s_banned_here - banned_handed_on : 0u);
            record->alive_tail = logits_here > not_alive ? logits_here - not_alive : 0u;
            record->overflow = handed_on > (uint32_t)kPartCap ? 1u : 0u;
        }
    }
    STAGE(19);
    if (any_noted) {  // slots in warp order, then lane, trip, component -- a fixed order
        uint32_t slot = flagged_total + before_mine + __reduce_add_sync(0xFFFFFFFFu, lane < warp ? s_wfill[lane] : 0u);
        for (uint32_t m2 = noted; m2; m2 &= m2 - 1) {
            const int v = (__ffs(m2) - 1) * kScanThreads + tid;
            const float4 d = data4[v];
            const float l[4] = {d.x, d.y, d.z, d.w};
            const uint32_t col = (uint32_t)(col_base + v * 4);
            uint32_t flag_nib = 0, ban_nib = 0;  // this vector's four bits of the bitmaps
            if (kRestore && use_flags) {
                flag_nib = (s_flag[v >> 3] >> ((v & 7) * 4)) & 15u;
                ban_nib = (s_ban[v >> 3] >> ((v & 7) * 4)) & 15u;
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (l[c] >= tprime) {
                    const uint32_t flags = ((ban_nib >> c) & 1u) ? kFlagBanned : ((flag_nib >> c) & 1u) ? kFlagPenalized : 0u;
                    if (slot < (uint32_t)kPartCap) part_out[slot] = make_uint2(__float_as_uint(l[c]), (col + c) | flags);
                    ++slot;
                }
            }
        }
    }
    announce_part();
    if (ends_the_grid) grid_dependency_wait();
#ifdef PSX_STAGE_CLOCKS
    STAGE(11);
    if (tid == 0 && part_index < 4096) {
        unsigned long long gt1; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt1));
        unsigned sm; asm volatile("mov.u32 %0, %smid;" : "=r"(sm));
        clk[12] = gt0; clk[13] = gt1; clk[14] = sm;
        for (int i = 0; i < 24; ++i) g_stage_clocks[part_index * 24 + i] = clk[i];
    }
#endif
}

#ifdef PSX_STAGE_CLOCKS
extern "C" __attribute__((visibility("default"))) int psx_debug_stage_clocks(unsigned long long* out, int n) {
    return (int)cudaMemcpyFromSymbol(out, g_stage_clocks, sizeof(unsigned long long) * n);
}
#endif

cudaError_t configure_scan_rows() {
    cudaError_t e = allow_all_dynamic_shared(scan_rows_kernel<true, false>);
    if (e == cudaSuccess) e = allow_all_dynamic_shared(scan_rows_kernel<false, false>);
    if (e == cudaSuccess) e = allow_all_dynamic_shared(scan_rows_kernel<false, true>);
    if (e == cudaSuccess) e = allow_all_dynamic_shared(scan_rows_kernel<false, false, true>);
    if (e == cudaSuccess) e = allow_all_dynamic_shared(scan_rows_kernel<false, true, true>);
    return e;
}

cudaError_t launch_scan_rows(const ScanParams& p, bool nucleus, cudaStream_t stream) {
    if (p.rows <= 0 || p.parts <= 0) return cudaSuccess;
    if (p.vecs_per_part > kPartVecs || p.rows > 65535ll * 65535ll) return cudaErrorInvalidConfiguration;
    const size_t shared = (size_t)((p.vecs_per_part + kScanThreads - 1) / kScanThreads * kScanThreads) * 16;
    const dim3 grid((unsigned)p.parts, (unsigned)(p.rows < 65535 ? p.rows : 65535), (unsigned)((p.rows + 65534) / 65535));
    // A flag can only lower a logit unless the penalty is below one (then l / p > l for l > 0).
    const bool flags_only_lower = !p.apply_penalty || p.penalty >= 1.0f;
    auto kernel = nucleus ? scan_rows_kernel<true, false> : flags_only_lower ? scan_rows_kernel<false, true> : scan_rows_kernel<false, false>;
    if (p.row_ready != nullptr) {  // (asked for by the vocabulary-sharded step, which has a top-k or is greedy)
        if (nucleus) return cudaErrorInvalidConfiguration;
        kernel = flags_only_lower ? scan_rows_kernel<false, true, true> : scan_rows_kernel<false, false, true>;
    }
    return launch_overlapping(kernel, grid, dim3(kScanThreads), shared, stream, p);
}

}  // namespace psx
