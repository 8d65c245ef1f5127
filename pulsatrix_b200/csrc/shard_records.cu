// Packs one GPU's row-pass output into one record per row for the all-gather of the
// vocabulary-sharded path: the shard's parts are joined into a single PartStats (max, tail
// sum-exp against that max, threshold = the largest part threshold) and only the candidates at
// or above that threshold are kept, in a fixed order (part, then place in the part's list); the
// others' mass moves into the tail.  One block of eight warps per row; a warp takes whole parts.
#include "shard_records.cuh"

namespace psx {

namespace {

constexpr int kPackThreads = 256;
constexpr int kPackWarps = kPackThreads / 32;
constexpr int kPackKeys = 4096;  // candidates of one row the exact local selection can look at;
                                 // afterwards the same words hold one kept-count per part

// The k-th largest (1-based, k <= m) of m keys in shared memory, by the whole block: four 8-bit
// radix passes, most significant digit first; the first warp finds the digit.  `pick` is two
// shared words for its answer.
__device__ uint32_t block_select_kth_key(const uint32_t* keys, int m, uint32_t k, uint32_t* hist, uint32_t* pick) {
    const int tid = threadIdx.x, lane = tid & 31;
    uint32_t prefix = 0, mask = 0, remaining = k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        hist[tid] = 0;  // kPackThreads == 256 bins
        __syncthreads();
        for (int i = tid; i < m; i += kPackThreads) {
            const uint32_t key = keys[i];
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid < 32) {
            uint32_t local = 0;  // lane L owns digits 255-8L down to 248-8L
            for (int b = 0; b < 8; ++b) local += hist[255 - 8 * lane - b];
            uint32_t incl = local;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (lane >= o) incl += up;
            }
            const uint32_t excl = incl - local;
            if (excl < remaining && remaining <= incl) {  // exactly one lane
                uint32_t above = excl;
                int d = 255 - 8 * lane;
                for (int b = 0; b < 8; ++b, --d) {
                    if (above + hist[d] >= remaining) break;
                    above += hist[d];
                }
                pick[0] = (uint32_t)d;
                pick[1] = above;
            }
        }
        __syncthreads();
        prefix |= pick[0] << shift;
        remaining -= pick[1];
        mask |= 255u << shift;
    }
    return prefix;
}

__global__ void __launch_bounds__(kPackThreads) pack_records_kernel(const PackParams p) {
    __shared__ uint32_t s_keys[kPackKeys];
    __shared__ uint32_t s_hist[256];
    __shared__ uint32_t s_pick[2];
    __shared__ uint32_t s_begin[32];
    __shared__ double s_sum[2][kPackWarps];
    __shared__ uint32_t s_dropped[kPackWarps];
    const int64_t row = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool apply_t = p.apply_temperature != 0;
    const PartStats* stats = p.stats + row * p.parts;
    bool in_time = true;
    if (p.to_peers && p.row_ready != nullptr) {
        // Under the row pass: this row's parts, and the step before this one, are waited for by name.
        __shared__ int s_in_time;
        if (tid == 0) {
            s_in_time = (wait_until_at_least_device(p.row_ready + row, p.row_ready_target, p.wait_limit_ns) &&
                         wait_until_at_least_device(p.step_done, p.step_done_target, p.wait_limit_ns)) ? 1 : 0;
        }
        __syncthreads();
        in_time = s_in_time != 0;
    } else {
        grid_dependency_wait();    // everything read here was written by the row pass before this kernel
    }
    // What follows this kernel may start now: it waits for this kernel's end, or for its records one by one.
    // (Not earlier: whoever starts after this point may rely on what this block has just waited for.)
    grid_dependents_may_launch();

    // Every warp joins the parts' records for itself (a few dozen small loads out of L2).
    float raw_max = -FLT_MAX, y_max = -INFINITY, thr = -INFINITY;
    uint32_t nonfinite = 0, overflow = 0, alive_tail = 0;
    for (int i = lane; i < p.parts; i += 32) {
        const PartStats s = stats[i];
        raw_max = fmaxf(raw_max, s.raw_max);
        y_max = fmaxf(y_max, s.y_max);
        thr = fmaxf(thr, s.thr);
        nonfinite |= s.nonfinite;
        overflow |= s.overflow;
        alive_tail += s.alive_tail;
    }
    raw_max = warp_max(raw_max);
    y_max = warp_max(y_max);
    thr = warp_max(thr);
    nonfinite = __reduce_or_sync(0xFFFFFFFFu, nonfinite);  // bit 0: a non-finite logit; bit 1: a copy that timed out
    overflow = __any_sync(0xFFFFFFFFu, overflow != 0) ? 1u : 0u;
    alive_tail = warp_sum_u32(alive_tail);
    float keep_from = relax_threshold(thr, apply_t, p.temperature);
    const float x_max = temper(y_max, apply_t, p.temperature);
    const int nseg = p.parts;  // one candidate list per part; at most kPackKeys parts (checked by the host)
    const uint32_t* seg_counts = p.part_counts + row * nseg;
    const uint2* cands = p.candidates + (size_t)row * nseg * kPartCap;
    // The parts' counts, asked for once and all together when a lane can hold one each (every warp for
    // itself), and their running sums: count_of(s) then costs a shuffle, not another trip to memory.
    const bool few = nseg <= 32;
    int my_count = 0, my_begin = 0, all_counts = 0;
    if (few) {
        my_count = lane < nseg ? min((int)seg_counts[lane], kPartCap) : 0;
        int incl = my_count;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += up;
        }
        my_begin = incl - my_count;
        all_counts = __shfl_sync(0xFFFFFFFFu, incl, 31);
        if (warp == 0 && lane < nseg) s_begin[lane] = (uint32_t)my_begin;
    }
    auto count_of = [&](int s) {  // (called by whole warps, with s the same in every lane)
        return few ? __shfl_sync(0xFFFFFFFFu, my_count, s) : min((int)seg_counts[s], kPartCap);
    };

    // The shard's own k-th largest processed value is a lower bound on the row's: nothing below
    // it (after the temperature divide's ties) can survive the merged top-k, so it need not travel.
    if (p.top_k > 0) {
        int m = 0;  // block-uniform
        if (few) {
            // all the candidates of the row as one list: a thread's loads do not wait for one another
            __syncthreads();  // s_begin
            m = all_counts;
#pragma unroll 2
            for (int f = tid; f < min(m, kPackKeys); f += kPackThreads) {
                int s = 0;
                while (s + 1 < nseg && (int)s_begin[s + 1] <= f) ++s;
                const uint2 c = cands[(size_t)s * kPartCap + (f - (int)s_begin[s])];
                s_keys[f] = ordered_key(processed_before_temperature(__uint_as_float(c.x), c.y, p.penalty));
            }
        } else {
            for (int s = 0; s < nseg; ++s) {
                const int cnt = min((int)seg_counts[s], kPartCap);
                for (int i = tid; i < cnt; i += kPackThreads) {
                    if (m + i < kPackKeys) {
                        const uint2 c = cands[(size_t)s * kPartCap + i];
                        s_keys[m + i] = ordered_key(processed_before_temperature(__uint_as_float(c.x), c.y, p.penalty));
                    }
                }
                m += cnt;
            }
        }
        __syncthreads();
        if (m <= kPackKeys && m > p.top_k) {
            const uint32_t kth = block_select_kth_key(s_keys, m, (uint32_t)p.top_k, s_hist, s_pick);
            keep_from = fmaxf(keep_from, relax_threshold(from_ordered_key(kth), apply_t, p.temperature));
        }
        __syncthreads();  // the keys are done with: their words now hold the parts' kept counts
    } else if (!p.do_sample) {
        keep_from = fmaxf(y_max, -FLT_MAX);  // greedy: the maximum and its ties
    }

    // Tails of the parts: thread t takes parts t, t + 256, ...
    double raw_tail = 0.0, proc_tail = 0.0;
    for (int i = tid; i < p.parts; i += kPackThreads) {
        const PartStats s = stats[i];
        raw_tail += s.raw_tail * exp((double)s.raw_max - (double)raw_max);
        if (s.y_max > -INFINITY && s.proc_tail > 0.0) {
            proc_tail += s.proc_tail * exp((double)temper(s.y_max, apply_t, p.temperature) - (double)x_max);
        }
    }

    // First sweep: warp w takes parts w, w + 8, ...; counts what each keeps, and moves the mass of
    // what it drops into the tails.  A dropped candidate belongs to the raw tail like the logits the row
    // pass left behind, and its exponential is taken the same way: ex2 in float against the rounded
    // exponent of the maximum, the rounding put back once for the whole sum.  The processed tail is only
    // ever read when no top-k is set; then it keeps its double-precision exponentials.
    uint32_t* s_kept = s_keys;
    uint32_t dropped = 0;  // warp-uniform
    constexpr float kLog2e = 1.4426950408889634f;
    const float c_l2 = __fmul_rn(raw_max, kLog2e);
    const float c_res = __fmaf_rn(raw_max, kLog2e, -c_l2);
    const bool want_processed = p.top_k <= 0;
    float dropped_raw = 0.0f;
    for (int s = warp; s < nseg; s += kPackWarps) {
        const int cnt = count_of(s);
        uint32_t kept = 0;
        for (int base = 0; base < cnt; base += 32) {
            const int i = base + lane;
            bool keep = false;
            if (i < cnt) {
                const uint2 c = cands[(size_t)s * kPartCap + i];
                const float l = __uint_as_float(c.x);
                const float y = processed_before_temperature(l, c.y, p.penalty);
                keep = y >= keep_from;
                if (!keep) {
                    dropped_raw += ex2_approx(__fmaf_rn(l, kLog2e, -c_l2));
                    if (want_processed && y > -INFINITY) proc_tail += exp((double)temper(y, apply_t, p.temperature) - (double)x_max);
                }
            }
            kept += __popc(__ballot_sync(0xFFFFFFFFu, keep));
        }
        dropped += (uint32_t)cnt - kept;
        if (lane == 0) s_kept[s] = kept;
    }
    raw_tail += (double)dropped_raw * exp2_of_minus_small(c_res);
    raw_tail = warp_sum(raw_tail);
    proc_tail = warp_sum(proc_tail);
    if (lane == 0) {
        s_sum[0][warp] = raw_tail;
        s_sum[1][warp] = proc_tail;
        s_dropped[warp] = dropped;
    }
    __syncthreads();

    // Second sweep: a part's kept candidates go where the parts before it end.
    char* record;
    uint32_t* arrival = nullptr;
    if (p.to_peers) {
        const PeerLayout& l = p.peers;
        const int64_t owner = row / l.rows_per_rank, within = row - owner * l.rows_per_rank;
        record = l.base[owner] + l.records_offset + ((int64_t)l.rank * l.rows_per_rank + within) * l.record_bytes;
        arrival = reinterpret_cast<uint32_t*>(l.base[owner] + l.arrivals_offset) + within;
    } else {
        record = static_cast<char*>(p.records) + row * (int64_t)shard_record_bytes(p.capacity);
    }
    uint2* out = reinterpret_cast<uint2*>(record + kRecordCandidatesOffset);
    for (int s = warp; s < nseg; s += kPackWarps) {
        uint32_t before = 0;
        for (int j = lane; j < s; j += 32) before += s_kept[j];
        before = warp_sum_u32(before);
        const int cnt = count_of(s);
        if (s_kept[s] == 0) continue;
        for (int base = 0; base < cnt; base += 32) {
            const int i = base + lane;
            bool keep = false;
            uint2 c = make_uint2(0, 0);
            if (i < cnt) {
                c = cands[(size_t)s * kPartCap + i];
                keep = processed_before_temperature(__uint_as_float(c.x), c.y, p.penalty) >= keep_from;
            }
            const uint32_t votes = __ballot_sync(0xFFFFFFFFu, keep);
            if (keep) {
                const uint32_t slot = before + __popc(votes & ((1u << lane) - 1u));
                if (slot < (uint32_t)p.capacity) out[slot] = c;
            }
            before += __popc(votes);
        }
    }
    if (tid == 0) {
        uint32_t kept = 0, all_dropped = 0;
        for (int s = 0; s < nseg; ++s) kept += s_kept[s];
        double t = 0.0, q = 0.0;
        for (int w = 0; w < kPackWarps; ++w) {  // a fixed order
            t += s_sum[0][w];
            q += s_sum[1][w];
            all_dropped += s_dropped[w];
        }
        PartStats s;
        s.raw_tail = t;
        s.proc_tail = q;
        s.raw_max = raw_max;
        s.y_max = y_max;
        s.thr = thr;
        s.nonfinite = nonfinite | (in_time ? 0u : 2u);
        s.alive_tail = alive_tail + all_dropped;
        s.overflow = (overflow || kept > (uint32_t)p.capacity) ? 1u : 0u;
        *reinterpret_cast<PartStats*>(record + kRecordStatsOffset) = s;
        *reinterpret_cast<uint32_t*>(record + kRecordCountOffset) = min(kept, (uint32_t)p.capacity);
        *reinterpret_cast<uint32_t*>(record + kRecordCountOffset + 4) = 0;
    }
    if (arrival != nullptr) {  // the record is complete: the whole CTA's stores before the count
        __syncthreads();
        if (tid == 0) add_release_system(arrival, 1u);  // (a release: what the CTA wrote before the barrier is visible to whoever sees the count)
        if (p.row_ready != nullptr) grid_dependency_wait();  // (so that this kernel's end still implies the row pass's)
    }
}

}  // namespace

cudaError_t launch_pack_records(const PackParams& p, cudaStream_t stream) {
    if (p.rows <= 0) return cudaSuccess;
    if (p.parts > kPackKeys) return cudaErrorInvalidConfiguration;
    return launch_overlapping(pack_records_kernel, dim3((unsigned)p.rows), dim3(kPackThreads), 0, stream, p);
}

}  // namespace psx
