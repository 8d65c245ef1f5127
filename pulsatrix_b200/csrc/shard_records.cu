// Packs one GPU's row-pass output into one record per row for the all-gather of the
// vocabulary-sharded path: the shard's parts are joined into a single PartStats (max, tail
// sum-exp against that max, threshold = the largest part threshold) and only the candidates at
// or above that threshold are kept, in a fixed order; the others' mass moves into the tail.
// One warp per row; a few KB read and about a KB written per row.
#include "shard_records.cuh"

namespace psx {

namespace {

constexpr int kPackKeys = 4096;  // candidates of one row the exact local selection can look at

// The k-th largest (1-based, k <= m) of m keys in shared memory, by one warp: four 8-bit radix
// passes, most significant digit first.
__device__ uint32_t warp_select_kth(const uint32_t* keys, int m, uint32_t k, uint32_t* hist, int lane) {
    uint32_t prefix = 0, mask = 0, remaining = k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int b = lane; b < 256; b += 32) hist[b] = 0;
        __syncwarp();
        for (int i = lane; i < m; i += 32) {
            const uint32_t key = keys[i];
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncwarp();
        uint32_t local = 0;  // lane L owns digits 255-8L down to 248-8L
        for (int b = 0; b < 8; ++b) local += hist[255 - 8 * lane - b];
        uint32_t incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += up;
        }
        const uint32_t excl = incl - local;
        const bool here = excl < remaining && remaining <= incl;
        uint32_t digit = 0, above = 0;
        if (here) {
            above = excl;
            int d = 255 - 8 * lane;
            for (int b = 0; b < 8; ++b, --d) {
                if (above + hist[d] >= remaining) break;
                above += hist[d];
            }
            digit = (uint32_t)d;
        }
        const int owner = __ffs(__ballot_sync(0xFFFFFFFFu, here)) - 1;
        digit = __shfl_sync(0xFFFFFFFFu, digit, owner);
        above = __shfl_sync(0xFFFFFFFFu, above, owner);
        prefix |= digit << shift;
        remaining -= above;
        mask |= 255u << shift;
        __syncwarp();
    }
    return prefix;
}

__global__ void __launch_bounds__(32) pack_records_kernel(const PackParams p) {
    __shared__ uint32_t s_keys[kPackKeys];
    __shared__ uint32_t s_hist[256];
    const int64_t row = blockIdx.x;
    const int lane = threadIdx.x;
    const bool apply_t = p.apply_temperature != 0;
    const PartStats* stats = p.stats + row * p.parts;

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
    nonfinite = __any_sync(0xFFFFFFFFu, nonfinite != 0) ? 1u : 0u;
    overflow = __any_sync(0xFFFFFFFFu, overflow != 0) ? 1u : 0u;
    alive_tail = warp_sum_u32(alive_tail);
    float keep_from = relax_threshold(thr, apply_t, p.temperature);
    const float x_max = temper(y_max, apply_t, p.temperature);
    const int nseg = p.parts;  // one candidate list per part
    const uint32_t* seg_counts = p.part_counts + row * nseg;
    const uint2* cands = p.candidates + (size_t)row * nseg * kPartCap;

    // The shard's own k-th largest processed value is a lower bound on the row's: nothing below
    // it (after the temperature divide's ties) can survive the merged top-k, so it need not travel.
    if (p.top_k > 0) {
        int m = 0;  // warp-uniform
        for (int s = 0; s < nseg; ++s) {
            const int cnt = min((int)seg_counts[s], kPartCap);
            for (int i = lane; i < cnt; i += 32) {
                if (m + i < kPackKeys) {
                    const uint2 c = cands[(size_t)s * kPartCap + i];
                    s_keys[m + i] = ordered_key(processed_before_temperature(__uint_as_float(c.x), c.y, p.penalty));
                }
            }
            m += cnt;
        }
        __syncwarp();
        if (m <= kPackKeys && m > p.top_k) {
            const uint32_t kth = warp_select_kth(s_keys, m, (uint32_t)p.top_k, s_hist, lane);
            keep_from = fmaxf(keep_from, relax_threshold(from_ordered_key(kth), apply_t, p.temperature));
        }
    } else if (!p.do_sample) {
        keep_from = fmaxf(y_max, -FLT_MAX);  // greedy: the maximum and its ties
    }

    double raw_tail = 0.0, proc_tail = 0.0;
    for (int i = lane; i < p.parts; i += 32) {
        const PartStats s = stats[i];
        raw_tail += s.raw_tail * exp((double)s.raw_max - (double)raw_max);
        if (s.y_max > -INFINITY && s.proc_tail > 0.0) {
            proc_tail += s.proc_tail * exp((double)temper(s.y_max, apply_t, p.temperature) - (double)x_max);
        }
    }

    char* record = static_cast<char*>(p.records) + row * (int64_t)shard_record_bytes(p.capacity);
    uint2* out = reinterpret_cast<uint2*>(record + kRecordCandidatesOffset);
    uint32_t kept = 0, dropped = 0;  // warp-uniform
    for (int s = 0; s < nseg; ++s) {
        const int cnt = min((int)seg_counts[s], kPartCap);
        for (int base = 0; base < cnt; base += 32) {
            const int i = base + lane;
            bool keep = false, drop = false;
            uint2 c = make_uint2(0, 0);
            if (i < cnt) {
                c = cands[(size_t)s * kPartCap + i];
                const float l = __uint_as_float(c.x);
                const float y = processed_before_temperature(l, c.y, p.penalty);
                keep = y >= keep_from;
                drop = !keep;
                if (drop) {
                    raw_tail += exp((double)l - (double)raw_max);
                    if (y > -INFINITY) {
                        proc_tail += exp((double)temper(y, apply_t, p.temperature) - (double)x_max);
                    }
                }
            }
            const uint32_t votes = __ballot_sync(0xFFFFFFFFu, keep);
            if (keep) {
                const uint32_t slot = kept + __popc(votes & ((1u << lane) - 1u));
                if (slot < (uint32_t)p.capacity) out[slot] = c;
            }
            kept += __popc(votes);
            dropped += __popc(__ballot_sync(0xFFFFFFFFu, drop));
        }
    }
    raw_tail = warp_sum(raw_tail);
    proc_tail = warp_sum(proc_tail);
    if (lane == 0) {
        PartStats s;
        s.raw_tail = raw_tail;
        s.proc_tail = proc_tail;
        s.raw_max = raw_max;
        s.y_max = y_max;
        s.thr = thr;
        s.nonfinite = nonfinite;
        s.alive_tail = alive_tail + dropped;
        s.overflow = (overflow || kept > (uint32_t)p.capacity) ? 1u : 0u;
        *reinterpret_cast<PartStats*>(record + kRecordStatsOffset) = s;
        *reinterpret_cast<uint32_t*>(record + kRecordCountOffset) = min(kept, (uint32_t)p.capacity);
        *reinterpret_cast<uint32_t*>(record + kRecordCountOffset + 4) = 0;
    }
}

}  // namespace

cudaError_t launch_pack_records(const PackParams& p, cudaStream_t stream) {
    if (p.rows <= 0) return cudaSuccess;
    pack_records_kernel<<<(unsigned)p.rows, 32, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace psx
