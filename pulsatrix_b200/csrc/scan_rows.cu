// The row pass: the one kernel that reads the logits from HBM.
//
// Each CTA owns one "part" of one row: up to 4096 float4 vectors (16384 logits) that it loads
// with 128-bit streaming loads, all issued up front, and then keeps in registers.  From the
// registers it derives, without touching HBM again,
//   * the part's raw maximum and, against it, the sum of exp over everything that is not handed
//     on as a candidate (the unprocessed log-softmax of src/generation.cpp:133,156 needs both),
//   * the repetition penalty and EOS ban for the few columns the row's history names
//     (src/generation.cpp:59-73), found through a per-thread bit mask built in shared memory,
//   * a threshold that at least `k_need` of the part's processed logits reach -- the smallest of
//     the per-warp kp-th largest per-thread maxima, so no sort of the data is needed -- and
//   * every logit at or above that threshold as a candidate (raw value, column, flags), written
//     warp by warp in a fixed order so that the survivor stage is reproducible bit for bit.
// Selection works on the logits BEFORE the temperature divide: dividing by a positive number is
// monotonic, so the k-th largest commutes with it, and the threshold is relaxed by the few ulps
// that the divide can merge (relax_threshold).
//
// HBM bound: 4 bytes per logit read once; everything written is a few hundred bytes per part.
#include "scan_rows.cuh"

namespace psx {

namespace {

constexpr float kLog2e = 1.4426950408889634f;
// log2(e) = kLog2e * (1 + kLog2eRel): the part of log2(e) that the float constant drops.
constexpr float kLog2eRel = (float)(1.4426950408889634073599246810019 / (double)1.4426950408889634f - 1.0);
constexpr float kPad = -FLT_MAX;  // stands for "no logit here": finite, never the maximum

__device__ __forceinline__ float max4(const float4& v) { return fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)); }
__device__ __forceinline__ float amax4(const float4& v) {
    return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
}
__device__ __forceinline__ float comp(const float4& v, int c) { return c == 0 ? v.x : c == 1 ? v.y : c == 2 ? v.z : v.w; }
__device__ __forceinline__ void blank(float4& v, int c) {
    if (c == 0) v.x = kPad; else if (c == 1) v.y = kPad; else if (c == 2) v.z = kPad; else v.w = kPad;
}

// Marks, in the per-thread bit masks, the columns of this part that `ids` names.
__device__ __forceinline__ void mark_ids(const int64_t* ids, int64_t begin, int64_t end, const ScanParams& p,
                                         uint32_t misalign, int v0, int v1, uint32_t* masks) {
    for (int64_t i = begin + threadIdx.x; i < end; i += kScanThreads) {
        const int64_t id = ids[i];
        if (id < 0 || id >= p.vocab) continue;  // src/generation.cpp:62: ids outside the vocabulary are ignored
        const int64_t col = id - p.col_begin;
        if (col < 0 || col >= p.cols) continue;
        const int64_t pos = col + misalign;
        const int64_t v = pos >> 2;
        if (v < v0 || v >= v1) continue;
        const int rel = (int)(v - v0);
        const int bit = (rel >> 8) * 4 + (int)(pos & 3);
        atomicOr(&masks[(rel & 255) * 2 + (bit >> 5)], 1u << (bit & 31));
    }
}

}  // namespace

template <bool kNucleus>
__global__ void __launch_bounds__(kScanThreads, 2) scan_rows_kernel(const ScanParams p) {
    const int part = blockIdx.x % p.parts;
    const int64_t row = blockIdx.x / p.parts;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    __shared__ uint32_t s_pen[kScanThreads * 2];
    __shared__ uint32_t s_ban[kScanThreads * 2];
    __shared__ float s_wraw[kScanWarps], s_wamax[kScanWarps], s_wymax[kScanWarps], s_wthr[kScanWarps];
    __shared__ double s_wtail[kScanWarps], s_wproc[kScanWarps];
    __shared__ uint32_t s_walive[kScanWarps], s_wover[kScanWarps];

    // ---- geometry: the row as aligned float4 vectors ------------------------------------------
    const float* row_ptr = p.logits + row * p.row_stride;
    const uint32_t misalign = (uint32_t)((reinterpret_cast<uintptr_t>(row_ptr) >> 2) & 3);
    const float4* vbase = reinterpret_cast<const float4*>(row_ptr - misalign);
    const int nv = (int)((misalign + p.cols + 3) >> 2);
    const int v0 = part * p.vecs_per_part;
    const int v1 = min(v0 + p.vecs_per_part, nv);
    if (v1 <= v0) {  // a part past the end of a row that starts on a 16-byte boundary: nothing to report
        if (tid < kScanWarps) p.seg_counts[((size_t)row * p.parts + part) * kScanWarps + tid] = 0;
        if (tid == 0) {
            PartStats s;
            s.raw_tail = 0.0; s.proc_tail = 0.0; s.raw_max = kPad; s.y_max = -INFINITY; s.thr = -INFINITY;
            s.nonfinite = 0; s.alive_tail = 0; s.overflow = 0;
            p.stats[(size_t)row * p.parts + part] = s;
        }
        return;
    }

    // ---- all loads first: 16 independent 128-bit streaming loads per thread ---------------------
    float4 d[kVecPerThread];
    uint64_t dead = 0;  // bit 4j+c set: component c of vector j holds no logit of this row
#pragma unroll
    for (int j = 0; j < kVecPerThread; ++j) {
        const int v = v0 + j * kScanThreads + tid;
        if (v < v1) {
            d[j] = __ldcs(vbase + v);
        } else {
            d[j] = make_float4(kPad, kPad, kPad, kPad);
            dead |= 0xFull << (4 * j);
        }
    }

    // ---- history -> per-thread masks, while the loads are in flight --------------------------------
    s_pen[tid * 2] = 0; s_pen[tid * 2 + 1] = 0;
    s_ban[tid * 2] = 0; s_ban[tid * 2 + 1] = 0;
    __syncthreads();
    if (p.apply_penalty) {
        mark_ids(p.history_ids, p.history_offsets[row], p.history_offsets[row + 1], p, misalign, v0, v1, s_pen);
    }
    if (p.num_banned > 0) mark_ids(p.banned_ids, 0, p.num_banned, p, misalign, v0, v1, s_ban);
    __syncthreads();
    const uint64_t pen = (uint64_t)s_pen[tid * 2] | ((uint64_t)s_pen[tid * 2 + 1] << 32);
    uint64_t ban = (uint64_t)s_ban[tid * 2] | ((uint64_t)s_ban[tid * 2 + 1] << 32);

    // The first and last vector of a row can reach outside it (rows need not start or end on a
    // 16-byte boundary): blank those components.
#pragma unroll
    for (int j = 0; j < kVecPerThread; ++j) {
        const int v = v0 + j * kScanThreads + tid;
        if (v < v1 && (v == 0 || v == nv - 1)) {
            const int64_t first_col = (int64_t)v * 4 - misalign;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (first_col + c < 0 || first_col + c >= p.cols) {
                    blank(d[j], c);
                    dead |= 1ull << (4 * j + c);
                }
            }
        }
    }
    ban |= dead;
    const uint64_t special = pen | ban;

    // ---- per-thread maxima ----------------------------------------------------------------------------
    float m_raw = kPad, amax = 0.0f, ymax = -INFINITY;
#pragma unroll
    for (int j = 0; j < kVecPerThread; ++j) {
        m_raw = fmaxf(m_raw, max4(d[j]));
        amax = fmaxf(amax, amax4(d[j]));
    }
    // Padding must not look like an infinity, and it does not: |kPad| is finite.
    if (special == 0) {
        ymax = m_raw;
    } else {
#pragma unroll
        for (int j = 0; j < kVecPerThread; ++j) {
            const uint32_t nib_p = (uint32_t)(pen >> (4 * j)) & 0xFu, nib_b = (uint32_t)(ban >> (4 * j)) & 0xFu;
            if ((nib_p | nib_b) == 0) {
                ymax = fmaxf(ymax, max4(d[j]));
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float l = comp(d[j], c);
                    const float y = ((nib_b >> c) & 1) ? -INFINITY : ((nib_p >> c) & 1) ? penalize(l, p.penalty) : l;
                    ymax = fmaxf(ymax, y);
                }
            }
        }
    }

    // ---- block: raw max, finite check, selection threshold ----------------------------------------
    const int live_threads = min(kScanThreads, max(v1 - v0, 0));
    const int full_warps = live_threads >> 5;
    int kp = 33;  // > 32: no threshold, hand everything on
    if (full_warps > 0) kp = (p.k_need + full_warps - 1) / full_warps;
    {
        const float wraw = warp_max(m_raw), wamax = warp_max(amax), wymax = warp_max(ymax);
        float wthr = -INFINITY;
        if (kp == 1) wthr = wymax;
        else if (kp <= 32) wthr = warp_kth_largest(ymax, kp, lane);
        if (lane == 0) {
            s_wraw[warp] = wraw;
            s_wamax[warp] = wamax;
            s_wymax[warp] = wymax;
            s_wthr[warp] = wthr;
        }
    }
    __syncthreads();
    float cmax = kPad, camax = 0.0f, cymax = -INFINITY, thr = INFINITY;
#pragma unroll
    for (int w = 0; w < kScanWarps; ++w) {
        cmax = fmaxf(cmax, s_wraw[w]);
        camax = fmaxf(camax, s_wamax[w]);
        cymax = fmaxf(cymax, s_wymax[w]);
        if (w < full_warps) thr = fminf(thr, s_wthr[w]);
    }
    if (full_warps == 0 || kp > 32) thr = -INFINITY;
    const float tprime = relax_threshold(thr, p.apply_temperature != 0, p.temperature);

    // ---- exp-sum of the non-candidates and candidate hand-off ------------------------------------------
    const float c_l2 = __fmul_rn(cmax, kLog2e);
    const float c_res = __fmaf_rn(cmax, kLog2e, -c_l2);  // cmax*kLog2e = c_l2 + c_res exactly
    const bool proc_same = !p.apply_temperature && (cymax == cmax);
    const float pc_l2 = __fmul_rn(cymax, p.log2e_over_t);
    const float pc_res = __fmaf_rn(cymax, p.log2e_over_t, -pc_l2);

    const size_t seg = ((size_t)row * p.parts + part) * kScanWarps + warp;
    uint2* seg_out = p.candidates + seg * kSegCap;
    uint32_t seg_fill = 0;       // warp-uniform
    uint32_t pushed = 0;         // this thread's candidates
    double tail = 0.0, proc = 0.0;
    const uint32_t lanes_below = (1u << lane) - 1u;

#pragma unroll
    for (int j = 0; j < kVecPerThread; ++j) {
        const uint32_t nib_p = (uint32_t)(pen >> (4 * j)) & 0xFu, nib_b = (uint32_t)(ban >> (4 * j)) & 0xFu;
        float e[4], ep[4];
        bool cand[4];
        uint32_t flags[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float l = comp(d[j], c);
            float y = l;
            flags[c] = 0;
            if ((nib_p | nib_b) != 0) {
                if ((nib_b >> c) & 1) { y = -INFINITY; flags[c] = kFlagBanned; }
                else if ((nib_p >> c) & 1) { y = penalize(l, p.penalty); flags[c] = kFlagPenalized; }
            }
            cand[c] = y >= tprime;
            float x = __fmaf_rn(l, kLog2e, -c_l2);
            if (kNucleus) x = __fmaf_rn(x, kLog2eRel, x);
            e[c] = cand[c] ? 0.0f : ex2_approx(x);
            if (kNucleus) {
                if (cand[c] || y == -INFINITY) {
                    ep[c] = 0.0f;
                } else if (proc_same && flags[c] == 0) {
                    ep[c] = e[c];
                } else {
                    float xp = __fmaf_rn(y, p.log2e_over_t, -pc_l2);
                    xp = __fmaf_rn(xp, kLog2eRel, xp);
                    ep[c] = ex2_approx(xp);
                }
            }
        }
        tail += (double)((e[0] + e[1]) + (e[2] + e[3]));
        if (kNucleus) proc += (double)((ep[0] + ep[1]) + (ep[2] + ep[3]));

        if (__any_sync(0xFFFFFFFFu, cand[0] | cand[1] | cand[2] | cand[3])) {
            const int v = v0 + j * kScanThreads + tid;
            const int64_t first_col = (int64_t)v * 4 - misalign + p.col_begin;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t votes = __ballot_sync(0xFFFFFFFFu, cand[c]);
                if (cand[c]) {
                    const uint32_t slot = seg_fill + __popc(votes & lanes_below);
                    if (slot < (uint32_t)kSegCap) {
                        seg_out[slot] = make_uint2(__float_as_uint(comp(d[j], c)), (uint32_t)(first_col + c) | flags[c]);
                    }
                    ++pushed;
                }
                seg_fill += __popc(votes);
            }
        }
    }

    // ---- block reduction in a fixed order, then the part's record ---------------------------------------
    const uint32_t alive = 4u * kVecPerThread - (uint32_t)__popcll(ban) - pushed;
    {
        const double wt = warp_sum(tail), wp = warp_sum(proc);
        const uint32_t wa = warp_sum_u32(alive);
        if (lane == 0) {
            s_wtail[warp] = wt;
            s_wproc[warp] = wp;
            s_walive[warp] = wa;
            s_wover[warp] = seg_fill > (uint32_t)kSegCap ? 1u : 0u;
            p.seg_counts[seg] = min(seg_fill, (uint32_t)kSegCap);
        }
    }
    __syncthreads();
    if (tid == 0) {
        double t = 0.0, q = 0.0;
        uint32_t a = 0, over = 0;
#pragma unroll
        for (int w = 0; w < kScanWarps; ++w) {
            t += s_wtail[w];
            q += s_wproc[w];
            a += s_walive[w];
            over |= s_wover[w];
        }
        // The exponent used c_l2 where cmax*log2(e) was meant: put the dropped part back.
        const double fix = exp2(-(double)c_res);
        const double pfix = exp2(-(double)pc_res);
        PartStats s;
        s.raw_tail = t * fix;
        s.proc_tail = q * (proc_same ? fix : pfix);
        s.raw_max = cmax;
        s.y_max = cymax;
        s.thr = thr;
        s.nonfinite = (!(camax < INFINITY) || t != t) ? 1u : 0u;
        s.alive_tail = a;
        s.overflow = over;
        p.stats[(size_t)row * p.parts + part] = s;
    }
}

cudaError_t launch_scan_rows(const ScanParams& p, bool nucleus, cudaStream_t stream) {
    const long long blocks = (long long)p.rows * p.parts;
    if (blocks <= 0) return cudaSuccess;
    if (blocks > 0x7FFFFFFFll) return cudaErrorInvalidConfiguration;
    if (nucleus) scan_rows_kernel<true><<<(unsigned)blocks, kScanThreads, 0, stream>>>(p);
    else scan_rows_kernel<false><<<(unsigned)blocks, kScanThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace psx
