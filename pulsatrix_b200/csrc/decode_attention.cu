// Attention of a few new positions over the KV cache (the per-token loop of generate()):
// MultiHeadAttentionModule::forward_cached, src/multihead_attention_module.cpp:562-586 --
//   scores = q . K^T per (batch, head) (gemm_ex), times the score scale (axpby), masked entries set
//   to the lowest float (attention_mask_fill: causal with the cache offset, sliding window, key
//   padding; src/row_math.hpp:117-127), softmax over the cached positions (softmax_rows),
//   context = P . V (gemm); grouped-query heads read K/V head h / group in place.
// The reference makes five passes over an (N, H, L, total) score tensor; here the cache is read once
// and the scores never exist in memory.
//
// HBM bound: K and V of every (batch, kv head) are read once, 8 * total * D bytes each.
// One CTA of six warps takes one (batch, kv head) and one slice of the cached positions; the query
// rows of the whole group -- group heads x L new positions, at most 8 -- are answered together, so
// grouped-query heads share one pass over their K/V head.  A warp works through its positions 32 at a
// time:
//   - the K rows of a tile arrive in shared memory by bulk asynchronous copies (one 4*D-byte row per
//     lane, completing on an mbarrier, no multicast), padded to D + 4 floats so that lanes reading
//     different rows at the same offset fall into different banks; the next tile's rows are asked for as
//     soon as this tile's scores are formed, and land under the softmax and the context;
//   - lane t forms the dot products of position t with every query row (the query rows are read as
//     broadcasts), scales and masks them;
//   - the running maximum and sum of every query row are brought up to date (online softmax: what has
//     been accumulated is rescaled when the maximum moves), the tile's probabilities go to shared memory;
//   - lane c accumulates floats 4c .. 4c+3 of the context rows from the V rows (one contiguous run per
//     tile, one bulk copy, asked for when the tile starts: it lands while the scores are formed).
// One K tile and one V tile per warp (34 KB for a head dimension of 128) leave room for six warps per SM.
// The warps' partial results (maximum, sum, unnormalised context) meet in shared memory; with several
// slices per (batch, kv head) they go to scratch and a second kernel joins them.
//
// Float arithmetic in another order than the reference's loops: results agree within the reference's
// own CPU/GPU equivalence tolerance (1e-4, tests/backend_primitive_equivalence_cases.hpp:22), not bit
// for bit.  A fully masked row comes out as the reference's: every score equals the lowest float, so
// the softmax is uniform over all positions.
#include "decode_attention.cuh"

#include <algorithm>

#include "psx_async.cuh"
#include "psx_device.cuh"

namespace psx {

namespace {

constexpr int kAttnWarps = 6;      // warps of a CTA up to a head dimension of 128 (34 KB of tiles each)
constexpr int kAttnWarpsWide = 3;  // beyond it (67 KB each at 256)
inline int attention_warps(int head_dim) { return head_dim > 128 ? kAttnWarpsWide : kAttnWarps; }
constexpr int kTile = 32;          // positions per warp and tile: one per lane
constexpr float kMasked = -FLT_MAX;  // std::numeric_limits<float>::lowest()

// src/row_math.hpp:117-127 (i: new position, j: cached position, offset: positions cached before).
__device__ __forceinline__ bool masked(const float* keep_row, int64_t i, int64_t j, bool causal, int64_t offset, int64_t window) {
    if (causal && j > i + offset) return true;
    if (causal && window > 0 && j + window <= i + offset) return true;
    return keep_row != nullptr && keep_row[j] == 0.0f;
}

// R: query rows answered together (group x L, padded to 1, 2, 4 or 8); C: float4 chunks of a
// context row per lane (D <= 128 C); W: warps of a CTA.
template <int R, int C, int W>
__global__ void __launch_bounds__(W * 32) decode_attention_kernel(const AttentionParams p) {
    constexpr int kAttnWarps = W, kAttnThreads = W * 32;
    extern __shared__ __align__(16) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int D = p.head_dim, pitch = D + 4;
    const int rows = p.group * p.q_len;  // query rows of this kv head (<= R)
    // shared memory: the query rows; per warp a K tile, a V tile and the tile's probabilities; the warps'
    // maxima and sums.  (At the end a warp's partial context rows lie over its own K tile.)
    const size_t per_warp = (size_t)kTile * pitch + (size_t)kTile * D + (size_t)kTile * R;
    float* s_q = reinterpret_cast<float*>(smem);                        // R x D
    float* s_k = s_q + R * D + warp * per_warp;                         // 32 x (D + 4)
    float* s_v = s_k + kTile * pitch;                                   // 32 x D
    float* s_p = s_v + kTile * D;                                       // 32 x R
    float* s_ml = s_q + R * D + kAttnWarps * per_warp;                  // warps x R x 2
    auto ctx_of_warp = [&](int w) { return s_q + R * D + w * per_warp; };  // R x D, over warp w's K tile
    __shared__ __align__(8) uint64_t s_bar[kAttnWarps][2];              // K, V

    const int64_t nkv = blockIdx.x;  // (batch, kv head)
    const int64_t n = nkv / p.kv_heads, kvh = nkv % p.kv_heads;
    const int split = blockIdx.y;
    const float* keys = p.keys + nkv * p.max_len * D;
    const float* values = p.values + nkv * p.max_len * D;
    const float* keep_row = p.key_keep ? p.key_keep + n * p.total : nullptr;

    // the query rows of the group: row r = (head within the group) * L + (new position)
    for (int i = threadIdx.x; i < R * D; i += kAttnThreads) {
        const int r = i / D, d = i % D;
        float v = 0.0f;
        if (r < rows) {
            const int64_t head = kvh * p.group + r / p.q_len;
            v = p.q[((n * p.heads + head) * p.q_len + r % p.q_len) * D + d];
        }
        s_q[i] = v;
    }
    if (lane == 0) {
        barrier_init(&s_bar[warp][0], 1);
        barrier_init(&s_bar[warp][1], 1);
        barrier_init_fence();
    }
    __syncthreads();

    // this warp's positions: the split's share, cut into the warps' shares, in whole tiles
    const int64_t per_split = (p.total + p.splits - 1) / p.splits;
    const int64_t s0 = split * per_split, s1 = min(s0 + per_split, p.total);
    const int64_t tiles_in_split = s1 > s0 ? (s1 - s0 + kTile - 1) / kTile : 0;
    const int64_t tiles_per_warp = (tiles_in_split + kAttnWarps - 1) / kAttnWarps;
    const int64_t t_begin = s0 + warp * tiles_per_warp * kTile, t_end = min(t_begin + tiles_per_warp * kTile, s1);
    const int64_t my_tiles = t_end > t_begin ? (t_end - t_begin + kTile - 1) / kTile : 0;

    auto fetch_values = [&](int64_t tile) {  // the V rows of a tile are one contiguous run: one copy
        const int64_t first = t_begin + tile * kTile;
        const int count = (int)min((int64_t)kTile, t_end - first);
        if (lane == 0) {
            barrier_expect_bytes(&s_bar[warp][1], (uint32_t)count * (uint32_t)D * 4u);
            bulk_copy_to_shared(s_v, values + first * D, (uint32_t)count * (uint32_t)D * 4u, &s_bar[warp][1]);
        }
    };
    auto fetch_tile = [&](int64_t tile) {  // lane t asks for the K row of position t
        const int64_t first = t_begin + tile * kTile;
        const int count = (int)min((int64_t)kTile, t_end - first);
        if (lane == 0) barrier_expect_bytes(&s_bar[warp][0], (uint32_t)count * (uint32_t)D * 4u);
        __syncwarp();
        if (lane < count) {
            bulk_copy_to_shared(s_k + (size_t)lane * pitch, keys + (first + lane) * D, (uint32_t)D * 4u, &s_bar[warp][0]);
        }
    };

    float m_run[R], l_run[R];
    float4 ctx[R][C];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        m_run[r] = kMasked;  // (a score is never below the lowest float, so the first tile always sets it)
        l_run[r] = 0.0f;
#pragma unroll
        for (int c = 0; c < C; ++c) ctx[r][c] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    bool landed = true;
    int64_t issued = -1, waited = 0;  // the last tile asked for; the tiles waited for so far
    int64_t values_issued = -1, values_waited = 0;
    if (my_tiles > 0) { fetch_tile(0); issued = 0; }
    for (int64_t tile = 0; tile < my_tiles; ++tile) {
        // every lane has finished with the V tile (the warp met after the context of the tile before); its reads
        // through ordinary loads are ordered before the copy engine's writes
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        fetch_values(tile);
        values_issued = tile;
        landed = barrier_wait_bounded(&s_bar[warp][0], (uint32_t)(tile & 1), p.wait_limit_ns) && landed;
        if (!__all_sync(0xFFFFFFFFu, landed)) break;
        waited = tile + 1;
        const int64_t first = t_begin + tile * kTile;
        const int count = (int)min((int64_t)kTile, t_end - first);
        const int64_t pos = first + lane;

        // ---- scores of position `pos` against every query row -----------------------------------------
        float s[R];
#pragma unroll
        for (int r = 0; r < R; ++r) s[r] = 0.0f;
        const float* krow = s_k + (size_t)lane * pitch;
#pragma unroll 4
        for (int d = 0; d < D; d += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(krow + d);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float4 q4 = *reinterpret_cast<const float4*>(s_q + r * D + d);  // the same address in every lane
                s[r] = __fmaf_rn(q4.x, k4.x, s[r]);
                s[r] = __fmaf_rn(q4.y, k4.y, s[r]);
                s[r] = __fmaf_rn(q4.z, k4.z, s[r]);
                s[r] = __fmaf_rn(q4.w, k4.w, s[r]);
            }
        }
        // The K tile is done with: the next tile's rows can land under the rest of this tile's work.
        __syncwarp();
        if (tile + 1 < my_tiles) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            fetch_tile(tile + 1);
            issued = tile + 1;
        }
        // ---- scale, mask, and the running softmax of every query row ------------------------------------
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float x = kMasked;
            if (lane < count && r < rows) {
                x = __fmul_rn(p.scale, s[r]);
                if (masked(keep_row, r % p.q_len, pos, p.causal != 0, p.offset, p.window)) x = kMasked;
            }
            const bool counts = lane < count;  // (a lane beyond the tile adds nothing)
            const float tile_max = warp_max(counts ? x : kMasked);
            const float m_new = fmaxf(m_run[r], tile_max);
            const float e = counts ? __expf(x - m_new) : 0.0f;
            float e_sum = e;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) e_sum += __shfl_xor_sync(0xFFFFFFFFu, e_sum, o);
            const float rescale = __expf(m_run[r] - m_new);  // 1 when the maximum stays; 0 from the very first tile
            l_run[r] = __fmaf_rn(l_run[r], rescale, e_sum);
            m_run[r] = m_new;
#pragma unroll
            for (int c = 0; c < C; ++c) {
                ctx[r][c].x *= rescale; ctx[r][c].y *= rescale; ctx[r][c].z *= rescale; ctx[r][c].w *= rescale;
            }
            s_p[lane * R + r] = e;
        }
        __syncwarp();
        // ---- context: lane c owns floats 4c .. 4c + 3 of every row; the V tile has had the scores' time to land ----
        landed = barrier_wait_bounded(&s_bar[warp][1], (uint32_t)(tile & 1), p.wait_limit_ns) && landed;
        if (!__all_sync(0xFFFFFFFFu, landed)) break;
        values_waited = tile + 1;
#pragma unroll 4
        for (int t = 0; t < count; ++t) {
            float4 v4[C];
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const int d = 4 * (lane + 32 * c);
                v4[c] = d < D ? *reinterpret_cast<const float4*>(s_v + (size_t)t * D + d) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float pr = s_p[t * R + r];  // the same address in every lane
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    ctx[r][c].x = __fmaf_rn(pr, v4[c].x, ctx[r][c].x);
                    ctx[r][c].y = __fmaf_rn(pr, v4[c].y, ctx[r][c].y);
                    ctx[r][c].z = __fmaf_rn(pr, v4[c].z, ctx[r][c].z);
                    ctx[r][c].w = __fmaf_rn(pr, v4[c].w, ctx[r][c].w);
                }
            }
        }
        __syncwarp();  // the probabilities and the V tile are done with
    }

    // ---- the warps' partial results meet (a warp whose wait ran out may still have copies in flight into its
    // tiles and writes nothing there; the block then leaves below) ----------------------------------------------
    const bool warp_landed = __all_sync(0xFFFFFFFFu, landed);
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int d = 4 * (lane + 32 * c);
            if (warp_landed && d < D) *reinterpret_cast<float4*>(ctx_of_warp(warp) + (size_t)r * D + d) = ctx[r][c];
        }
        if (lane == 0) {
            s_ml[(warp * R + r) * 2] = m_run[r];
            s_ml[(warp * R + r) * 2 + 1] = l_run[r];
        }
    }
    const int timed_out = __syncthreads_or(landed ? 0 : 1);
    if (timed_out) {  // a copy did not complete in time: say so, let the copies in flight drain, leave
        if (threadIdx.x == 0 && p.status != nullptr) atomicOr(p.status, 1);
        if (lane == 0) {  // the last two fetches of this warp, if they have not been waited for
            if (issued >= waited) barrier_wait_bounded(&s_bar[warp][0], (uint32_t)(issued & 1), p.wait_limit_ns);
            if (values_issued >= values_waited) barrier_wait_bounded(&s_bar[warp][1], (uint32_t)(values_issued & 1), p.wait_limit_ns);
        }
        return;
    }
    // thread (r, d): joins the four warps' row r at column d
    for (int i = threadIdx.x; i < rows * D; i += kAttnThreads) {
        const int r = i / D, d = i % D;
        float m = kMasked;
        bool any = false;
        for (int w = 0; w < kAttnWarps; ++w) {
            if (s_ml[(w * R + r) * 2 + 1] > 0.0f) { m = fmaxf(m, s_ml[(w * R + r) * 2]); any = true; }
        }
        float l = 0.0f, acc = 0.0f;
        for (int w = 0; w < kAttnWarps; ++w) {
            const float lw = s_ml[(w * R + r) * 2 + 1];
            if (lw > 0.0f) {
                const float f = __expf(s_ml[(w * R + r) * 2] - m);
                l = __fmaf_rn(lw, f, l);
                acc = __fmaf_rn(ctx_of_warp(w)[(size_t)r * D + d], f, acc);
            }
        }
        const int64_t head = kvh * p.group + r / p.q_len;
        const int64_t out_row = (n * p.heads + head) * p.q_len + r % p.q_len;
        if (p.splits == 1) {
            p.context[out_row * D + d] = any ? __fdiv_rn(acc, l) : 0.0f;
        } else {  // unnormalised, with its maximum and sum, for the second kernel
            float* part = p.partial + ((out_row * p.splits + split) * (D + 2));
            part[d] = acc;
            if (d == 0) { part[D] = any ? m : kMasked; part[D + 1] = l; }
        }
    }
}

// Joins the slices of every query row: thread per (row, column).
__global__ void join_attention_splits_kernel(const AttentionParams p) {
    const int D = p.head_dim;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t out_rows = p.batch * p.heads * p.q_len;
    if (i >= out_rows * D) return;
    const int64_t row = i / D;
    const int d = (int)(i % D);
    const float* part = p.partial + row * p.splits * (D + 2);
    float m = kMasked;
    for (int s = 0; s < p.splits; ++s) {
        if (part[s * (D + 2) + D + 1] > 0.0f) m = fmaxf(m, part[s * (D + 2) + D]);
    }
    float l = 0.0f, acc = 0.0f;
    for (int s = 0; s < p.splits; ++s) {
        const float ls = part[s * (D + 2) + D + 1];
        if (ls > 0.0f) {
            const float f = __expf(part[s * (D + 2) + D] - m);
            l = __fmaf_rn(ls, f, l);
            acc = __fmaf_rn(part[s * (D + 2) + d], f, acc);
        }
    }
    p.context[i] = l > 0.0f ? __fdiv_rn(acc, l) : 0.0f;
}

template <int R, int C, int W>
cudaError_t launch_one(const AttentionParams& p, size_t shared, cudaStream_t stream) {
    static bool configured = false;  // (per instantiation; raising the limit twice is harmless)
    if (!configured) {
        const cudaError_t e = allow_all_dynamic_shared(decode_attention_kernel<R, C, W>);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    decode_attention_kernel<R, C, W><<<dim3((unsigned)(p.batch * p.kv_heads), (unsigned)p.splits), W * 32, shared, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace

int attention_rows_padded(int rows) { return rows <= 1 ? 1 : rows <= 2 ? 2 : rows <= 4 ? 4 : 8; }

size_t attention_shared_bytes(int rows_padded, int head_dim) {
    const size_t per_warp = (size_t)kTile * (head_dim + 4) + (size_t)kTile * head_dim + (size_t)kTile * rows_padded;
    const size_t warps = (size_t)attention_warps(head_dim);
    const size_t floats = (size_t)rows_padded * head_dim + warps * per_warp + warps * rows_padded * 2;
    return floats * sizeof(float);
}

int attention_splits(int64_t batch_kv, int64_t total, int sm_count, int head_dim) {
    // One CTA fills an SM, so the CTAs run in rounds of sm_count: the slices are chosen so that the last round
    // is as full as the others (512 CTAs on 148 SMs are 3.46 rounds, i.e. four, an eighth of the time idle;
    // 1024 are 6.92), with at least two tiles per warp in a slice, and only when that wins a few per cent (the
    // slices cost a second kernel).
    const int64_t most = std::max<int64_t>(1, std::min<int64_t>(128, total / (2 * attention_warps(head_dim) * kTile)));
    auto filled = [&](int64_t ctas) { return (double)ctas / (double)(((ctas + sm_count - 1) / sm_count) * sm_count); };
    int best = 1;
    double best_fill = filled(batch_kv);
    for (int64_t splits = 2; splits <= most; ++splits) {
        const double f = filled(batch_kv * splits);
        if (f > best_fill * 1.03) { best = (int)splits; best_fill = f; }
    }
    return best;
}

size_t attention_partial_bytes(const AttentionParams& p) {
    return p.splits > 1 ? (size_t)p.batch * p.heads * p.q_len * p.splits * (p.head_dim + 2) * sizeof(float) : 0;
}

cudaError_t launch_decode_attention(const AttentionParams& p, cudaStream_t stream) {
    if (p.batch <= 0 || p.total <= 0) return cudaSuccess;
    const int rows = p.group * p.q_len;
    if (rows < 1 || rows > 8 || p.head_dim % 4 != 0 || p.head_dim > 256 || p.head_dim < 4) return cudaErrorInvalidValue;
    const int R = attention_rows_padded(rows);
    const size_t shared = attention_shared_bytes(R, p.head_dim);
    const bool wide = p.head_dim > 128;  // two chunks of a context row per lane, three warps per CTA
    cudaError_t e;
    switch (R) {
        case 1: e = wide ? launch_one<1, 2, kAttnWarpsWide>(p, shared, stream) : launch_one<1, 1, kAttnWarps>(p, shared, stream); break;
        case 2: e = wide ? launch_one<2, 2, kAttnWarpsWide>(p, shared, stream) : launch_one<2, 1, kAttnWarps>(p, shared, stream); break;
        case 4: e = wide ? launch_one<4, 2, kAttnWarpsWide>(p, shared, stream) : launch_one<4, 1, kAttnWarps>(p, shared, stream); break;
        default: e = wide ? launch_one<8, 2, kAttnWarpsWide>(p, shared, stream) : launch_one<8, 1, kAttnWarps>(p, shared, stream); break;
    }
    if (e != cudaSuccess || p.splits == 1) return e;
    const int64_t elements = p.batch * p.heads * p.q_len * p.head_dim;
    join_attention_splits_kernel<<<(unsigned)((elements + 255) / 256), 256, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace psx
