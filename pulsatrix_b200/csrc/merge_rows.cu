// The survivor stage: one CTA per row turns the row pass's candidates into a token.
//
// Input per row: for each part its raw max / tail sum-exp and a few dozen candidates (raw logit,
// column, flags).  The stage
//   1. joins the parts' partial log-sum-exp (raw, and processed when a full-vocabulary top-p or
//      min-p needs it): M = max m_i, Z = sum z_i * exp(m_i - M) + sum over candidates, in double;
//   2. keeps the candidates at or above the largest part threshold (only those can survive any
//      filter), applies penalty and temperature with the reference's float operations, and sorts
//      them by (value descending, column ascending) in shared memory;
//   3. replays src/generation.cpp:80-152 on that short list in the reference's own order and
//      precision -- the k-th value with its ties, softmax sums in column order, the top-p walk in
//      ascending (value, column) order against 1 - (double)top_p, min-p against the first
//      maximum, the inverse-CDF walk in column order against the row's uniform -- all in double;
//   4. writes the token, float(log(exp(l - M) / Z)) of the raw logits (src/generation.cpp:156),
//      a row status and the distances of the two decisions from their boundaries.
// Reads a few KB per row and never touches the logits -- except for a row that does not fit the
// lists (more survivors or ties than they hold): that row is decided from the logits themselves
// by the same CTA (general_row_impl.cuh).
#ifdef PSX_STAGE_CLOCKS
// Profiling build only: thread 0 of each row's CTA stamps the SM clock at the stage boundaries.
__device__ unsigned long long g_merge_clocks[1024 * 16];
#define PSX_MERGE_STAGE(i) \
    do { if (threadIdx.x == 0) g_merge_clocks[(size_t)(blockIdx.x & 1023) * 16 + (i)] = clock64(); } while (0)
// wall-clock (globaltimer) stamps of each CTA: entry, after the wait for the row pass, exit
__device__ unsigned long long g_merge_times[1024 * 4];
#define PSX_MERGE_TIME(i) \
    do { if (threadIdx.x == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); \
         g_merge_times[(size_t)(blockIdx.x & 1023) * 4 + (i)] = t_; } } while (0)
#else
#define PSX_MERGE_TIME(i) do {} while (0)
#endif
#include "general_row_impl.cuh"
#include "merge_rows_impl.cuh"
#include "merge_rows_warp_impl.cuh"
#include "peer_exchange.cuh"

namespace psx {

namespace {

__device__ __forceinline__ void decide_row(const MergeParams& p, const int64_t row, unsigned long long* dyn) {
    if (p.general != 2) survivor::merge_row(p, row, dyn);
    if (p.general != 0 && p.logits != nullptr) {
        // A row the candidate lists could not decide is decided from the row itself.
        __syncthreads();
        if (p.general == 2 || p.row_status[row] == PSX_ROW_TOO_WIDE) survivor::general_row(p, row, dyn);
    }
}

__global__ void __launch_bounds__(kMergeThreads, 3) merge_rows_kernel(const MergeParams p) {
    extern __shared__ unsigned long long dyn[];
    PSX_MERGE_TIME(0);
    if (p.only_undecided) {
        // After a launch by warps: a few CTAs look through the rows for what the warps left undecided
        // (usually nothing).  The kernel after this one may start at once: it waits for this one where it must.
        grid_dependents_may_launch();
        grid_dependency_wait();
        __shared__ int s_found[kMergeThreads];
        __shared__ int s_n;
        const int64_t per_cta = (p.rows + gridDim.x - 1) / gridDim.x;
        const int64_t begin = p.row_begin + (int64_t)blockIdx.x * per_cta, end = min(begin + per_cta, p.row_begin + p.rows);
        for (int64_t r0 = begin; r0 < end; r0 += kMergeThreads) {
            if (threadIdx.x == 0) s_n = 0;
            __syncthreads();
            const int64_t r = r0 + threadIdx.x;
            if (r < end && p.row_status[r] == kRowUndecided) s_found[atomicAdd(&s_n, 1)] = (int)(r - r0);
            __syncthreads();
            const int found = s_n;
            for (int i = 0; i < found; ++i) {  // (in any order: rows do not depend on one another)
                const int64_t row = r0 + s_found[i];
                __syncthreads();
                decide_row(p, row, dyn);
                __syncthreads();
            }
        }
        return;
    }
    if (p.arrivals != nullptr) {
        // Lists that other GPUs write (peer_exchange.cuh): nothing here is read before the row's arrival
        // counter says that every shard's record is complete -- this GPU's own among them, so the kernel
        // before this one is not waited for as a whole, and the kernel after this one may start at once.
        grid_dependents_may_launch();
        __shared__ int s_arrived;
        const int64_t row = p.row_begin + blockIdx.x;
        if (threadIdx.x == 0) s_arrived = wait_until_at_least(p.arrivals + row, p.arrivals_target, p.arrivals_wait_ns) ? 1 : 0;
        __syncthreads();
        if (s_arrived) {
            decide_row(p, row, dyn);
        } else if (threadIdx.x == 0) {
            p.tokens[row] = -1;
            p.log_probs[row] = 0.0f;
            p.row_status[row] = PSX_ROW_DEVICE_TIMEOUT;
            if (p.diag) p.diag[row] = psx_row_diag{0, 0, INFINITY, INFINITY};
        }
        __syncthreads();
        if (p.publish && (int)threadIdx.x < p.peers.world) {  // one thread per rank: the row's 16 bytes, then the count
            const PeerLayout& l = p.peers;
            const int64_t within = row - (int64_t)l.rank * l.rows_per_rank;
            char* block = l.base[threadIdx.x] + l.results_offset + (int64_t)l.rank * peer_results_block_bytes(l.rows_per_rank);
            reinterpret_cast<int64_t*>(block)[within] = p.tokens[row];
            reinterpret_cast<float*>(block + 8 * l.rows_per_rank)[within] = p.log_probs[row];
            reinterpret_cast<int32_t*>(block + 12 * l.rows_per_rank)[within] = p.row_status[row];
            add_release_system(reinterpret_cast<uint32_t*>(l.base[threadIdx.x] + l.flags_offset) + l.rank, 1u);  // (a release)
        }
        grid_dependency_wait();  // (so that this kernel's end still implies the end of the kernel before it)
        return;
    }
    grid_dependency_wait();        // everything this kernel reads was written by the kernel before it
    grid_dependents_may_launch();  // a row pass that follows reads none of this kernel's results
    PSX_MERGE_TIME(1);
    decide_row(p, p.row_begin + blockIdx.x, dyn);
    PSX_MERGE_TIME(2);
}

template <int N>
__global__ void __launch_bounds__(kMergeThreads) merge_rows_warp_kernel(const MergeParams p) {
    extern __shared__ unsigned long long dyn[];
    grid_dependency_wait();        // everything this kernel reads was written by the kernel before it
    grid_dependents_may_launch();
    const int warp = threadIdx.x >> 5;
    const int64_t row = p.row_begin + (int64_t)blockIdx.x * survivor::kRowsPerCta + warp;
    if (row >= p.row_begin + p.rows) return;  // (no barrier in this kernel: a warp may leave)
    survivor::warp_merge_row<N>(p, row, reinterpret_cast<unsigned char*>(dyn) + (size_t)warp * survivor::warp_arena_bytes(p.warp_list_cap));
}

}  // namespace

#ifdef PSX_STAGE_CLOCKS
extern "C" __attribute__((visibility("default"))) int psx_debug_merge_clocks(unsigned long long* out, int n) {
    return (int)cudaMemcpyFromSymbol(out, g_merge_clocks, sizeof(unsigned long long) * n);
}
extern "C" __attribute__((visibility("default"))) int psx_debug_merge_times(unsigned long long* out, int n) {
    return (int)cudaMemcpyFromSymbol(out, g_merge_times, sizeof(unsigned long long) * n);
}
#endif

size_t merge_rows_shared_bytes(int sort_capacity, int gather_capacity, bool overlay) {
    const size_t list = (size_t)sort_capacity * 8, rest = (size_t)sort_capacity * (8 + 8 + 1), gathered = (size_t)gather_capacity * 8;
    return list + (overlay ? (rest > gathered ? rest : gathered) : rest + gathered) + 16;
}

int merge_slot_shift(int parts, int part_cap, int expected) {
    int shift = 0;
    // room for about twice what is expected, inside a list, inside what 16 fetches per thread reach
    while ((1 << shift) < 2 * expected && (2 << shift) <= part_cap && ((long long)parts << (shift + 1)) <= 16 * kMergeThreads) {
        ++shift;
    }
    return shift;
}

cudaError_t configure_merge_rows() { return allow_all_dynamic_shared(merge_rows_kernel); }

bool plan_merge_by_warp(MergeParams& p, int k_need, bool greedy, int expected) {
    p.by_warp = 0;
    if (!greedy && k_need > 64) return false;
    int shift = 0;
    while ((1 << shift) < expected && (2 << shift) <= p.part_cap) ++shift;
    while (shift > 0 && ((long long)p.parts << shift) > 512) --shift;
    if (((long long)p.parts << shift) > 512) return false;
    p.by_warp = 1;
    p.warp_slot_shift = shift;
    p.warp_list_cap = (greedy || k_need <= 32) ? 64 : 128;
    return true;
}

cudaError_t launch_merge_rows(const MergeParams& p, cudaStream_t stream, uint64_t* launched) {
    if (p.rows <= 0) return cudaSuccess;
    // The same condition as the kernel's: the overlaid layout is for plans without a top-k.
    const bool overlay = p.overlay != 0 && p.logits != nullptr && !(p.do_sample && p.top_k > 0 && p.top_k < p.vocab);
    const size_t shared = merge_rows_shared_bytes(p.sort_capacity, p.gather_capacity, overlay);
    MergeParams with_size = p;
    with_size.dyn_bytes = (int32_t)shared;
    with_size.only_undecided = 0;
    // By warps from 256 rows on: a warp takes longer over a row than a block does (about 13 us against 7 on
    // 64 rows of 152 K logits), so few rows are answered sooner by blocks; many rows get through faster by
    // warps (1000 x 49 K, top-k 50: 70 -> 59 us per step; 1024 greedy rows: 47 -> 37 us).
    const bool by_warp = p.by_warp != 0 && p.general != 2 && p.survivor_cols == nullptr && p.arrivals == nullptr && p.rows >= kRowsByWarpFrom;
    if (launched != nullptr) *launched += by_warp ? 2 : 1;
    if (!by_warp) {
        return launch_overlapping(merge_rows_kernel, dim3((unsigned)p.rows), dim3(kMergeThreads), shared, stream, with_size);
    }
    // One warp per row, eight rows per CTA; then the block-per-row kernel over what the warps left undecided.
    const int fetches = (int)((((long long)p.parts << p.warp_slot_shift) + 31) / 32);
    const size_t warp_shared = survivor::warp_arena_bytes(p.warp_list_cap) * survivor::kRowsPerCta;
    const dim3 grid((unsigned)((p.rows + survivor::kRowsPerCta - 1) / survivor::kRowsPerCta));
    cudaError_t e;
    if (fetches <= 1) e = launch_overlapping(merge_rows_warp_kernel<1>, grid, dim3(kMergeThreads), warp_shared, stream, with_size);
    else if (fetches <= 2) e = launch_overlapping(merge_rows_warp_kernel<2>, grid, dim3(kMergeThreads), warp_shared, stream, with_size);
    else if (fetches <= 4) e = launch_overlapping(merge_rows_warp_kernel<4>, grid, dim3(kMergeThreads), warp_shared, stream, with_size);
    else if (fetches <= 8) e = launch_overlapping(merge_rows_warp_kernel<8>, grid, dim3(kMergeThreads), warp_shared, stream, with_size);
    else e = launch_overlapping(merge_rows_warp_kernel<16>, grid, dim3(kMergeThreads), warp_shared, stream, with_size);
    if (e != cudaSuccess) return e;
    with_size.only_undecided = 1;
    const unsigned ctas = (unsigned)(p.rows < 32 ? p.rows : 32);
    return launch_overlapping(merge_rows_kernel, dim3(ctas), dim3(kMergeThreads), shared, stream, with_size);
}

}  // namespace psx
