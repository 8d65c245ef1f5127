// The last kernel of a vocabulary-sharded step over peer memory: waits for every rank's results.
#include "peer_exchange.cuh"

#include "../../include/psx_b200.h"
#include "psx_device.cuh"

namespace psx {

namespace {

__global__ void __launch_bounds__(32) await_results_kernel(const AwaitParams p) {
    // The kernel after this one (the next step's row pass) may start reading its logits at once; what it
    // writes waits for this kernel's end.
    grid_dependents_may_launch();
    const PeerLayout& l = p.layout;
    const int peer = threadIdx.x;
    if (peer < l.world) {
        const int64_t first = (int64_t)peer * l.rows_per_rank;
        const int64_t count = first >= p.rows ? 0 : (p.rows - first < l.rows_per_rank ? p.rows - first : l.rows_per_rank);
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(l.base[l.rank] + l.flags_offset) + peer;
        if (count > 0 && !wait_until_at_least(flag, p.turn * (uint32_t)count, p.wait_limit_ns)) {
            char* block = l.base[l.rank] + l.results_offset + (int64_t)peer * peer_results_block_bytes(l.rows_per_rank);
            int64_t* tokens = reinterpret_cast<int64_t*>(block);
            int32_t* status = reinterpret_cast<int32_t*>(block + 12 * l.rows_per_rank);
            for (int64_t i = 0; i < count; ++i) {
                tokens[i] = -1;
                status[i] = PSX_ROW_DEVICE_TIMEOUT;
            }
        }
    }
    __syncwarp();
    // The next step's packing kernel, already waiting under its row pass, may now overwrite what this
    // step's survivor stages have read (everywhere: every result of the step has been seen here).
    if (threadIdx.x == 0 && p.step_done != nullptr) {
        __threadfence();
        atomicMax(p.step_done, p.step);  // (two steps are in flight: never back)
    }
    grid_dependency_wait();  // (so that this kernel's end still implies the end of the kernels before it)
}

}  // namespace

cudaError_t launch_await_results(const AwaitParams& p, cudaStream_t stream) {
    if (p.layout.world < 1 || p.layout.world > kMaxPeers) return cudaErrorInvalidValue;
    return launch_overlapping(await_results_kernel, dim3(1), dim3(32), 0, stream, p);
}

}  // namespace psx
