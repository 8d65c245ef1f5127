// The last kernel of a vocabulary-sharded step over peer memory: every rank's results to every rank.
#include "peer_exchange.cuh"

#include "../../include/psx_b200.h"

namespace psx {

namespace {

constexpr int kPublishThreads = 128;

__global__ void __launch_bounds__(kPublishThreads) publish_results_kernel(const PublishParams p) {
    const PeerLayout& l = p.layout;
    const int peer = blockIdx.x, tid = threadIdx.x;
    const int64_t block_bytes = peer_results_block_bytes(l.rows_per_rank);
    // this rank's block, 16 bytes at a time (the block is a multiple of 16 bytes and 256-byte aligned on both sides)
    const uint4* src = static_cast<const uint4*>(p.block);
    uint4* dst = reinterpret_cast<uint4*>(l.base[peer] + l.results_offset + (int64_t)l.rank * block_bytes);
    for (int64_t i = tid; i < block_bytes / 16; i += kPublishThreads) dst[i] = src[i];
    __syncthreads();
    if (tid == 0) {
        __threadfence_system();  // the whole CTA's stores before the flag
        store_release_system(reinterpret_cast<uint32_t*>(l.base[peer] + l.flags_offset) + l.rank, p.step);
    }
    // ... and the peer's block here
    __shared__ int s_arrived;
    if (tid == 0) {
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(l.base[l.rank] + l.flags_offset) + peer;
        s_arrived = wait_until_at_least(flag, p.step, p.wait_limit_ns) ? 1 : 0;
    }
    __syncthreads();
    if (!s_arrived) {
        char* block = l.base[l.rank] + l.results_offset + (int64_t)peer * block_bytes;
        int64_t* tokens = reinterpret_cast<int64_t*>(block);
        int32_t* status = reinterpret_cast<int32_t*>(block + 12 * l.rows_per_rank);
        for (int64_t i = tid; i < l.rows_per_rank; i += kPublishThreads) {
            tokens[i] = -1;
            status[i] = PSX_ROW_DEVICE_TIMEOUT;
        }
    }
}

}  // namespace

cudaError_t launch_publish_results(const PublishParams& p, cudaStream_t stream) {
    if (p.layout.world < 1 || p.layout.world > kMaxPeers) return cudaErrorInvalidValue;
    publish_results_kernel<<<(unsigned)p.layout.world, kPublishThreads, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace psx
