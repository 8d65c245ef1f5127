// A plain read-only pass over a buffer: 128-bit streaming loads and a max in registers, nothing
// else.  It exists so that benchmarks can measure, on the same inputs and with the same launch
// cadence as the row pass, what a kernel that only READS those bytes achieves -- the practical
// ceiling for a batch of a given size (launch and ramp-up are a visible share of a ~10 us kernel).
#include "../../include/psx_b200.h"

#include <string>

#include <cuda_runtime.h>

namespace psx_internal {
psx_status set_error(psx_status code, const std::string& message);  // c_abi.cu
}

namespace {

constexpr int kThreads = 512, kPerThread = 4;

__global__ void __launch_bounds__(kThreads) read_floor_kernel(const float4* __restrict__ src, size_t vectors,
                                                              float* sink) {
    const size_t base = (size_t)blockIdx.x * kThreads * kPerThread;
    float4 d[kPerThread];
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {
        const size_t v = base + (size_t)j * kThreads + threadIdx.x;
        d[j] = v < vectors ? __ldcs(src + v) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float m = -3.0e38f;
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) m = fmaxf(m, fmaxf(fmaxf(d[j].x, d[j].y), fmaxf(d[j].z, d[j].w)));
    if (m == 1.2345e38f) *sink = m;  // keeps the loads alive; practically never true
}

}  // namespace

extern "C" psx_status psx_b200_read_only_pass(void* stream, const void* data, size_t bytes, float* sink) {
    if (!data || !sink || (reinterpret_cast<uintptr_t>(data) % 16) != 0) {
        return psx_internal::set_error(PSX_ERR_BAD_ARGUMENT, "psx_b200_read_only_pass: data must be 16-byte aligned");
    }
    const size_t vectors = bytes / 16;
    if (vectors == 0) return PSX_OK;
    const size_t per_block = (size_t)kThreads * kPerThread;
    const size_t blocks = (vectors + per_block - 1) / per_block;
    if (blocks > 0x7FFFFFFFull) return psx_internal::set_error(PSX_ERR_UNSUPPORTED, "psx_b200_read_only_pass: buffer too large");
    read_floor_kernel<<<(unsigned)blocks, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float4*>(data), vectors, sink);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return psx_internal::set_error(PSX_ERR_CUDA, std::string("CUDA error: ") + cudaGetErrorString(e));
    return PSX_OK;
}
