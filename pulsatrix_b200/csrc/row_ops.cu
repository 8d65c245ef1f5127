// Row primitives beside the sampling path: softmax_rows, logsumexp_rows and gather_rows of the
// reference's DeviceBackend (include/pulsatrix/device_backend.hpp:456,465,596; CPU semantics
// src/cpu_backend.cpp:292-338,459-466; the reference's CUDA kernels run one thread per row,
// src/gpu_kernels.cuh:315-365, or one thread per element, :665).
//
// softmax / logsumexp read every element once and (softmax) write it once:
//   - a row of at most 1024 columns is one warp's: 32 values per lane in registers;
//   - a longer row is a thread-block cluster's: each of up to eight CTAs holds 32,768 columns in
//     registers (64 per thread), and the row's maximum and sum meet in distributed shared memory;
//   - beyond 262,144 columns one CTA walks the row three times.
// Float arithmetic like the reference's: exp(x - max) as one ex2 of (x - max) * log2(e) (relative
// error below 1e-5, against the reference's CPU/GPU tolerance of 1e-4), float sums in a fixed tree
// (the same input gives the same bits; the reference's sequential sum differs from it by rounding
// only), y = e / sum, lse = max + logf(sum).
#include <cooperative_groups.h>

#include "row_ops.cuh"

namespace psx {

namespace {

namespace cg = cooperative_groups;

constexpr int kWarpRowCols = 1024;      // the widest row one warp takes
constexpr int kCtaThreads = 512;
constexpr int kCtaVecs = 16;            // float4 per thread
constexpr int kCtaCols = kCtaThreads * kCtaVecs * 4;  // 32,768
constexpr int kMaxCluster = 8;

__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// ---- one warp per row ------------------------------------------------------------------------------
template <bool kSoftmax>
__global__ void __launch_bounds__(256) warp_rows_kernel(const float* __restrict__ in, float* out, size_t rows, size_t cols) {
    const size_t row = (size_t)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float* x = in + row * cols;
    float v[kWarpRowCols / 32];
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < kWarpRowCols / 32; ++k) {
        const size_t j = (size_t)k * 32 + lane;
        v[k] = j < cols ? x[j] : -INFINITY;
        m = fmaxf(m, v[k]);
    }
    m = warp_max_f(m);
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < kWarpRowCols / 32; ++k) {
        const size_t j = (size_t)k * 32 + lane;
        v[k] = j < cols ? __expf(v[k] - m) : 0.0f;
        s += v[k];
    }
    s = warp_sum_f(s);
    if (kSoftmax) {
        float* y = out + row * cols;
#pragma unroll
        for (int k = 0; k < kWarpRowCols / 32; ++k) {
            const size_t j = (size_t)k * 32 + lane;
            if (j < cols) y[j] = v[k] / s;
        }
    } else if (lane == 0) {
        out[row] = m + logf(s);
    }
}

// ---- one cluster per row ---------------------------------------------------------------------------
// Block-wide max / sum in a fixed order; `scratch` holds one float per warp.
__device__ __forceinline__ float block_max_f(float v, float* scratch) {
    v = warp_max_f(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = scratch[0];
#pragma unroll
    for (int w = 1; w < kCtaThreads / 32; ++w) r = fmaxf(r, scratch[w]);
    return r;
}
__device__ __forceinline__ float block_sum_f(float v, float* scratch) {
    v = warp_sum_f(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.0f;
#pragma unroll
    for (int w = 0; w < kCtaThreads / 32; ++w) r += scratch[w];
    return r;
}

template <bool kSoftmax, int kVecs>
__global__ void __launch_bounds__(kCtaThreads) cluster_rows_kernel(const float* __restrict__ in, float* out, size_t rows,
                                                                     size_t cols, int vector_ok) {
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned ctas = cluster.num_blocks(), rank = cluster.block_rank();
    const size_t row = blockIdx.x / ctas;
    __shared__ float s_warp[kCtaThreads / 32];
    __shared__ float s_share[2];  // this CTA's maximum and sum, read by the others of the cluster
    const int tid = threadIdx.x;
    // the CTA's slice of the row: whole float4 vectors, the same count for every CTA but the last
    const size_t vecs = (cols + 3) / 4, per = (vecs + ctas - 1) / ctas;
    const size_t begin = min((size_t)rank * per * 4, cols), end = min(begin + per * 4, cols);
    const float* x = in + row * cols;
    float v[kVecs * 4];
    float m = -INFINITY;
    if (vector_ok) {  // rows start on 16-byte boundaries: cols % 4 == 0 and an aligned base
#pragma unroll
        for (int k = 0; k < kVecs; ++k) {
            const size_t j = begin + ((size_t)k * kCtaThreads + tid) * 4;
            float4 d = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            if (j < end) d = *reinterpret_cast<const float4*>(x + j);
            v[4 * k] = d.x; v[4 * k + 1] = d.y; v[4 * k + 2] = d.z; v[4 * k + 3] = d.w;
            m = fmaxf(fmaxf(m, fmaxf(d.x, d.y)), fmaxf(d.z, d.w));
        }
    } else {
#pragma unroll
        for (int k = 0; k < kVecs * 4; ++k) {
            const size_t j = begin + (size_t)k * kCtaThreads + tid;
            v[k] = j < end ? x[j] : -INFINITY;
            m = fmaxf(m, v[k]);
        }
    }
    m = block_max_f(m, s_warp);
    if (ctas > 1) {
        if (tid == 0) s_share[0] = m;
        cluster.sync();
        for (unsigned r = 0; r < ctas; ++r) m = fmaxf(m, *cluster.map_shared_rank(&s_share[0], r));
    }
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < kVecs * 4; ++k) {
        v[k] = __expf(v[k] - m);  // (slots past the slice hold -inf: they give 0)
        s += v[k];
    }
    s = block_sum_f(s, s_warp);
    if (ctas > 1) {
        if (tid == 0) s_share[1] = s;
        cluster.sync();
        s = 0.0f;
        for (unsigned r = 0; r < ctas; ++r) s += *cluster.map_shared_rank(&s_share[1], r);
        cluster.sync();  // nobody leaves while its shared memory may still be read
    }
    if (kSoftmax) {
        float* y = out + row * cols;
        if (vector_ok) {
#pragma unroll
            for (int k = 0; k < kVecs; ++k) {
                const size_t j = begin + ((size_t)k * kCtaThreads + tid) * 4;
                if (j < end) {
                    *reinterpret_cast<float4*>(y + j) = make_float4(v[4 * k] / s, v[4 * k + 1] / s, v[4 * k + 2] / s, v[4 * k + 3] / s);
                }
            }
        } else {
#pragma unroll
            for (int k = 0; k < kVecs * 4; ++k) {
                const size_t j = begin + (size_t)k * kCtaThreads + tid;
                if (j < end) y[j] = v[k] / s;
            }
        }
    } else if (rank == 0 && tid == 0) {
        out[row] = m + logf(s);
    }
}

// ---- rows beyond a cluster's reach: one CTA, three walks -----------------------------------------------
template <bool kSoftmax>
__global__ void __launch_bounds__(kCtaThreads) long_rows_kernel(const float* in, float* out, size_t rows, size_t cols) {
    __shared__ float s_warp[kCtaThreads / 32];
    const size_t row = blockIdx.x;
    const float* x = in + row * cols;
    float m = -INFINITY;
    for (size_t j = threadIdx.x; j < cols; j += kCtaThreads) m = fmaxf(m, x[j]);
    m = block_max_f(m, s_warp);
    float s = 0.0f;
    for (size_t j = threadIdx.x; j < cols; j += kCtaThreads) s += __expf(x[j] - m);
    s = block_sum_f(s, s_warp);
    if (kSoftmax) {
        float* y = out + row * cols;
        for (size_t j = threadIdx.x; j < cols; j += kCtaThreads) y[j] = __expf(x[j] - m) / s;  // (out may alias in: element by element)
    } else if (threadIdx.x == 0) {
        out[row] = m + logf(s);
    }
}

template <bool kSoftmax>
cudaError_t launch_rows(const float* in, float* out, size_t rows, size_t cols, cudaStream_t stream) {
    if (rows == 0 || cols == 0) return cudaSuccess;
    if (rows > 0x7FFFFFFFull / kMaxCluster) return cudaErrorInvalidConfiguration;
    if (cols <= (size_t)kWarpRowCols) {
        const unsigned blocks = (unsigned)((rows + 7) / 8);
        warp_rows_kernel<kSoftmax><<<blocks, 256, 0, stream>>>(in, out, rows, cols);
        return cudaGetLastError();
    }
    if (cols > (size_t)kCtaCols * kMaxCluster) {
        long_rows_kernel<kSoftmax><<<(unsigned)rows, kCtaThreads, 0, stream>>>(in, out, rows, cols);
        return cudaGetLastError();
    }
    const unsigned ctas = (unsigned)((cols + kCtaCols - 1) / kCtaCols);
    const bool aligned = cols % 4 == 0 && reinterpret_cast<uintptr_t>(in) % 16 == 0 &&
                         (!kSoftmax || reinterpret_cast<uintptr_t>(out) % 16 == 0);
    // a float4 slice per thread needs per-CTA slices of at most kCtaCols columns: true by the choice of `ctas`
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)rows * ctas);
    config.blockDim = dim3(kCtaThreads);
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = ctas;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    // the fewest vectors per thread that cover a CTA's slice
    const size_t slice = ((cols + 3) / 4 + ctas - 1) / ctas;  // float4 vectors
    const int vec_ok = aligned ? 1 : 0;
    if (slice <= (size_t)kCtaThreads * 2) return cudaLaunchKernelEx(&config, cluster_rows_kernel<kSoftmax, 2>, in, out, rows, cols, vec_ok);
    if (slice <= (size_t)kCtaThreads * 4) return cudaLaunchKernelEx(&config, cluster_rows_kernel<kSoftmax, 4>, in, out, rows, cols, vec_ok);
    if (slice <= (size_t)kCtaThreads * 8) return cudaLaunchKernelEx(&config, cluster_rows_kernel<kSoftmax, 8>, in, out, rows, cols, vec_ok);
    return cudaLaunchKernelEx(&config, cluster_rows_kernel<kSoftmax, kCtaVecs>, in, out, rows, cols, vec_ok);
}

// ---- gather_rows -----------------------------------------------------------------------------------------
// One CTA per output row; 128-bit copies when the rows allow it.
__global__ void __launch_bounds__(256) gather_rows_kernel(const float* __restrict__ table, const float* __restrict__ indices,
                                                          float* __restrict__ out, size_t count, size_t dim, int vector_ok) {
    for (size_t i = blockIdx.x; i < count; i += gridDim.x) {
        const float* row = table + (size_t)indices[i] * dim;  // whole-number floats, as the reference passes them
        float* dst = out + i * dim;
        if (vector_ok) {
            for (size_t d = threadIdx.x; d < dim / 4; d += blockDim.x) {
                reinterpret_cast<float4*>(dst)[d] = reinterpret_cast<const float4*>(row)[d];
            }
        } else {
            for (size_t d = threadIdx.x; d < dim; d += blockDim.x) dst[d] = row[d];
        }
    }
}

}  // namespace

cudaError_t launch_softmax_rows(const float* in, float* out, size_t rows, size_t cols, cudaStream_t stream) {
    return launch_rows<true>(in, out, rows, cols, stream);
}

cudaError_t launch_logsumexp_rows(const float* in, float* out, size_t rows, size_t cols, cudaStream_t stream) {
    return launch_rows<false>(in, out, rows, cols, stream);
}

cudaError_t launch_gather_rows(const float* table, const float* indices, float* out, size_t count, size_t dim,
                               cudaStream_t stream) {
    if (count == 0 || dim == 0) return cudaSuccess;
    const bool aligned = dim % 4 == 0 && reinterpret_cast<uintptr_t>(table) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
    const unsigned blocks = (unsigned)(count < 65535u * 16u ? count : 65535u * 16u);
    gather_rows_kernel<<<blocks, 256, 0, stream>>>(table, indices, out, count, dim, aligned ? 1 : 0);
    return cudaGetLastError();
}

}  // namespace psx
