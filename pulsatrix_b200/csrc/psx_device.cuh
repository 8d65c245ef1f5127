// Shared device-side definitions of the sm_100a sampling kernels: layouts of the scratch records
// that the row pass hands to the survivor stage, the few float operations whose rounding must
// match the host reference, and small warp/block helpers.
#pragma once

#include <cuda_runtime.h>
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

namespace psx {

// ---- geometry of the row pass ----------------------------------------------------------------
constexpr int kScanThreads = 256;
constexpr int kScanWarps = kScanThreads / 32;
constexpr int kVecPerThread = 16;                            // float4 a thread looks at per pass
constexpr int kPartVecs = kScanThreads * kVecPerThread;      // 4096 vectors = 16384 logits = 64 KB per CTA, three CTAs per SM
constexpr int kPartCap = 1024;                               // candidate slots per part
constexpr int kMergeThreads = 256;

// A candidate is (raw logit bits, column | flags).  The flags say how the survivor stage must
// turn the raw logit into the processed one, with the same float operations as the row pass.
constexpr uint32_t kFlagPenalized = 0x80000000u;
constexpr uint32_t kFlagBanned = 0x40000000u;
constexpr uint32_t kColumnMask = 0x3FFFFFFFu;

// What one part (a contiguous run of columns of one row, scanned by one CTA or, after an
// all-gather, by one GPU) reports besides its candidates.
struct PartStats {
    double raw_tail;      // sum of exp(l - raw_max) over the part's logits that are NOT candidates
    double proc_tail;     // sum of exp(x' - x'_max) over non-candidates that are still alive
    float raw_max;        // max raw logit of the part
    float y_max;          // max processed logit before temperature (-inf when nothing is alive)
    float thr;            // every alive logit >= relax(thr) of this part is a candidate
    uint32_t nonfinite;   // 1 when the part holds a NaN or an infinity
    uint32_t alive_tail;  // non-candidates that are still alive (not banned, not padding)
    uint32_t overflow;    // 1 when the part's candidate list ran out of slots
};

// ---- float operations that must round like the reference's host code ---------------------------

// src/generation.cpp:66 -- negative logits are multiplied, the others divided (-0.0 is divided).
__device__ __forceinline__ float penalize(float l, float penalty) {
    return l < 0.0f ? __fmul_rn(l, penalty) : __fdiv_rn(l, penalty);
}

// Processed logit before temperature from the raw one and the candidate flags.
__device__ __forceinline__ float processed_before_temperature(float l, uint32_t flags, float penalty) {
    if (flags & kFlagBanned) return -INFINITY;
    return (flags & kFlagPenalized) ? penalize(l, penalty) : l;
}

// src/generation.cpp:78 -- one IEEE float divide.
__device__ __forceinline__ float temper(float y, bool apply, float temperature) {
    return apply ? __fdiv_rn(y, temperature) : y;
}

// The float just below q (nextafterf(q, -inf)) in integer arithmetic; -inf and NaN stay as they are.
__device__ __forceinline__ float next_below(float q) {
    const uint32_t b = __float_as_uint(q);
    if (q != q || b == 0xFF800000u) return q;
    if ((b << 1) == 0u) return __uint_as_float(0x80000001u);  // below +-0: the smallest negative subnormal
    return __uint_as_float((b & 0x80000000u) ? b + 1u : b - 1u);
}

// A value t' <= t such that y < t' implies y / T < t / T after rounding: dividing by the
// temperature can map neighbouring floats to the same quotient, and every logit whose quotient
// ties with the threshold's must be kept as a candidate.  Never below -FLT_MAX, so that -inf
// (banned) entries never pass `y >= t'`.  Non-decreasing in t, and one definition for the row pass
// and the survivor stage: a part's relaxed threshold never exceeds the relaxed largest threshold.
__device__ __forceinline__ float relax_threshold(float t, bool apply_temp, float temperature) {
    float r = t;
    if (apply_temp && t > -INFINITY) {
        // With y < t - (|t| 2^-21 + T 2^-147) the exact quotients y / T and t / T are more than
        // |t / T| 2^-21 + 2^-147 apart, which is more than their two rounding errors (2^-24 relative or
        // 2^-150 absolute each): the rounded ones differ too.  No divide needed.
        r = __fsub_rn(t, __fmaf_rn(fabsf(t), 0x1p-21f, __fmul_rn(temperature, 0x1p-147f)));
        if (!(fabsf(t) <= __fmul_rn(temperature, 1e37f))) {
            // Quotients near t / T may overflow, where the argument above ends: take the neighbour of
            // the rounded quotient back through the multiplication as well, and the lower of the two.
            const float q = __fdiv_rn(t, temperature);
            float e = __fmul_rd(temperature, next_below(q));
            if (!(e <= t)) e = (e != e) ? -INFINITY : t;
            r = fminf(r, e);
        }
    }
    return fmaxf(r, -FLT_MAX);
}

// Order-preserving map of finite/infinite floats to uint32; -0.0 and +0.0 share a key because
// the reference's comparisons treat them as equal.
__device__ __forceinline__ uint32_t ordered_key(float x) {
    const uint32_t u = __float_as_uint(x + 0.0f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float from_ordered_key(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

// max of three floats in one instruction (sm_100 has a three-input FMNMX); NaN operands are skipped.
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two independent IEEE single-precision operations in one instruction (sm_100 packed fp32): the same
// results as two scalar ones, half the issue slots.
__device__ __forceinline__ void fma_pair(float& r0, float& r1, float a0, float a1, float b0, float b1, float c0, float c1) {
    asm("{\n\t.reg .b64 a, b, c, d;\n\t"
        "mov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %5};\n\tmov.b64 c, {%6, %7};\n\t"
        "fma.rn.f32x2 d, a, b, c;\n\tmov.b64 {%0, %1}, d;\n\t}"
        : "=f"(r0), "=f"(r1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void add_pair(float& r0, float& r1, float a0, float a1, float b0, float b1) {
    asm("{\n\t.reg .b64 a, b, d;\n\t"
        "mov.b64 a, {%2, %3};\n\tmov.b64 b, {%4, %5};\n\t"
        "add.rn.f32x2 d, a, b;\n\tmov.b64 {%0, %1}, d;\n\t}"
        : "=f"(r0), "=f"(r1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}


// exp2(-r) for the remainder r that a float exponent dropped (|r| is half an ulp of the exponent: 1e-5
// or less for any logit whose exponential matters); the series ends after the square term there.
__device__ __forceinline__ double exp2_of_minus_small(float r) {
    if (fabsf(r) > 1e-4f) return exp2(-(double)r);
    const double x = -(double)r * 0.69314718055994530942;
    return fma(x, fma(x, 0.5, 1.0), 1.0);
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// The row pass and the survivor stage are launched so that a kernel may start while the kernel
// before it in the stream is still running (cudaLaunchAttributeProgrammaticStreamSerialization).
// grid_dependency_wait() returns once that earlier kernel has finished and its writes are
// visible; a kernel calls it before it reads what the earlier kernel wrote and before it writes
// anything the earlier kernel may still read.  Launched the ordinary way, both calls do nothing.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- warp / block helpers ------------------------------------------------------------------------

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

__device__ __forceinline__ uint32_t warp_sum_u32(uint32_t v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// Warp maximum through the integer reduction unit: one REDUX on an order-preserving key instead
// of five shuffle/max pairs.  v must not be NaN.
__device__ __forceinline__ uint32_t monotone_key(float x) {
    const uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float warp_max_redux(float v) {
    return from_ordered_key(__reduce_max_sync(0xFFFFFFFFu, monotone_key(v)));
}

// The kp-th largest (1-based, small kp) of the 32 lane values: take the maximum away kp - 1
// times (one lane each time, the lowest lane among equals), then the maximum of what is left.
__device__ __forceinline__ float warp_kth_largest_small(float v, int kp, int lane) {
    uint32_t key = monotone_key(v);
    for (int i = 1; i < kp; ++i) {
        const uint32_t top = __reduce_max_sync(0xFFFFFFFFu, key);
        const uint32_t holders = __ballot_sync(0xFFFFFFFFu, key == top);
        if (lane == __ffs(holders) - 1) key = 0;
    }
    return from_ordered_key(__reduce_max_sync(0xFFFFFFFFu, key));
}

// The kp-th largest (1-based) of the 32 lane values: a bitonic sort across the lanes, largest
// in lane 0, then a broadcast.
__device__ __forceinline__ float warp_kth_largest(float v, int kp, int lane) {
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            const float o = __shfl_xor_sync(0xFFFFFFFFu, v, j);
            const bool descending_block = (lane & k) == 0;
            const bool lower_lane = (lane & j) == 0;
            v = (lower_lane == descending_block) ? fmaxf(v, o) : fminf(v, o);
        }
    }
    return __shfl_sync(0xFFFFFFFFu, v, kp - 1);
}

// In-place bitonic sort of n_pad (a power of two) 64-bit keys in shared memory by the whole
// block; descending when `descending`.  Ends with a barrier.
__device__ __forceinline__ void block_bitonic_sort(unsigned long long* keys, int n_pad, bool descending) {
    for (int k = 2; k <= n_pad; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < n_pad; i += blockDim.x) {
                const int partner = i ^ j;
                if (partner > i) {
                    const unsigned long long a = keys[i], b = keys[partner];
                    const bool first_block = (i & k) == 0;
                    const bool want_a_larger = (first_block == descending);
                    if (want_a_larger ? (a < b) : (a > b)) {
                        keys[i] = b;
                        keys[partner] = a;
                    }
                }
            }
            __syncthreads();
        }
    }
}

// Lets `kernel` be launched with as much dynamic shared memory as the current device gives a block.
// The limit belongs to the kernel and the device, not to a caller: contexts and host threads that
// need different amounts must not lower it under one another, so it is raised to the most, once.
template <class Kernel>
inline cudaError_t allow_all_dynamic_shared(Kernel kernel) {
    int device = 0, most = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&most, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    if (e != cudaSuccess) return e;
    cudaFuncAttributes attributes;
    e = cudaFuncGetAttributes(&attributes, kernel);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                most - (int)attributes.sharedSizeBytes);
}

// Launches `kernel` so that it may begin while the kernel before it in `stream` is still running
// (see grid_dependency_wait above); PSX_B200_NO_PDL=1 in the environment launches the ordinary way.
template <class Params>
inline cudaError_t launch_overlapping(void (*kernel)(Params), dim3 grid, dim3 block, size_t shared, cudaStream_t stream,
                                      const Params& params) {
    static const bool plain = [] { const char* e = getenv("PSX_B200_NO_PDL"); return e && e[0] == '1'; }();
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = plain ? 0 : 1;
    return cudaLaunchKernelEx(&config, kernel, params);
}

}  // namespace psx
