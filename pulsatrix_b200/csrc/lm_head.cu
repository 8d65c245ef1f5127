// The language-model head on the device: logits[m][j] = sum_p hidden[m][p] * w_j[p], the step right
// before the sampling path (src/tied_lm_head_module.cpp:31-53: gemm_ex(hidden, E^T); an untied head
// is a bias-free Linear, src/linear_module.cpp: gemm(hidden, W)).
//
// Exact by construction: the reference's CPU backend forms every logit as one float accumulator
// that takes the products in ascending p, each product rounded, then the sum rounded
// (src/cpu_backend.cpp:188-196 and GemmRowRange; its x86-64 build has no fused multiply-add).  A
// thread here owns one vocabulary entry and up to 64 rows of hidden states, and does exactly that:
// __fmul_rn, then __fadd_rn, p ascending.  The logits are therefore the reference's bit for bit,
// and so is every token drawn from them.  (Tensor cores would round differently -- TF32 products,
// tree-shaped sums -- so they are not used here.  Neither are the packed mul.rn.f32x2 / add.rn.f32x2: a
// build that paired two rows per instruction gave logits two ulps away from the scalar operations'.)
//
// Bound: at decode sizes (a few rows) by HBM -- the weight matrix is read once, 4 * vocab * d
// bytes; from about 16 rows up by the FP32 pipes (two instructions per multiply-add).
// Two weight layouts:
//   - token-major (vocab x d, the tied embedding): a CTA of 128 threads stages 128 entries x 32
//     features at a time in shared memory with cp.async (16-byte pieces, two stages), a thread
//     reads its own entry's row from there;
//   - feature-major (d x vocab, an untied Linear): consecutive threads read consecutive floats.
#include "lm_head.cuh"

#include <cuda_pipeline_primitives.h>

namespace psx {

namespace {

constexpr int kHeadThreads = 128;  // vocabulary entries per CTA, one per thread
constexpr int kHeadChunk = 32;     // features per stage
constexpr int kHeadPitch = 36;     // floats per staged row: 16-byte aligned, and 128-bit reads of eight
                                   // consecutive rows fall into distinct banks

template <int MT>
__global__ void __launch_bounds__(kHeadThreads) head_token_major_kernel(const float* __restrict__ hidden,
                                                                        const float* __restrict__ weight,
                                                                        float* __restrict__ logits, int rows, int64_t d,
                                                                        int64_t vocab, int64_t row_stride, int vector_ok) {
    __shared__ __align__(16) float s_w[2][kHeadThreads * kHeadPitch];
    __shared__ __align__(16) float s_h[kHeadChunk * MT];  // [feature][row], of the chunk at work
    const int tid = threadIdx.x;
    const int64_t j0 = (int64_t)blockIdx.x * kHeadThreads;
    const int64_t j = j0 + tid;
    const int chunks = (int)((d + kHeadChunk - 1) / kHeadChunk);

    auto stage = [&](int c, int buf) {
        const int64_t k0 = (int64_t)c * kHeadChunk;
        const int kc = (int)min((int64_t)kHeadChunk, d - k0);
        if (vector_ok && kc == kHeadChunk) {
            // 128 rows of 128 bytes: eight 16-byte pieces each; consecutive threads take one row's pieces
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int q = it * kHeadThreads + tid, r = q >> 3, seg = q & 7;
                const int64_t jr = min(j0 + r, vocab - 1);  // (entries past the vocabulary read the last one; never stored)
                __pipeline_memcpy_async(&s_w[buf][r * kHeadPitch + seg * 4], weight + jr * d + k0 + seg * 4, 16);
            }
        } else {
            for (int q = tid; q < kHeadThreads * kHeadChunk; q += kHeadThreads) {
                const int r = q >> 5, p = q & 31;
                const int64_t jr = min(j0 + r, vocab - 1);
                s_w[buf][r * kHeadPitch + p] = p < kc ? weight[jr * d + k0 + p] : 0.0f;
            }
        }
        __pipeline_commit();
    };
    auto stage_hidden = [&](int c) {  // (nobody reads the chunk before any more: the loop ends with a barrier)
        const int64_t k0 = (int64_t)c * kHeadChunk;
        const int kc = (int)min((int64_t)kHeadChunk, d - k0);
        for (int q = tid; q < kHeadChunk * MT; q += kHeadThreads) {
            const int p = q / MT, m = q % MT;
            s_h[q] = (m < rows && p < kc) ? hidden[(int64_t)m * d + k0 + p] : 0.0f;
        }
    };

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.0f;
    stage(0, 0);
    for (int c = 0; c < chunks; ++c) {
        const int buf = c & 1;
        if (c + 1 < chunks) stage(c + 1, buf ^ 1);
        stage_hidden(c);
        __pipeline_wait_prior(c + 1 < chunks ? 1 : 0);
        __syncthreads();
        const int kc = (int)min((int64_t)kHeadChunk, d - (int64_t)c * kHeadChunk);
        const float* wrow = &s_w[buf][tid * kHeadPitch];
        auto take = [&](int p, float w) {  // acc[m] += hidden[m][p] * w, each step rounded (src/cpu_backend.cpp:193)
            if (MT >= 4) {
#pragma unroll
                for (int m = 0; m < MT; m += 4) {
                    const float4 h = *reinterpret_cast<const float4*>(&s_h[p * MT + m]);
                    acc[m] = __fadd_rn(acc[m], __fmul_rn(h.x, w));
                    acc[m + 1] = __fadd_rn(acc[m + 1], __fmul_rn(h.y, w));
                    acc[m + 2] = __fadd_rn(acc[m + 2], __fmul_rn(h.z, w));
                    acc[m + 3] = __fadd_rn(acc[m + 3], __fmul_rn(h.w, w));
                }
            } else {
#pragma unroll
                for (int m = 0; m < MT; ++m) acc[m] = __fadd_rn(acc[m], __fmul_rn(s_h[p * MT + m], w));
            }
        };
        if (kc == kHeadChunk) {
#pragma unroll
            for (int p4 = 0; p4 < kHeadChunk / 4; ++p4) {
                const float4 w = *reinterpret_cast<const float4*>(wrow + 4 * p4);
                take(4 * p4, w.x);
                take(4 * p4 + 1, w.y);
                take(4 * p4 + 2, w.z);
                take(4 * p4 + 3, w.w);
            }
        } else {  // the last, shorter chunk: no padded products (they could turn a -0 sum into +0)
            for (int p = 0; p < kc; ++p) take(p, wrow[p]);
        }
        __syncthreads();
    }
    if (j < vocab) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < rows) logits[(int64_t)m * row_stride + j] = acc[m];
        }
    }
}

template <int MT>
__global__ void __launch_bounds__(kHeadThreads) head_feature_major_kernel(const float* __restrict__ hidden,
                                                                          const float* __restrict__ weight,
                                                                          float* __restrict__ logits, int rows, int64_t d,
                                                                          int64_t vocab, int64_t row_stride) {
    __shared__ __align__(16) float s_h[kHeadChunk * MT];  // [feature][row]
    const int tid = threadIdx.x;
    const int64_t j = (int64_t)blockIdx.x * kHeadThreads + tid;
    const int64_t jr = min(j, vocab - 1);
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.0f;
    for (int64_t k0 = 0; k0 < d; k0 += kHeadChunk) {
        const int kc = (int)min((int64_t)kHeadChunk, d - k0);
        __syncthreads();
        for (int q = tid; q < kHeadChunk * MT; q += kHeadThreads) {
            const int p = q / MT, m = q % MT;
            s_h[q] = (m < rows && p < kc) ? hidden[(int64_t)m * d + k0 + p] : 0.0f;
        }
        float w[kHeadChunk];
#pragma unroll
        for (int p = 0; p < kHeadChunk; ++p) w[p] = p < kc ? weight[(k0 + p) * vocab + jr] : 0.0f;  // all loads in flight together
        __syncthreads();
#pragma unroll
        for (int p = 0; p < kHeadChunk; ++p) {
            if (p < kc) {
#pragma unroll
                for (int m = 0; m < MT; ++m) acc[m] = __fadd_rn(acc[m], __fmul_rn(s_h[p * MT + m], w[p]));
            }
        }
    }
    if (j < vocab) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < rows) logits[(int64_t)m * row_stride + j] = acc[m];
        }
    }
}

template <int MT>
cudaError_t launch_group(const float* hidden, const float* weight, float* logits, int rows, int64_t d, int64_t vocab,
                         int64_t row_stride, bool token_major, cudaStream_t stream) {
    const unsigned blocks = (unsigned)((vocab + kHeadThreads - 1) / kHeadThreads);
    if (token_major) {
        const bool vector_ok = d % 4 == 0 && reinterpret_cast<uintptr_t>(weight) % 16 == 0;
        head_token_major_kernel<MT><<<blocks, kHeadThreads, 0, stream>>>(hidden, weight, logits, rows, d, vocab, row_stride,
                                                                        vector_ok ? 1 : 0);
    } else {
        head_feature_major_kernel<MT><<<blocks, kHeadThreads, 0, stream>>>(hidden, weight, logits, rows, d, vocab, row_stride);
    }
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_lm_head(const float* hidden, int64_t rows, int64_t d, const float* weight, int64_t vocab, bool token_major,
                           float* logits, int64_t row_stride, cudaStream_t stream) {
    if (rows <= 0 || vocab <= 0) return cudaSuccess;
    if (d <= 0 || (vocab + kHeadThreads - 1) / kHeadThreads > 0x7FFFFFFF) return cudaErrorInvalidValue;
    // Rows go through in groups of up to 64 (a thread keeps one accumulator per row); every group reads
    // the weights once.
    for (int64_t m0 = 0; m0 < rows; m0 += 64) {
        const int group = (int)min((int64_t)64, rows - m0);
        const float* h = hidden + m0 * d;
        float* out = logits + m0 * row_stride;
        cudaError_t e;
        if (group <= 1) e = launch_group<1>(h, weight, out, group, d, vocab, row_stride, token_major, stream);
        else if (group <= 2) e = launch_group<2>(h, weight, out, group, d, vocab, row_stride, token_major, stream);
        else if (group <= 4) e = launch_group<4>(h, weight, out, group, d, vocab, row_stride, token_major, stream);
        else if (group <= 8) e = launch_group<8>(h, weight, out, group, d, vocab, row_stride, token_major, stream);
        else if (group <= 16) e = launch_group<16>(h, weight, out, group, d, vocab, row_stride, token_major, stream);
        else if (group <= 32) e = launch_group<32>(h, weight, out, group, d, vocab, row_stride, token_major, stream);
        else e = launch_group<64>(h, weight, out, group, d, vocab, row_stride, token_major, stream);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace psx
