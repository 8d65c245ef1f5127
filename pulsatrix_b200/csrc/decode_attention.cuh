// Launch interface of the attention over the KV cache (decode_attention.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace psx {

struct AttentionParams {
    const float* q;         // (batch, heads, q_len, head_dim): the new positions' queries
    const float* keys;      // (batch, kv_heads, max_len, head_dim): the cache, positions 0 .. total - 1 valid
    const float* values;    // likewise
    const float* key_keep;  // (batch, total), 0 = padding; may be null
    float* context;         // (batch, heads, q_len, head_dim)
    float* partial;         // scratch for splits > 1: (batch * heads * q_len, splits, head_dim + 2)
    int32_t* status;        // device; bit 0 is set when a bounded wait for a copy ran out; may be null
    int64_t batch, total, max_len;
    int64_t offset;         // positions cached before the new ones (total = offset + q_len)
    int64_t window;         // sliding window of a causal mask; 0: none
    int32_t heads, kv_heads, group, q_len, head_dim;
    int32_t causal;
    int32_t splits;         // slices of the cached positions, each a CTA of its own
    float scale;            // the score scale (1 / sqrt(head_dim) unless the model says otherwise)
    uint64_t wait_limit_ns;
};

int attention_rows_padded(int rows);                              // group * q_len rounded up to 1, 2, 4 or 8
size_t attention_shared_bytes(int rows_padded, int head_dim);     // dynamic shared memory of a CTA
int attention_splits(int64_t batch_kv, int64_t total, int sm_count, int head_dim);
size_t attention_partial_bytes(const AttentionParams& p);
// cudaErrorInvalidValue: more than 8 query rows per kv head, or a head dimension that is not a multiple
// of 4 up to 256.
cudaError_t launch_decode_attention(const AttentionParams& p, cudaStream_t stream);

}  // namespace psx
