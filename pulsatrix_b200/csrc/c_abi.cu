// The C ABI (include/psx_b200.h): argument checks with the reference's own error texts, scratch
// management, launch planning and the kernel launches.  No computation happens on the host and
// there is no fallback: every entry point that computes needs the CUDA device of its context.
#include "../../include/psx_b200.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "lm_head.cuh"
#include "merge_rows.cuh"
#include "peer_exchange.cuh"
#include "decode_attention.cuh"
#include "process_rows.cuh"
#include "row_ops.cuh"
#include "sample_plan.cuh"
#include "scan_rows.cuh"
#include "shard_records.cuh"
#include "topk_rows.cuh"

namespace {

thread_local std::string g_error;

psx_status fail(psx_status code, std::string message) {
    g_error = std::move(message);
    return code;
}

// Same text as the reference's PULSATRIX_CUDA_CHECK (include/pulsatrix/cuda_check.hpp:24-32).
#define PSX_CUDA(call)                                                                                   \
    do {                                                                                                 \
        const cudaError_t psx_cuda_result = (call);                                                      \
        if (psx_cuda_result != cudaSuccess) {                                                            \
            return fail(PSX_ERR_CUDA, std::string("CUDA error: ") + cudaGetErrorString(psx_cuda_result) + \
                                          " at " __FILE__ ":" + std::to_string(__LINE__));               \
        }                                                                                                \
    } while (0)

struct Buffer {
    void* ptr = nullptr;
    size_t bytes = 0;
};

}  // namespace

// For the library's other translation units: record an error where psx_b200_last_error() finds it.
namespace psx_internal {
psx_status set_error(psx_status code, const std::string& message) { return fail(code, message); }
}

struct psx_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    uint64_t launches = 0;
    bool merge_configured = false;
    bool scan_configured = false;
    // Row-pass scratch, twice: successive sampling calls alternate between the two sets, so that the row
    // pass of one call never writes what the survivor stage of the call before it is still reading
    // (see ScanParams::wait_before_writes).
    Buffer stats[2], part_counts[2], candidates[2];
    int scratch_set = 0;
    Buffer banned, sort_keys, head_logits, attention_partial;
    // ProcessLogits: the surviving set between the survivor stage and the write-back, dummy draw outputs
    Buffer surv_cols, surv_vals, surv_counts, pl_tokens, pl_log_probs, pl_status;
    // staging of the host entry point
    Buffer h_logits, h_history, h_offsets, h_uniforms, h_tokens, h_log_probs, h_status, h_diag;
    // staging of the sharded path
    Buffer shard_uniform_scratch;
    // optional per-kernel timing: (before row pass, between, after survivor stage) per call
    bool timing = false;
    std::vector<cudaEvent_t> timing_events;
    bool inputs_ready = false;  // psx_b200_ctx_inputs_are_ready
    uint64_t wait_limit_ns = psx::kDefaultWaitLimitNs;  // psx_b200_ctx_set_wait_limit
    bool test_short_copy = false;                       // psx_b200_test_short_copy
};

namespace {

psx_status reserve(Buffer& b, size_t bytes) {
    if (bytes <= b.bytes) return PSX_OK;
    if (b.ptr) PSX_CUDA(cudaFree(b.ptr));
    b.ptr = nullptr;
    b.bytes = 0;
    const size_t want = bytes + bytes / 4 + 256;
    PSX_CUDA(cudaMalloc(&b.ptr, want));
    b.bytes = want;
    return PSX_OK;
}

// src/generation.cpp:19-38, with the reference's messages.
psx_status check_config(const psx_sampling_config* c) {
    if (!c) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: config is null");
    if (c->min_new_tokens < 0) {
        return fail(PSX_ERR_BAD_ARGUMENT, "GenerationConfig: max_new_tokens and min_new_tokens must not be negative");
    }
    if (!(c->temperature > 0.0f) || std::isinf(c->temperature)) {
        return fail(PSX_ERR_BAD_ARGUMENT, "GenerationConfig: temperature must be positive and finite");
    }
    if (c->top_k < 0) return fail(PSX_ERR_BAD_ARGUMENT, "GenerationConfig: top_k must not be negative");
    if (!(c->top_p > 0.0f && c->top_p <= 1.0f)) {
        return fail(PSX_ERR_BAD_ARGUMENT, "GenerationConfig: top_p must be in (0, 1]");
    }
    if (!(c->min_p >= 0.0f && c->min_p <= 1.0f)) {
        return fail(PSX_ERR_BAD_ARGUMENT, "GenerationConfig: min_p must be in [0, 1]");
    }
    if (!(c->repetition_penalty > 0.0f) || std::isinf(c->repetition_penalty)) {
        return fail(PSX_ERR_BAD_ARGUMENT, "GenerationConfig: repetition_penalty must be positive and finite");
    }
    if (c->num_eos_token_ids < 0 || (c->num_eos_token_ids > 0 && !c->eos_token_ids)) {
        return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: eos_token_ids is null");
    }
    return PSX_OK;
}

using psx::Plan;

// The survivor stage holds one row's candidates in shared memory.
psx_status configure_merge(psx_ctx* ctx, const Plan& plan, int parts) {
    if (parts > 16 * psx::kMergeThreads) {
        return fail(PSX_ERR_UNSUPPORTED, "psx_b200: rows wider than 64M logits per GPU are not supported");
    }
    (void)plan;
    if (ctx->merge_configured) return PSX_OK;
    PSX_CUDA(psx::configure_merge_rows());
    ctx->merge_configured = true;
    return PSX_OK;
}

// Fills the part of ScanParams that depends on the settings; uploads the banned ids.
psx_status prepare_scan(psx_ctx* ctx, cudaStream_t stream, const psx_sampling_config* c, const Plan& plan,
                        psx::ScanParams& sp) {
    if (!ctx->scan_configured) {  // a part's ring is more shared memory than a kernel gets without asking
        PSX_CUDA(psx::configure_scan_rows());
        ctx->scan_configured = true;
    }
    psx::fill_scan_settings(sp, c, plan);
    sp.inputs_ready = ctx->inputs_ready ? 1 : 0;
    sp.wait_limit_ns = ctx->wait_limit_ns;
    sp.test_short_copy = ctx->test_short_copy ? 1 : 0;
    if (c->num_new_tokens < c->min_new_tokens && c->num_eos_token_ids > 0) {  // src/generation.cpp:69
        if (c->num_eos_token_ids > (1 << 20)) return fail(PSX_ERR_UNSUPPORTED, "psx_b200: too many eos ids");
        const size_t bytes = (size_t)c->num_eos_token_ids * sizeof(int64_t);
        if (psx_status s = reserve(ctx->banned, bytes)) return s;
        PSX_CUDA(cudaMemcpyAsync(ctx->banned.ptr, c->eos_token_ids, bytes, cudaMemcpyHostToDevice, stream));
        sp.banned_ids = static_cast<const int64_t*>(ctx->banned.ptr);
        sp.num_banned = (int32_t)c->num_eos_token_ids;
    }
    return PSX_OK;
}

psx_status reserve_scan_scratch(psx_ctx* ctx, int64_t rows, const Plan& plan, psx::ScanParams& sp, int set = 0) {
    const size_t parts = (size_t)rows * plan.parts;
    if (psx_status s = reserve(ctx->stats[set], parts * sizeof(psx::PartStats))) return s;
    if (psx_status s = reserve(ctx->part_counts[set], parts * sizeof(uint32_t))) return s;
    if (psx_status s = reserve(ctx->candidates[set], parts * psx::kPartCap * sizeof(uint2))) return s;
    sp.stats = static_cast<psx::PartStats*>(ctx->stats[set].ptr);
    sp.part_counts = static_cast<uint32_t*>(ctx->part_counts[set].ptr);
    sp.candidates = static_cast<uint2*>(ctx->candidates[set].ptr);
    return PSX_OK;
}

// What a failed row means, in the reference's words where it has them (src/generation.cpp:130,137).
const char* row_failure_text(int32_t status) {
    switch (status) {
        case PSX_ROW_NON_FINITE: return "Generate: the model returned a non-finite logit";
        case PSX_ROW_ALL_REMOVED: return "Generate: every token was removed";
        case PSX_ROW_DEVICE_TIMEOUT: return "psx_b200: a device-side wait for a copy of the row ran out";
        default: return "psx_b200: too many tokens survive the filters for the device path";
    }
}

psx_status check_common(psx_ctx* ctx, const psx_sampling_config* config, int64_t rows, int64_t cols,
                        int64_t row_stride, int64_t vocab, const void* logits, const void* history_ids,
                        const void* history_offsets) {
    if (!ctx) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: context is null");
    if (psx_status s = check_config(config)) return s;
    if (rows < 0) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: rows must not be negative");
    if (vocab <= 0 || cols <= 0) return fail(PSX_ERR_BAD_ARGUMENT, "Generate: the model returned no logits");
    if (vocab > (int64_t)psx::kColumnMask) {
        return fail(PSX_ERR_UNSUPPORTED, "psx_b200: vocabulary exceeds 2^30 - 1 columns");
    }
    if (row_stride < cols) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: row_stride is smaller than the row");
    if (rows > 0 && !logits) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: logits is null");
    if (config->repetition_penalty != 1.0f && rows > 0 && (!history_ids || !history_offsets)) {
        return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: a repetition penalty needs history_ids and history_offsets");
    }
    return PSX_OK;
}

}  // namespace

extern "C" {

const char* psx_b200_version(void) { return "0.1.0"; }
const char* psx_b200_last_error(void) { return g_error.c_str(); }

psx_status psx_b200_ctx_create(int device, psx_ctx** out) {
    if (!out) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: out is null");
    *out = nullptr;
    int count = 0;
    PSX_CUDA(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: no such CUDA device");
    PSX_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    PSX_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major < 10) {
        return fail(PSX_ERR_UNSUPPORTED, "psx_b200: the kernels are built for sm_100a (B200) only");
    }
    psx_ctx* ctx = new psx_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    const cudaError_t e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete ctx;
        return fail(PSX_ERR_CUDA, std::string("CUDA error: ") + cudaGetErrorString(e));
    }
    *out = ctx;
    return PSX_OK;
}

void psx_b200_ctx_destroy(psx_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (Buffer* b : {&ctx->stats[0], &ctx->stats[1], &ctx->part_counts[0], &ctx->part_counts[1], &ctx->candidates[0], &ctx->candidates[1], &ctx->banned, &ctx->sort_keys, &ctx->head_logits, &ctx->attention_partial, &ctx->surv_cols, &ctx->surv_vals,
                      &ctx->surv_counts, &ctx->pl_tokens, &ctx->pl_log_probs, &ctx->pl_status, &ctx->h_logits, &ctx->h_history,
                      &ctx->h_offsets, &ctx->h_uniforms, &ctx->h_tokens, &ctx->h_log_probs, &ctx->h_status,
                      &ctx->h_diag, &ctx->shard_uniform_scratch}) {
        if (b->ptr) cudaFree(b->ptr);
    }
    for (cudaEvent_t e : ctx->timing_events) cudaEventDestroy(e);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
}

void* psx_b200_ctx_stream(psx_ctx* ctx) { return ctx ? ctx->stream : nullptr; }

psx_status psx_b200_sync(psx_ctx* ctx, void* stream) {
    if (!ctx) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: context is null");
    PSX_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    return PSX_OK;
}

uint64_t psx_b200_launch_count(const psx_ctx* ctx) { return ctx ? ctx->launches : 0; }

}  // extern "C"

namespace {

// Argument checks, plan, scratch and parameters shared by the sampling entry points.
psx_status plan_row_pass(psx_ctx* ctx, cudaStream_t stream, const float* logits, int64_t rows, int64_t vocab,
                         int64_t row_stride, const int64_t* history_ids, const int64_t* history_offsets,
                         const psx_sampling_config* config, Plan& plan, psx::ScanParams& sp, bool alternate = false) {
    PSX_CUDA(cudaSetDevice(ctx->device));
    plan = psx::make_plan(logits, vocab, row_stride, vocab, config);
    sp = psx::ScanParams{};
    sp.logits = logits;
    sp.row_stride = row_stride;
    sp.rows = rows;
    sp.cols = vocab;
    sp.col_begin = 0;
    sp.vocab = vocab;
    sp.history_ids = history_ids;
    sp.history_offsets = history_offsets;
    if (psx_status s = prepare_scan(ctx, stream, config, plan, sp)) return s;
    if (!alternate) return reserve_scan_scratch(ctx, rows, plan, sp);
    // A row pass followed by a survivor stage, call after call on one stream: this call's scratch is the set
    // that the call before it did not use, and only the row pass's last CTA waits for the kernel before it.
    ctx->scratch_set ^= 1;
    sp.wait_before_writes = 0;
    return reserve_scan_scratch(ctx, rows, plan, sp, ctx->scratch_set);
}

}  // namespace

extern "C" {

psx_status psx_b200_row_pass_only(psx_ctx* ctx, void* stream_ptr, const float* logits, int64_t rows, int64_t vocab,
                                  int64_t row_stride, const int64_t* history_ids, const int64_t* history_offsets,
                                  const psx_sampling_config* config) {
    if (psx_status s = check_common(ctx, config, rows, vocab, row_stride, vocab, logits, history_ids, history_offsets)) {
        return s;
    }
    if (rows == 0) return PSX_OK;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    Plan plan;
    psx::ScanParams sp;
    if (psx_status s = plan_row_pass(ctx, stream, logits, rows, vocab, row_stride, history_ids, history_offsets, config,
                                     plan, sp)) {
        return s;
    }
    PSX_CUDA(psx::launch_scan_rows(sp, plan.nucleus, stream));
    ++ctx->launches;
    return PSX_OK;
}

psx_status psx_b200_sample_rows(psx_ctx* ctx, void* stream_ptr, const float* logits, int64_t rows, int64_t vocab,
                                int64_t row_stride, const int64_t* history_ids, const int64_t* history_offsets,
                                const psx_sampling_config* config, const double* uniforms, int64_t* tokens,
                                float* log_probs, int32_t* row_status, psx_row_diag* diag) {
    if (psx_status s = check_common(ctx, config, rows, vocab, row_stride, vocab, logits, history_ids, history_offsets)) {
        return s;
    }
    if (rows == 0) return PSX_OK;
    if (!tokens || !log_probs || !row_status) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: an output pointer is null");
    if (config->do_sample && !uniforms) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: sampling needs uniforms");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    Plan plan;
    psx::ScanParams sp;
    if (psx_status s = plan_row_pass(ctx, stream, logits, rows, vocab, row_stride, history_ids, history_offsets, config,
                                     plan, sp, /*alternate=*/true)) {
        return s;
    }
    if (psx_status s = configure_merge(ctx, plan, plan.parts)) return s;

    psx::MergeParams mp{};
    psx::fill_merge_params(mp, sp, plan, config, rows, vocab, uniforms, tokens, log_probs, row_status, diag, logits, row_stride);

    cudaEvent_t marks[3] = {nullptr, nullptr, nullptr};
    if (ctx->timing) {
        for (cudaEvent_t& e : marks) PSX_CUDA(cudaEventCreate(&e));
        PSX_CUDA(cudaEventRecord(marks[0], stream));
    }
    if (!plan.lists_cannot_bound) {
        PSX_CUDA(psx::launch_scan_rows(sp, plan.nucleus, stream));
        ++ctx->launches;
    }
    if (ctx->timing) PSX_CUDA(cudaEventRecord(marks[1], stream));
    PSX_CUDA(psx::launch_merge_rows(mp, stream, &ctx->launches));
    if (ctx->timing) {
        PSX_CUDA(cudaEventRecord(marks[2], stream));
        ctx->timing_events.insert(ctx->timing_events.end(), marks, marks + 3);
    }
    return PSX_OK;
}

psx_status psx_b200_process_logits(psx_ctx* ctx, void* stream_ptr, float* logits, int64_t rows, int64_t vocab,
                                   int64_t row_stride, const int64_t* history_ids, const int64_t* history_offsets,
                                   const psx_sampling_config* config, int32_t* row_status) {
    if (psx_status s = check_common(ctx, config, rows, vocab, row_stride, vocab, logits, history_ids, history_offsets)) {
        return s;
    }
    if (rows == 0) return PSX_OK;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    const bool sample = config->do_sample != 0;
    const bool top_k_on = sample && config->top_k > 0 && config->top_k < vocab;
    // src/generation.cpp:74-76: greedy stops after the penalty and the EOS ban.
    const bool filters_on = sample && (top_k_on || config->top_p < 1.0f || config->min_p > 0.0f);
    Plan plan;
    psx::ScanParams sp;
    if (psx_status s = plan_row_pass(ctx, stream, logits, rows, vocab, row_stride, history_ids, history_offsets, config,
                                     plan, sp)) {
        return s;
    }
    if (psx_status s = reserve(ctx->pl_status, (size_t)rows * sizeof(int32_t))) return s;
    int32_t* status = row_status ? row_status : static_cast<int32_t*>(ctx->pl_status.ptr);

    psx::ProcessParams pp{};
    pp.logits = logits;
    pp.row_stride = row_stride;
    pp.rows = rows;
    pp.vocab = vocab;
    pp.history_ids = history_ids;
    pp.history_offsets = history_offsets;
    pp.banned_ids = sp.banned_ids;
    pp.num_banned = sp.num_banned;
    pp.apply_penalty = sp.apply_penalty;
    pp.penalty = sp.penalty;
    pp.apply_temperature = sp.apply_temperature;
    pp.temperature = sp.temperature;
    pp.filters_on = filters_on ? 1 : 0;
    pp.row_status = status;
    if (filters_on) {
        if (psx_status s = configure_merge(ctx, plan, plan.parts)) return s;
        const size_t slots = (size_t)rows * plan.sort_capacity;
        if (psx_status s = reserve(ctx->surv_cols, slots * sizeof(uint32_t))) return s;
        if (psx_status s = reserve(ctx->surv_vals, slots * sizeof(float))) return s;
        if (psx_status s = reserve(ctx->surv_counts, (size_t)rows * sizeof(uint32_t))) return s;
        if (psx_status s = reserve(ctx->pl_tokens, (size_t)rows * sizeof(int64_t))) return s;
        if (psx_status s = reserve(ctx->pl_log_probs, (size_t)rows * sizeof(float))) return s;
        if (!plan.lists_cannot_bound) {
            PSX_CUDA(psx::launch_scan_rows(sp, plan.nucleus, stream));
            ++ctx->launches;
        }
        psx::MergeParams mp{};
        psx::fill_merge_params(mp, sp, plan, config, rows, vocab, /*uniforms=*/nullptr,
                               static_cast<int64_t*>(ctx->pl_tokens.ptr), static_cast<float*>(ctx->pl_log_probs.ptr), status,
                               nullptr, logits, row_stride);
        mp.process_out = logits;  // a row that is decided from the row itself is rewritten in place right there
        mp.survivor_cols = static_cast<uint32_t*>(ctx->surv_cols.ptr);
        mp.survivor_vals = static_cast<float*>(ctx->surv_vals.ptr);
        mp.survivor_counts = static_cast<uint32_t*>(ctx->surv_counts.ptr);
        mp.survivor_cap = plan.sort_capacity;
        PSX_CUDA(psx::launch_merge_rows(mp, stream));
        ++ctx->launches;
        pp.survivor_cols = mp.survivor_cols;
        pp.survivor_vals = mp.survivor_vals;
        pp.survivor_counts = mp.survivor_counts;
        pp.survivor_cap = mp.survivor_cap;
    } else if (row_status) {
        PSX_CUDA(cudaMemsetAsync(row_status, 0, (size_t)rows * sizeof(int32_t), stream));
    }
    PSX_CUDA(psx::launch_process_rows(pp, stream));
    ctx->launches += filters_on ? 2 : 1;
    return PSX_OK;
}

psx_status psx_b200_process_logits_host(psx_ctx* ctx, float* logits, int64_t rows, int64_t vocab, int64_t row_stride,
                                        const int64_t* history_ids, const int64_t* history_offsets,
                                        const psx_sampling_config* config, int32_t* row_status) {
    if (psx_status s = check_common(ctx, config, rows, vocab, row_stride, vocab, logits, history_ids, history_offsets)) {
        return s;
    }
    if (rows == 0) return PSX_OK;
    PSX_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t stream = ctx->stream;
    const bool with_history = history_ids && history_offsets;
    const int64_t history_total = with_history ? history_offsets[rows] : 0;
    if (psx_status s = reserve(ctx->h_logits, (size_t)rows * vocab * sizeof(float))) return s;
    if (psx_status s = reserve(ctx->h_history, (size_t)std::max<int64_t>(history_total, 1) * sizeof(int64_t))) return s;
    if (psx_status s = reserve(ctx->h_offsets, (size_t)(rows + 1) * sizeof(int64_t))) return s;
    if (psx_status s = reserve(ctx->h_status, (size_t)rows * sizeof(int32_t))) return s;
    PSX_CUDA(cudaMemcpy2DAsync(ctx->h_logits.ptr, (size_t)vocab * sizeof(float), logits, (size_t)row_stride * sizeof(float),
                               (size_t)vocab * sizeof(float), (size_t)rows, cudaMemcpyHostToDevice, stream));
    if (with_history) {
        if (history_total > 0) {
            PSX_CUDA(cudaMemcpyAsync(ctx->h_history.ptr, history_ids, (size_t)history_total * sizeof(int64_t),
                                     cudaMemcpyHostToDevice, stream));
        }
        PSX_CUDA(cudaMemcpyAsync(ctx->h_offsets.ptr, history_offsets, (size_t)(rows + 1) * sizeof(int64_t),
                                 cudaMemcpyHostToDevice, stream));
    }
    struct RestorePromise {  // the staged inputs are being copied in by the transfers just enqueued
        psx_ctx* ctx;
        bool saved;
        ~RestorePromise() { ctx->inputs_ready = saved; }
    } restore{ctx, ctx->inputs_ready};
    ctx->inputs_ready = false;
    if (psx_status s = psx_b200_process_logits(ctx, stream, static_cast<float*>(ctx->h_logits.ptr), rows, vocab, vocab,
                                               with_history ? static_cast<const int64_t*>(ctx->h_history.ptr) : nullptr,
                                               with_history ? static_cast<const int64_t*>(ctx->h_offsets.ptr) : nullptr,
                                               config, static_cast<int32_t*>(ctx->h_status.ptr))) {
        return s;
    }
    PSX_CUDA(cudaMemcpy2DAsync(logits, (size_t)row_stride * sizeof(float), ctx->h_logits.ptr, (size_t)vocab * sizeof(float),
                               (size_t)vocab * sizeof(float), (size_t)rows, cudaMemcpyDeviceToHost, stream));
    std::vector<int32_t> local((size_t)rows);
    int32_t* out_status = row_status ? row_status : local.data();
    PSX_CUDA(cudaMemcpyAsync(out_status, ctx->h_status.ptr, (size_t)rows * sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
    PSX_CUDA(cudaStreamSynchronize(stream));
    for (int64_t r = 0; r < rows; ++r) {
        if (out_status[r] != PSX_ROW_OK && out_status[r] != PSX_ROW_ALL_REMOVED) {
            return fail(PSX_ERR_ROW_FAILED, std::string(row_failure_text(out_status[r])) + " (row " + std::to_string(r) + ")");
        }
    }
    return PSX_OK;
}

psx_status psx_b200_ctx_enable_timing(psx_ctx* ctx, int enable) {
    if (!ctx) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: context is null");
    ctx->timing = enable != 0;
    return PSX_OK;
}

psx_status psx_b200_ctx_inputs_are_ready(psx_ctx* ctx, int ready) {
    if (!ctx) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: context is null");
    ctx->inputs_ready = ready != 0;
    return PSX_OK;
}

psx_status psx_b200_ctx_set_wait_limit(psx_ctx* ctx, uint64_t nanoseconds) {
    if (!ctx) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: context is null");
    if (nanoseconds == 0) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: the wait limit must be positive");
    ctx->wait_limit_ns = nanoseconds;
    return PSX_OK;
}

psx_status psx_b200_test_short_copy(psx_ctx* ctx, int enable) {
    if (!ctx) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: context is null");
    ctx->test_short_copy = enable != 0;
    return PSX_OK;
}

psx_status psx_b200_ctx_read_timing(psx_ctx* ctx, double* row_pass_ms, double* survivor_stage_ms, uint64_t* calls) {
    if (!ctx) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: context is null");
    double scan = 0.0, merge = 0.0;
    const size_t n = ctx->timing_events.size() / 3;
    for (size_t i = 0; i < n; ++i) {
        cudaEvent_t* e = &ctx->timing_events[3 * i];
        float a = 0.0f, b = 0.0f;
        PSX_CUDA(cudaEventSynchronize(e[2]));
        PSX_CUDA(cudaEventElapsedTime(&a, e[0], e[1]));
        PSX_CUDA(cudaEventElapsedTime(&b, e[1], e[2]));
        scan += a;
        merge += b;
    }
    for (cudaEvent_t e : ctx->timing_events) cudaEventDestroy(e);
    ctx->timing_events.clear();
    if (row_pass_ms) *row_pass_ms = scan;
    if (survivor_stage_ms) *survivor_stage_ms = merge;
    if (calls) *calls = n;
    return PSX_OK;
}

psx_status psx_b200_sample_rows_host(psx_ctx* ctx, const float* logits, int64_t rows, int64_t vocab,
                                     int64_t row_stride, const int64_t* history_ids,
                                     const int64_t* history_offsets, const psx_sampling_config* config,
                                     const double* uniforms, int64_t* tokens, float* log_probs,
                                     int32_t* row_status, psx_row_diag* diag) {
    if (psx_status s = check_common(ctx, config, rows, vocab, row_stride, vocab, logits, history_ids, history_offsets)) {
        return s;
    }
    if (rows == 0) return PSX_OK;
    if (!tokens || !log_probs || !row_status) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: an output pointer is null");
    if (config->do_sample && !uniforms) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: sampling needs uniforms");
    PSX_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t stream = ctx->stream;
    const bool with_history = history_ids && history_offsets;
    const int64_t history_total = with_history ? history_offsets[rows] : 0;
    if (with_history && history_total < 0) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: history_offsets must ascend");

    if (psx_status s = reserve(ctx->h_logits, (size_t)rows * vocab * sizeof(float))) return s;
    if (psx_status s = reserve(ctx->h_history, (size_t)std::max<int64_t>(history_total, 1) * sizeof(int64_t))) return s;
    if (psx_status s = reserve(ctx->h_offsets, (size_t)(rows + 1) * sizeof(int64_t))) return s;
    if (psx_status s = reserve(ctx->h_uniforms, (size_t)rows * sizeof(double))) return s;
    if (psx_status s = reserve(ctx->h_tokens, (size_t)rows * sizeof(int64_t))) return s;
    if (psx_status s = reserve(ctx->h_log_probs, (size_t)rows * sizeof(float))) return s;
    if (psx_status s = reserve(ctx->h_status, (size_t)rows * sizeof(int32_t))) return s;
    if (psx_status s = reserve(ctx->h_diag, (size_t)rows * sizeof(psx_row_diag))) return s;

    // Rows are packed on the device (stride = vocab) whatever the host stride is.
    if (row_stride == vocab) {
        PSX_CUDA(cudaMemcpyAsync(ctx->h_logits.ptr, logits, (size_t)rows * vocab * sizeof(float), cudaMemcpyHostToDevice,
                                 stream));
    } else {
        PSX_CUDA(cudaMemcpy2DAsync(ctx->h_logits.ptr, (size_t)vocab * sizeof(float), logits,
                                   (size_t)row_stride * sizeof(float), (size_t)vocab * sizeof(float), (size_t)rows,
                                   cudaMemcpyHostToDevice, stream));
    }
    if (with_history) {
        if (history_total > 0) {
            PSX_CUDA(cudaMemcpyAsync(ctx->h_history.ptr, history_ids, (size_t)history_total * sizeof(int64_t),
                                     cudaMemcpyHostToDevice, stream));
        }
        PSX_CUDA(cudaMemcpyAsync(ctx->h_offsets.ptr, history_offsets, (size_t)(rows + 1) * sizeof(int64_t),
                                 cudaMemcpyHostToDevice, stream));
    }
    if (config->do_sample) {
        PSX_CUDA(cudaMemcpyAsync(ctx->h_uniforms.ptr, uniforms, (size_t)rows * sizeof(double), cudaMemcpyHostToDevice,
                                 stream));
    }
    // The staged inputs are being copied in by the transfers just enqueued: no promise holds for them.
    struct RestorePromise {
        psx_ctx* ctx;
        bool saved;
        ~RestorePromise() { ctx->inputs_ready = saved; }
    } restore{ctx, ctx->inputs_ready};
    ctx->inputs_ready = false;
    if (psx_status s = psx_b200_sample_rows(
            ctx, stream, static_cast<const float*>(ctx->h_logits.ptr), rows, vocab, vocab,
            with_history ? static_cast<const int64_t*>(ctx->h_history.ptr) : nullptr,
            with_history ? static_cast<const int64_t*>(ctx->h_offsets.ptr) : nullptr, config,
            static_cast<const double*>(ctx->h_uniforms.ptr), static_cast<int64_t*>(ctx->h_tokens.ptr),
            static_cast<float*>(ctx->h_log_probs.ptr), static_cast<int32_t*>(ctx->h_status.ptr),
            diag ? static_cast<psx_row_diag*>(ctx->h_diag.ptr) : nullptr)) {
        return s;
    }
    PSX_CUDA(cudaMemcpyAsync(tokens, ctx->h_tokens.ptr, (size_t)rows * sizeof(int64_t), cudaMemcpyDeviceToHost, stream));
    PSX_CUDA(cudaMemcpyAsync(log_probs, ctx->h_log_probs.ptr, (size_t)rows * sizeof(float), cudaMemcpyDeviceToHost,
                             stream));
    PSX_CUDA(cudaMemcpyAsync(row_status, ctx->h_status.ptr, (size_t)rows * sizeof(int32_t), cudaMemcpyDeviceToHost,
                             stream));
    if (diag) {
        PSX_CUDA(cudaMemcpyAsync(diag, ctx->h_diag.ptr, (size_t)rows * sizeof(psx_row_diag), cudaMemcpyDeviceToHost,
                                 stream));
    }
    PSX_CUDA(cudaStreamSynchronize(stream));
    for (int64_t r = 0; r < rows; ++r) {
        if (row_status[r] != PSX_ROW_OK) {
            const char* what = row_failure_text(row_status[r]);
            return fail(PSX_ERR_ROW_FAILED, std::string(what) + " (row " + std::to_string(r) + ")");
        }
    }
    return PSX_OK;
}

size_t psx_b200_shard_record_bytes(const psx_sampling_config* config) {
    return psx::shard_record_bytes(psx::shard_record_capacity(config ? config->do_sample != 0 : false,
                                                              config ? config->top_k : 0));
}

namespace {
// Where the records of a step through peer memory go, and what its packing kernel waits for.
struct PeerTargets {
    const psx::PeerLayout* layout;
    uint32_t* row_ready;         // one counter per row, raised by the row pass's parts
    uint32_t* ready_total;       // host: parts announced per row so far (all steps); this step's are added
    const uint32_t* step_done;   // device word: the last step whose results have all arrived here
    uint32_t step;               // this step (the first is 1)
    uint64_t wait_limit_ns;
    Buffer* stats;               // this step's set of row-pass scratch (the exchange's own, one of three)
    Buffer* part_counts;
    Buffer* candidates;
};

// The row pass over this GPU's columns and the packing of one record per row: into `records`, or
// (peers != nullptr) straight into the exchange buffers of the ranks that decide the rows.
psx_status shard_scan_impl(psx_ctx* ctx, void* stream_ptr, const float* shard_logits, int64_t rows,
                           int64_t shard_cols, int64_t row_stride, int64_t shard_begin, int64_t vocab,
                           const int64_t* history_ids, const int64_t* history_offsets,
                           const psx_sampling_config* config, void* records, const PeerTargets* peers) {
    if (psx_status s = check_common(ctx, config, rows, shard_cols, row_stride, vocab, shard_logits, history_ids,
                                    history_offsets)) {
        return s;
    }
    if (shard_begin < 0 || shard_begin + shard_cols > vocab) {
        return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: the shard does not lie inside the vocabulary");
    }
    if (rows == 0) return PSX_OK;
    if (!records && !peers) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: records is null");
    const bool sample = config->do_sample != 0;
    if (sample && !(config->top_k > 0 && config->top_k < vocab)) {
        return fail(PSX_ERR_UNSUPPORTED, "psx_b200: the vocabulary-sharded path samples with a top-k only");
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    PSX_CUDA(cudaSetDevice(ctx->device));

    const Plan plan = psx::make_plan(shard_logits, shard_cols, row_stride, vocab, config);
    psx::ScanParams sp{};
    sp.logits = shard_logits;
    sp.row_stride = row_stride;
    sp.rows = rows;
    sp.cols = shard_cols;
    sp.col_begin = shard_begin;
    sp.vocab = vocab;
    sp.history_ids = history_ids;
    sp.history_offsets = history_offsets;
    if (psx_status s = prepare_scan(ctx, stream, config, plan, sp)) return s;
    if (peers) {
        // Steps through peer memory follow one another kernel under kernel: this step's row pass writes a
        // scratch set of the exchange's own that the two steps before it did not use (their packing kernels
        // may still be reading theirs) and raises a counter per row; the packing kernel takes the rows as
        // they finish.
        sp.wait_before_writes = 0;
        sp.row_ready = peers->row_ready;
        const size_t parts = (size_t)rows * plan.parts;
        if (psx_status s = reserve(*peers->stats, parts * sizeof(psx::PartStats))) return s;
        if (psx_status s = reserve(*peers->part_counts, parts * sizeof(uint32_t))) return s;
        if (psx_status s = reserve(*peers->candidates, parts * psx::kPartCap * sizeof(uint2))) return s;
        sp.stats = static_cast<psx::PartStats*>(peers->stats->ptr);
        sp.part_counts = static_cast<uint32_t*>(peers->part_counts->ptr);
        sp.candidates = static_cast<uint2*>(peers->candidates->ptr);
    } else if (psx_status s = reserve_scan_scratch(ctx, rows, plan, sp)) {
        return s;
    }
    PSX_CUDA(psx::launch_scan_rows(sp, plan.nucleus, stream));
    ++ctx->launches;

    psx::PackParams pp{};
    pp.stats = sp.stats;
    pp.part_counts = sp.part_counts;
    pp.candidates = sp.candidates;
    pp.parts = plan.parts;
    pp.rows = rows;
    pp.apply_temperature = plan.apply_temperature ? 1 : 0;
    pp.temperature = config->temperature;
    pp.penalty = config->repetition_penalty;
    pp.capacity = psx::shard_record_capacity(sample, config->top_k);
    pp.do_sample = sample ? 1 : 0;
    pp.top_k = sample ? (int32_t)std::min<int64_t>(config->top_k, 1 << 20) : 0;
    pp.records = records;
    if (peers) {
        pp.to_peers = 1;
        pp.peers = *peers->layout;
        *peers->ready_total += (uint32_t)plan.parts;
        pp.row_ready = peers->row_ready;
        pp.row_ready_target = *peers->ready_total;
        pp.step_done = peers->step_done;
        pp.step_done_target = peers->step > 2 ? peers->step - 2 : 0;  // two steps are in flight: see psx_exchange
        pp.wait_limit_ns = peers->wait_limit_ns;
    }
    PSX_CUDA(psx::launch_pack_records(pp, stream));
    ++ctx->launches;
    return PSX_OK;
}

// The survivor stage over records that lie shard-major in this GPU's memory: the record of shard s and
// row r at base + s * shard_stride + r * record (r the absolute row).  arrivals (optional, indexed by the
// absolute row): see MergeParams.
psx_status shard_merge_impl(psx_ctx* ctx, cudaStream_t stream, const char* base, int64_t shard_stride, int32_t num_shards,
                            int64_t row_begin, int64_t row_count, int64_t vocab, const psx_sampling_config* config,
                            const double* uniforms, int64_t* tokens, float* log_probs, int32_t* row_status,
                            psx_row_diag* diag, const uint32_t* arrivals, uint32_t arrivals_target, uint64_t arrivals_wait_ns,
                            const psx::PeerLayout* publish_to = nullptr) {
    const bool sample = config->do_sample != 0;
    Plan plan;
    plan.apply_temperature = sample && config->temperature != 1.0f;
    plan.sort_capacity = 1024;
    plan.gather_capacity = 4096;
    if (psx_status s = configure_merge(ctx, plan, num_shards)) return s;
    const int capacity = psx::shard_record_capacity(sample, config->top_k);
    const int64_t record = (int64_t)psx::shard_record_bytes(capacity);
    psx::MergeParams mp{};
    mp.stats = base + psx::kRecordStatsOffset;
    mp.part_counts = base + psx::kRecordCountOffset;
    mp.candidates = base + psx::kRecordCandidatesOffset;
    mp.parts = num_shards;
    mp.part_cap = capacity;
    mp.slot_shift = psx::merge_slot_shift(num_shards, capacity, capacity / 2);
    mp.stats_row_stride = mp.count_row_stride = mp.cand_row_stride = record;
    mp.stats_part_stride = mp.count_part_stride = mp.cand_part_stride = shard_stride;
    mp.rows = row_count;
    mp.row_begin = row_begin;
    mp.vocab = vocab;
    mp.do_sample = sample ? 1 : 0;
    mp.apply_temperature = plan.apply_temperature ? 1 : 0;
    mp.temperature = config->temperature;
    mp.penalty = config->repetition_penalty;
    mp.top_k = config->top_k;
    mp.top_p = config->top_p;
    mp.min_p = config->min_p;
    mp.uniforms = uniforms;  // by absolute row; the outputs hold the merged rows only, the first of them at [0]
    mp.tokens = tokens - row_begin;
    mp.log_probs = log_probs - row_begin;
    mp.row_status = row_status - row_begin;
    mp.diag = diag ? diag - row_begin : nullptr;
    mp.sort_capacity = plan.sort_capacity;
    mp.gather_capacity = plan.gather_capacity;
    mp.arrivals = arrivals;
    mp.arrivals_target = arrivals_target;
    mp.arrivals_wait_ns = arrivals_wait_ns;
    if (publish_to) {
        mp.publish = 1;
        mp.peers = *publish_to;
    }
    PSX_CUDA(psx::launch_merge_rows(mp, stream, &ctx->launches));
    return PSX_OK;
}
}  // namespace

psx_status psx_b200_shard_scan(psx_ctx* ctx, void* stream_ptr, const float* shard_logits, int64_t rows,
                               int64_t shard_cols, int64_t row_stride, int64_t shard_begin, int64_t vocab,
                               const int64_t* history_ids, const int64_t* history_offsets,
                               const psx_sampling_config* config, void* records) {
    return shard_scan_impl(ctx, stream_ptr, shard_logits, rows, shard_cols, row_stride, shard_begin, vocab, history_ids,
                           history_offsets, config, records, nullptr);
}

psx_status psx_b200_shard_merge_rows(psx_ctx* ctx, void* stream_ptr, const void* gathered, int32_t num_shards,
                                     int64_t rows, int64_t row_begin, int64_t row_count, int64_t vocab,
                                     const psx_sampling_config* config, const double* uniforms, int64_t* tokens,
                                     float* log_probs, int32_t* row_status, psx_row_diag* diag) {
    if (!ctx) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: context is null");
    if (psx_status s = check_config(config)) return s;
    if (rows < 0 || num_shards < 1 || vocab <= 0) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: bad sizes");
    if (row_begin < 0 || row_count < 0 || row_begin + row_count > rows) {
        return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: the rows to merge do not lie inside the batch");
    }
    if (rows == 0 || row_count == 0) return PSX_OK;
    if (!gathered || !tokens || !log_probs || !row_status) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: null pointer");
    const bool sample = config->do_sample != 0;
    if (sample && !uniforms) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: sampling needs uniforms");
    if (sample && !(config->top_k > 0 && config->top_k < vocab)) {
        return fail(PSX_ERR_UNSUPPORTED, "psx_b200: the vocabulary-sharded path samples with a top-k only");
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    PSX_CUDA(cudaSetDevice(ctx->device));

    const int64_t record = (int64_t)psx_b200_shard_record_bytes(config);
    return shard_merge_impl(ctx, stream, static_cast<const char*>(gathered), record * rows, num_shards, row_begin, row_count,
                            vocab, config, uniforms, tokens, log_probs, row_status, diag, nullptr, 0, 0);
}

psx_status psx_b200_shard_merge(psx_ctx* ctx, void* stream_ptr, const void* gathered, int32_t num_shards,
                                int64_t rows, int64_t vocab, const psx_sampling_config* config,
                                const double* uniforms, int64_t* tokens, float* log_probs, int32_t* row_status,
                                psx_row_diag* diag) {
    return psx_b200_shard_merge_rows(ctx, stream_ptr, gathered, num_shards, rows, 0, rows < 0 ? 0 : rows, vocab, config,
                                     uniforms, tokens, log_probs, row_status, diag);
}

psx_status psx_b200_top_k_rows(psx_ctx* ctx, void* stream_ptr, const float* in, float* values, float* indices,
                               size_t rows, size_t cols, size_t k, int largest) {
    if (!ctx) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: context is null");
    if (rows == 0) return PSX_OK;  // src/cuda_backend.cu:853-855
    if (cols == 0) return fail(PSX_ERR_BAD_ARGUMENT, "top_k: input must be non-empty with rank >= 1");
    if (k < 1 || k > cols) {  // src/top_k.cpp:14-17
        return fail(PSX_ERR_BAD_ARGUMENT,
                    "top_k: k must be in [1, " + std::to_string(cols) + "], got " + std::to_string(k));
    }
    if (cols > (size_t(1) << 24)) {  // src/top_k.cpp:19-21
        return fail(PSX_ERR_BAD_ARGUMENT, "top_k: last dimension exceeds 2^24, beyond exact float indices");
    }
    if (rows > 0x7FFFFFFFull) return fail(PSX_ERR_UNSUPPORTED, "psx_b200: too many rows for one launch");
    if (!in || !values || !indices) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: null pointer");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    PSX_CUDA(cudaSetDevice(ctx->device));
    if (k > (size_t)psx::kTopKMax) {  // more than one CTA sorts in shared memory: the rows are sorted whole, in scratch
        size_t batch = 0;
        if (psx_status s = reserve(ctx->sort_keys, psx::sort_rows_scratch_bytes(rows, cols, &batch))) return s;
        PSX_CUDA(psx::launch_sort_rows(in, values, indices, rows, cols, k, largest != 0, ctx->sort_keys.ptr, stream));
        ctx->launches += (rows + batch - 1) / batch;
        return PSX_OK;
    }
    PSX_CUDA(psx::launch_topk_rows(in, values, indices, rows, cols, k, largest != 0, stream));
    ++ctx->launches;
    return PSX_OK;
}

namespace {
psx_status check_head(psx_ctx* ctx, const float* hidden, int64_t rows, int64_t d, const float* weight, int64_t vocab,
                      int32_t weight_layout) {
    if (!ctx) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: context is null");
    if (rows < 0) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: rows must not be negative");
    if (d <= 0 || vocab <= 0) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: the head needs d_model > 0 and vocab > 0");
    if (weight_layout != PSX_HEAD_VOCAB_BY_D && weight_layout != PSX_HEAD_D_BY_VOCAB) {
        return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: unknown weight layout");
    }
    if (rows > 0 && (!hidden || !weight)) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: null pointer");
    return PSX_OK;
}
}  // namespace

psx_status psx_b200_lm_head_logits(psx_ctx* ctx, void* stream_ptr, const float* hidden, int64_t rows, int64_t d,
                                   const float* weight, int64_t vocab, int32_t weight_layout, float* logits,
                                   int64_t row_stride) {
    if (psx_status s = check_head(ctx, hidden, rows, d, weight, vocab, weight_layout)) return s;
    if (rows == 0) return PSX_OK;
    if (!logits || row_stride < vocab) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: logits is null or row_stride is smaller than the row");
    PSX_CUDA(cudaSetDevice(ctx->device));
    PSX_CUDA(psx::launch_lm_head(hidden, rows, d, weight, vocab, weight_layout == PSX_HEAD_VOCAB_BY_D, logits, row_stride,
                                 static_cast<cudaStream_t>(stream_ptr)));
    ctx->launches += (uint64_t)((rows + 63) / 64);
    return PSX_OK;
}

psx_status psx_b200_lm_head_sample_rows(psx_ctx* ctx, void* stream_ptr, const float* hidden, int64_t rows, int64_t d,
                                        const float* weight, int64_t vocab, int32_t weight_layout,
                                        const int64_t* history_ids, const int64_t* history_offsets,
                                        const psx_sampling_config* config, const double* uniforms, int64_t* tokens,
                                        float* log_probs, int32_t* row_status, psx_row_diag* diag) {
    if (psx_status s = check_head(ctx, hidden, rows, d, weight, vocab, weight_layout)) return s;
    if (psx_status s = check_config(config)) return s;
    if (rows == 0) return PSX_OK;
    PSX_CUDA(cudaSetDevice(ctx->device));
    const int64_t stride = (vocab + 3) / 4 * 4;  // rows of the scratch start on 16-byte boundaries
    if (psx_status s = reserve(ctx->head_logits, (size_t)rows * stride * sizeof(float))) return s;
    float* logits = static_cast<float*>(ctx->head_logits.ptr);
    PSX_CUDA(psx::launch_lm_head(hidden, rows, d, weight, vocab, weight_layout == PSX_HEAD_VOCAB_BY_D, logits, stride,
                                 static_cast<cudaStream_t>(stream_ptr)));
    ctx->launches += (uint64_t)((rows + 63) / 64);
    // The logits were written by the kernel just enqueued: the row pass must wait for it whatever the
    // caller promised about its own inputs.
    struct RestorePromise {
        psx_ctx* ctx;
        bool saved;
        ~RestorePromise() { ctx->inputs_ready = saved; }
    } restore{ctx, ctx->inputs_ready};
    ctx->inputs_ready = false;
    return psx_b200_sample_rows(ctx, stream_ptr, logits, rows, vocab, stride, history_ids, history_offsets, config, uniforms,
                                tokens, log_probs, row_status, diag);
}

psx_status psx_b200_softmax_rows(psx_ctx* ctx, void* stream_ptr, const float* in, float* out, size_t rows, size_t cols) {
    if (!ctx) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: context is null");
    if (rows == 0 || cols == 0) return PSX_OK;  // src/cuda_backend.cu: every op returns early on an empty size
    if (!in || !out) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: null pointer");
    PSX_CUDA(cudaSetDevice(ctx->device));
    PSX_CUDA(psx::launch_softmax_rows(in, out, rows, cols, static_cast<cudaStream_t>(stream_ptr)));
    ++ctx->launches;
    return PSX_OK;
}

psx_status psx_b200_logsumexp_rows(psx_ctx* ctx, void* stream_ptr, const float* in, float* out, size_t rows, size_t cols) {
    if (!ctx) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: context is null");
    if (rows == 0 || cols == 0) return PSX_OK;
    if (!in || !out) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: null pointer");
    PSX_CUDA(cudaSetDevice(ctx->device));
    PSX_CUDA(psx::launch_logsumexp_rows(in, out, rows, cols, static_cast<cudaStream_t>(stream_ptr)));
    ++ctx->launches;
    return PSX_OK;
}

psx_status psx_b200_gather_rows(psx_ctx* ctx, void* stream_ptr, const float* table, const float* indices, float* out,
                                size_t count, size_t dim) {
    if (!ctx) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: context is null");
    if (count == 0 || dim == 0) return PSX_OK;
    if (!table || !indices || !out) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: null pointer");
    PSX_CUDA(cudaSetDevice(ctx->device));
    PSX_CUDA(psx::launch_gather_rows(table, indices, out, count, dim, static_cast<cudaStream_t>(stream_ptr)));
    ++ctx->launches;
    return PSX_OK;
}

psx_status psx_b200_decode_attention(psx_ctx* ctx, void* stream_ptr, const float* q, const float* keys, const float* values,
                                     const float* key_keep, float* context, int64_t batch, int64_t heads, int64_t kv_heads,
                                     int64_t q_len, int64_t head_dim, int64_t cached, int64_t max_len, float scale,
                                     int32_t causal, int64_t window, int32_t* status) {
    if (!ctx) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: context is null");
    if (batch < 0 || heads <= 0 || kv_heads <= 0 || q_len <= 0 || head_dim <= 0 || cached < 0 || window < 0) {
        return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: attention sizes must be positive");
    }
    if (heads % kv_heads != 0) {  // src/multihead_attention_module.cpp: num_heads must be a multiple of num_kv_heads
        return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: heads must be a multiple of kv_heads");
    }
    const int64_t total = cached + q_len;
    if (total > max_len) return fail(PSX_ERR_BAD_ARGUMENT, "KVCache: the cache is full");  // src/kv_cache.cpp
    if (batch == 0) return PSX_OK;
    if (!q || !keys || !values || !context) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: null pointer");
    if ((reinterpret_cast<uintptr_t>(keys) | reinterpret_cast<uintptr_t>(values)) % 16 != 0) {
        return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: the cache must start on a 16-byte boundary");
    }
    const int64_t group = heads / kv_heads;
    if (group * q_len > 8 || head_dim % 4 != 0 || head_dim > 256) {
        return fail(PSX_ERR_UNSUPPORTED,
                    "psx_b200: attention over the cache takes at most 8 query rows per kv head (group x new positions) "
                    "and a head dimension that is a multiple of 4 up to 256");
    }
    PSX_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    psx::AttentionParams p{};
    p.q = q; p.keys = keys; p.values = values; p.key_keep = key_keep; p.context = context; p.status = status;
    p.batch = batch; p.total = total; p.max_len = max_len; p.offset = cached; p.window = window;
    p.heads = (int32_t)heads; p.kv_heads = (int32_t)kv_heads; p.group = (int32_t)group; p.q_len = (int32_t)q_len;
    p.head_dim = (int32_t)head_dim; p.causal = causal ? 1 : 0; p.scale = scale;
    p.wait_limit_ns = ctx->wait_limit_ns;
    p.splits = psx::attention_splits(batch * kv_heads, total, ctx->sm_count, (int)head_dim);
    if (p.splits > 1) {
        if (psx_status s = reserve(ctx->attention_partial, psx::attention_partial_bytes(p))) return s;
        p.partial = static_cast<float*>(ctx->attention_partial.ptr);
    }
    PSX_CUDA(psx::launch_decode_attention(p, stream));
    ctx->launches += p.splits > 1 ? 2 : 1;
    return PSX_OK;
}

void psx_uniforms_mt19937_64(const uint64_t* seeds, int64_t n, double* out) {
    for (int64_t i = 0; i < n; ++i) {
        std::mt19937_64 engine(seeds[i]);
        out[i] = static_cast<double>(engine() >> 11) * 0x1.0p-53;
    }
}

void psx_uniforms_portable(const uint64_t* seeds, int64_t n, double* out) {
    for (int64_t i = 0; i < n; ++i) {
        uint64_t z = seeds[i] + 0x9E3779B97F4A7C15ULL;  // SplitMix64: one step from state = seed
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
        z ^= z >> 31;
        out[i] = (static_cast<double>(z >> 11) + 0.5) / static_cast<double>(1ULL << 53);
    }
}

// ---- vocabulary shards exchanged over peer memory (peer_exchange.cuh) ----------------------------------

// Two steps are in flight at a time: everything a step exchanges exists twice, once for odd steps and once
// for even ones (two halves of the exchange buffer, two blocks of local results), so that a step's
// records and results never wait for the step before to have been read everywhere -- only for the step
// before that (step_done).  The row-pass scratch exists three times: the packing kernel of step e + 2
// only starts once step e is done everywhere, so what step e + 3 overwrites has long been read.
struct psx_exchange {
    psx_ctx* ctx = nullptr;
    psx::PeerLayout layout{};  // base[r]: the first half of rank r's buffer
    int64_t rows = 0;
    size_t half_bytes = 0;
    size_t buffer_bytes = 0;
    char* buffer = nullptr;  // this rank's exchange buffer (cudaMalloc: its IPC handle goes to the peers)
    char* block = nullptr;   // this rank's results of a step (the survivor stage's own outputs), twice
    Buffer stats[3], part_counts[3], candidates[3];
    uint32_t* words = nullptr;   // rows + 1 device words: a counter per row for the row pass, then step_done
    uint32_t ready_total = 0;    // parts per row announced so far, over all steps
    bool opened[psx::kMaxPeers] = {};
    bool ready = false;
    uint32_t step = 0;
    uint64_t wait_limit_ns = psx::kDefaultWaitLimitNs;
    uint32_t test_extra_arrivals = 0;  // psx_b200_exchange_test_wait
};

size_t psx_b200_exchange_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

psx_status psx_b200_exchange_create(psx_ctx* ctx, int32_t world, int32_t rank, int64_t rows,
                                    const psx_sampling_config* config, psx_exchange** out, void* handle) {
    if (!ctx || !out || !handle) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: null pointer");
    if (psx_status s = check_config(config)) return s;
    if (world < 1 || world > psx::kMaxPeers || rank < 0 || rank >= world) {
        return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: an exchange spans 1 to 8 ranks, and the rank lies among them");
    }
    if (rows < 1) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: an exchange needs at least one row");
    PSX_CUDA(cudaSetDevice(ctx->device));
    psx_exchange* ex = new psx_exchange();
    ex->ctx = ctx;
    ex->rows = rows;
    psx::PeerLayout& l = ex->layout;
    l.world = world;
    l.rank = rank;
    l.rows_per_rank = (rows + world - 1) / world;
    l.record_bytes = (int64_t)psx_b200_shard_record_bytes(config);
    ex->half_bytes = (size_t)psx::peer_layout_offsets(world, l.rows_per_rank, l.record_bytes, &l.records_offset,
                                                      &l.arrivals_offset, &l.results_offset, &l.flags_offset);
    ex->buffer_bytes = 2 * ex->half_bytes;
    const size_t block_bytes = (size_t)psx::peer_results_block_bytes(l.rows_per_rank);
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&ex->buffer), ex->buffer_bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&ex->block), 2 * block_bytes);
    if (e == cudaSuccess) e = cudaMemset(ex->buffer, 0, ex->buffer_bytes);
    if (e == cudaSuccess) e = cudaMemset(ex->block, 0, 2 * block_bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&ex->words), sizeof(uint32_t) * (size_t)(rows + 1));
    if (e == cudaSuccess) e = cudaMemset(ex->words, 0, sizeof(uint32_t) * (size_t)(rows + 1));
    if (e == cudaSuccess) e = cudaDeviceSynchronize();  // zero before any peer can learn the handle
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle), ex->buffer);
    if (e != cudaSuccess) {
        if (ex->buffer) cudaFree(ex->buffer);
        if (ex->block) cudaFree(ex->block);
        if (ex->words) cudaFree(ex->words);
        delete ex;
        return fail(PSX_ERR_CUDA, std::string("psx_b200: exchange buffer: ") + cudaGetErrorString(e));
    }
    l.base[rank] = ex->buffer;
    *out = ex;
    return PSX_OK;
}

psx_status psx_b200_exchange_open(psx_exchange* ex, const void* handles) {
    if (!ex || !handles) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: null pointer");
    if (ex->ready) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: the exchange is already open");
    PSX_CUDA(cudaSetDevice(ex->ctx->device));
    const cudaIpcMemHandle_t* all = static_cast<const cudaIpcMemHandle_t*>(handles);
    for (int r = 0; r < ex->layout.world; ++r) {
        if (r == ex->layout.rank) continue;
        void* ptr = nullptr;
        PSX_CUDA(cudaIpcOpenMemHandle(&ptr, all[r], cudaIpcMemLazyEnablePeerAccess));
        ex->layout.base[r] = static_cast<char*>(ptr);
        ex->opened[r] = true;
    }
    ex->ready = true;
    return PSX_OK;
}

void psx_b200_exchange_destroy(psx_exchange* ex) {
    if (!ex) return;
    cudaSetDevice(ex->ctx->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < ex->layout.world; ++r) {
        if (ex->opened[r]) cudaIpcCloseMemHandle(ex->layout.base[r]);
    }
    if (ex->buffer) cudaFree(ex->buffer);
    if (ex->block) cudaFree(ex->block);
    if (ex->words) cudaFree(ex->words);
    for (int i = 0; i < 3; ++i) {
        for (Buffer* b : {&ex->stats[i], &ex->part_counts[i], &ex->candidates[i]}) {
            if (b->ptr) cudaFree(b->ptr);
        }
    }
    delete ex;
}

psx_status psx_b200_exchange_results(const psx_exchange* ex, const void** results, int64_t* rows_per_rank) {
    if (!ex || !results || !rows_per_rank) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: null pointer");
    *results = ex->buffer + (ex->step & 1u) * ex->half_bytes + ex->layout.results_offset;  // the last step's half
    *rows_per_rank = ex->layout.rows_per_rank;
    return PSX_OK;
}

psx_status psx_b200_exchange_test_wait(psx_exchange* ex, uint64_t wait_limit_ns, uint32_t extra_arrivals) {
    if (!ex) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: null pointer");
    ex->wait_limit_ns = wait_limit_ns ? wait_limit_ns : psx::kDefaultWaitLimitNs;
    ex->test_extra_arrivals = extra_arrivals;
    return PSX_OK;
}

psx_status psx_b200_exchange_sample(psx_exchange* ex, void* stream_ptr, const float* shard_logits, int64_t shard_cols,
                                    int64_t row_stride, int64_t shard_begin, int64_t vocab, const int64_t* history_ids,
                                    const int64_t* history_offsets, const psx_sampling_config* config,
                                    const double* uniforms) {
    if (!ex) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: null pointer");
    if (!ex->ready) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: the exchange is not open yet");
    psx_ctx* ctx = ex->ctx;
    if (psx_status s = check_config(config)) return s;
    const uint32_t step = ex->step + 1, half = step & 1u, turn = (step + 1) / 2;  // this half's turn-th step
    psx::PeerLayout l = ex->layout;
    for (int r = 0; r < l.world; ++r) l.base[r] += half * ex->half_bytes;
    char* const own = ex->buffer + half * ex->half_bytes;
    char* const block = ex->block + half * (size_t)psx::peer_results_block_bytes(l.rows_per_rank);
    if ((int64_t)psx_b200_shard_record_bytes(config) != l.record_bytes) {
        return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: the settings need records of another size than the exchange was created for");
    }
    const bool sample = config->do_sample != 0;
    if (sample && !uniforms) return fail(PSX_ERR_BAD_ARGUMENT, "psx_b200: sampling needs uniforms");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    const int set = (int)(step % 3);
    const PeerTargets targets{&l, ex->words, &ex->ready_total, ex->words + ex->rows, step, ex->wait_limit_ns,
                              &ex->stats[set], &ex->part_counts[set], &ex->candidates[set]};
    if (psx_status s = shard_scan_impl(ctx, stream_ptr, shard_logits, ex->rows, shard_cols, row_stride, shard_begin, vocab,
                                       history_ids, history_offsets, config, nullptr, &targets)) {
        return s;  // (the peers' waits for this rank's records of the step run out)
    }
    ex->step = step;
    const int64_t row_begin = std::min<int64_t>((int64_t)l.rank * l.rows_per_rank, ex->rows);
    const int64_t row_count = std::min<int64_t>(l.rows_per_rank, ex->rows - row_begin);
    if (row_count > 0) {
        // this rank's rows: their records lie here, shard after shard; absolute row r at [r - row_begin]
        const char* base = own + l.records_offset - row_begin * l.record_bytes;
        const uint32_t* arrivals = reinterpret_cast<const uint32_t*>(own + l.arrivals_offset) - row_begin;
        int64_t* tokens = reinterpret_cast<int64_t*>(block);
        float* log_probs = reinterpret_cast<float*>(block + 8 * l.rows_per_rank);
        int32_t* status = reinterpret_cast<int32_t*>(block + 12 * l.rows_per_rank);
        if (psx_status s = shard_merge_impl(ctx, stream, base, l.rows_per_rank * l.record_bytes, l.world, row_begin, row_count,
                                            vocab, config, uniforms, tokens, log_probs, status, nullptr, arrivals,
                                            turn * (uint32_t)l.world + ex->test_extra_arrivals, ex->wait_limit_ns, &l)) {
            return s;
        }
    }
    psx::AwaitParams aw{};
    aw.layout = l;
    aw.rows = ex->rows;
    aw.step = step;
    aw.turn = turn;
    aw.wait_limit_ns = ex->wait_limit_ns;
    aw.step_done = ex->words + ex->rows;
    PSX_CUDA(psx::launch_await_results(aw, stream));
    ++ctx->launches;
    return PSX_OK;
}

}  // extern "C"
