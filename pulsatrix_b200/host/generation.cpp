// ProcessLogits and Generate over the C ABI (include/psx_b200.h).  The loop, the engine and the
// exceptions are the reference's (src/generation.cpp:114-164); each step's arithmetic runs on
// the GPU.  One psx_ctx per host thread, created on first use on the current CUDA device.
#include "pulsatrix/generation.hpp"

#include <cuda_runtime.h>

#include <algorithm>
#include <memory>
#include <random>
#include <stdexcept>
#include <string>

#include "psx_b200.h"
#include "pulsatrix/determinism.hpp"

namespace pulsatrix {
namespace {

struct ContextHolder {
    psx_ctx* ctx = nullptr;
    int64_t* history = nullptr;  // device copy of the sequence, for the device-logits overload
    size_t history_capacity = 0;
    double* uniform = nullptr;   // device: the step's draw, then its outputs
    int64_t* token = nullptr;
    float* log_prob = nullptr;
    int32_t* status = nullptr;
    int64_t* offsets = nullptr;
    cudaEvent_t produced = nullptr;  // marks what a model has enqueued on its own stream
    ~ContextHolder() {
        if (produced) cudaEventDestroy(produced);
        for (void* p : {(void*)history, (void*)uniform, (void*)token, (void*)log_prob, (void*)status, (void*)offsets}) {
            if (p) cudaFree(p);
        }
        if (ctx) psx_b200_ctx_destroy(ctx);
    }
};

[[noreturn]] void raise(psx_status s) {
    const std::string message = psx_b200_last_error();
    if (s == PSX_ERR_BAD_ARGUMENT || s == PSX_ERR_ROW_FAILED) throw std::invalid_argument(message);
    throw std::runtime_error(message);
}

ContextHolder& thread_context() {
    thread_local ContextHolder holder;
    if (!holder.ctx) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess) device = 0;
        const psx_status s = psx_b200_ctx_create(device, &holder.ctx);
        if (s != PSX_OK) raise(s);
    }
    return holder;
}

psx_sampling_config to_c(const GenerationConfig& c, int64_t num_new_tokens) {
    psx_sampling_config out{};
    out.min_new_tokens = c.min_new_tokens;
    out.num_new_tokens = num_new_tokens;
    out.eos_token_ids = c.eos_token_ids.data();
    out.num_eos_token_ids = static_cast<int64_t>(c.eos_token_ids.size());
    out.do_sample = c.do_sample ? 1 : 0;
    out.temperature = c.temperature;
    out.top_k = c.top_k;
    out.top_p = c.top_p;
    out.min_p = c.min_p;
    out.repetition_penalty = c.repetition_penalty;
    return out;
}

// The one check the C configuration does not carry (src/generation.cpp:20-22).
void check_loop_fields(const GenerationConfig& c) {
    if (c.max_new_tokens < 0 || c.min_new_tokens < 0) {
        throw std::invalid_argument("GenerationConfig: max_new_tokens and min_new_tokens must not be negative");
    }
}

bool is_eos(const GenerationConfig& c, int64_t token) {
    return std::find(c.eos_token_ids.begin(), c.eos_token_ids.end(), token) != c.eos_token_ids.end();
}

// Shared loop: `step` returns (token, log-prob) for the sequence so far and the step number.
template <typename Step>
GenerationResult run_loop(const std::vector<int64_t>& prompt, const GenerationConfig& config, Step&& step) {
    check_loop_fields(config);
    {   // an invalid config is rejected before anything else, even with max_new_tokens == 0:
        // a call over zero rows runs the library's CheckConfig and nothing more
        const psx_sampling_config c = to_c(config, 0);
        const psx_status s = psx_b200_process_logits_host(thread_context().ctx, nullptr, 0, 1, 1, nullptr, nullptr, &c, nullptr);
        if (s != PSX_OK) raise(s);
    }
    if (prompt.empty()) throw std::invalid_argument("Generate: the prompt is empty");
    std::mt19937_64 engine(config.seed ? *config.seed : next_seed());
    GenerationResult result;
    result.tokens = prompt;
    for (int64_t n = 0; n < config.max_new_tokens; ++n) {
        const double u = config.do_sample ? static_cast<double>(engine() >> 11) * 0x1.0p-53 : 0.0;
        int64_t token = -1;
        float log_prob = 0.0f;
        step(result.tokens, n, u, token, log_prob);
        result.tokens.push_back(token);
        result.new_tokens.push_back(token);
        result.log_probs.push_back(log_prob);
        if (is_eos(config, token)) {
            result.finish_reason = FinishReason::Eos;
            return result;
        }
    }
    result.finish_reason = FinishReason::Length;
    return result;
}

}  // namespace

void ProcessLogits(std::vector<float>& logits, const std::vector<int64_t>& tokens, int64_t num_new_tokens,
                   const GenerationConfig& config) {
    check_loop_fields(config);
    const psx_sampling_config c = to_c(config, num_new_tokens);
    const int64_t offsets[2] = {0, static_cast<int64_t>(tokens.size())};
    const int64_t placeholder = -1;  // an id outside every vocabulary, for an empty history
    const int64_t vocab = static_cast<int64_t>(logits.size());
    const int64_t rows = vocab > 0 ? 1 : 0;
    const psx_status s = psx_b200_process_logits_host(thread_context().ctx, logits.data(), rows, std::max<int64_t>(vocab, 1),
                                                      std::max<int64_t>(vocab, 1), tokens.empty() ? &placeholder : tokens.data(),
                                                      offsets, &c, nullptr);
    if (s != PSX_OK) raise(s);
}

GenerationResult Generate(const NextTokenLogitsFn& model, const std::vector<int64_t>& prompt, const GenerationConfig& config) {
    ContextHolder& holder = thread_context();
    return run_loop(prompt, config, [&](const std::vector<int64_t>& tokens, int64_t n, double u, int64_t& token, float& log_prob) {
        const std::vector<float> logits = model(tokens);
        if (logits.empty()) throw std::invalid_argument("Generate: the model returned no logits");
        const psx_sampling_config c = to_c(config, n);
        const int64_t offsets[2] = {0, static_cast<int64_t>(tokens.size())};
        int32_t status = 0;
        const int64_t vocab = static_cast<int64_t>(logits.size());
        const psx_status s = psx_b200_sample_rows_host(holder.ctx, logits.data(), 1, vocab, vocab, tokens.data(), offsets, &c, &u,
                                                       &token, &log_prob, &status, nullptr);
        if (s != PSX_OK) raise(s);
    });
}

GenerationResult Generate(const DeviceNextTokenLogitsFn& model, const std::vector<int64_t>& prompt,
                          const GenerationConfig& config) {
    ContextHolder& holder = thread_context();
    auto cuda = [](cudaError_t e) {
        if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA error: ") + cudaGetErrorString(e));
    };
    if (!holder.uniform) {
        cuda(cudaMalloc(&holder.uniform, sizeof(double)));
        cuda(cudaMalloc(&holder.token, sizeof(int64_t)));
        cuda(cudaMalloc(&holder.log_prob, sizeof(float)));
        cuda(cudaMalloc(&holder.status, sizeof(int32_t)));
        cuda(cudaMalloc(&holder.offsets, 2 * sizeof(int64_t)));
    }
    cudaStream_t stream = static_cast<cudaStream_t>(psx_b200_ctx_stream(holder.ctx));
    size_t on_device = 0;  // ids of the sequence already copied
    return run_loop(prompt, config, [&](const std::vector<int64_t>& tokens, int64_t n, double u, int64_t& token, float& log_prob) {
        const DeviceLogits logits = model(tokens);
        if (!logits.data || logits.vocab <= 0) throw std::invalid_argument("Generate: the model returned no logits");
        if (n == 0) {  // the row must live on this thread's device
            cudaPointerAttributes where{};
            int device = -1;
            if (cudaPointerGetAttributes(&where, logits.data) == cudaSuccess && cudaGetDevice(&device) == cudaSuccess &&
                where.type == cudaMemoryTypeDevice && where.device != device) {
                throw std::invalid_argument("Generate: the logits live on another device than this thread's");
            }
        }
        if (logits.stream && logits.stream != static_cast<void*>(stream)) {  // after whatever the model enqueued there
            if (!holder.produced) cuda(cudaEventCreateWithFlags(&holder.produced, cudaEventDisableTiming));
            cuda(cudaEventRecord(holder.produced, static_cast<cudaStream_t>(logits.stream)));
            cuda(cudaStreamWaitEvent(stream, holder.produced, 0));
        }
        if (tokens.size() > holder.history_capacity) {  // grow and start over
            if (holder.history) cuda(cudaFree(holder.history));
            holder.history_capacity = std::max<size_t>(2 * tokens.size(), 1024);
            cuda(cudaMalloc(&holder.history, holder.history_capacity * sizeof(int64_t)));
            on_device = 0;
        }
        cuda(cudaMemcpyAsync(holder.history + on_device, tokens.data() + on_device, (tokens.size() - on_device) * sizeof(int64_t),
                             cudaMemcpyHostToDevice, stream));  // only what was appended since the last step
        on_device = tokens.size();
        const int64_t offsets[2] = {0, static_cast<int64_t>(tokens.size())};
        cuda(cudaMemcpyAsync(holder.offsets, offsets, sizeof(offsets), cudaMemcpyHostToDevice, stream));
        cuda(cudaMemcpyAsync(holder.uniform, &u, sizeof(double), cudaMemcpyHostToDevice, stream));
        const psx_sampling_config c = to_c(config, n);
        const psx_status s = psx_b200_sample_rows(holder.ctx, stream, logits.data, 1, logits.vocab, logits.vocab, holder.history,
                                                  holder.offsets, &c, holder.uniform, holder.token, holder.log_prob,
                                                  holder.status, nullptr);
        if (s != PSX_OK) raise(s);
        int32_t status = 0;
        cuda(cudaMemcpyAsync(&token, holder.token, sizeof(int64_t), cudaMemcpyDeviceToHost, stream));
        cuda(cudaMemcpyAsync(&log_prob, holder.log_prob, sizeof(float), cudaMemcpyDeviceToHost, stream));
        cuda(cudaMemcpyAsync(&status, holder.status, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
        cuda(cudaStreamSynchronize(stream));
        if (status == PSX_ROW_NON_FINITE) throw std::invalid_argument("Generate: the model returned a non-finite logit");
        if (status == PSX_ROW_ALL_REMOVED) throw std::invalid_argument("Generate: every token was removed");
        if (status != PSX_ROW_OK) throw std::runtime_error("psx_b200: the device path declined the row (status " + std::to_string(status) + ")");
    });
}

DeviceLmHead::DeviceLmHead(const std::vector<float>& weight, int64_t vocab, int64_t d_model, bool tied)
    : vocab_(vocab), d_model_(d_model), tied_(tied) {
    if (vocab <= 0 || d_model <= 0 || static_cast<int64_t>(weight.size()) != vocab * d_model) {
        throw std::invalid_argument("DeviceLmHead: the weight must hold vocab * d_model values");
    }
    thread_context();  // (sets up the device's context)
    auto cuda = [](cudaError_t e) {
        if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA error: ") + cudaGetErrorString(e));
    };
    cuda(cudaMalloc(&weight_, weight.size() * sizeof(float)));
    cuda(cudaMalloc(&hidden_, static_cast<size_t>(d_model) * sizeof(float)));
    cuda(cudaMalloc(&logits_, static_cast<size_t>((vocab + 3) / 4 * 4) * sizeof(float)));
    cuda(cudaMemcpy(weight_, weight.data(), weight.size() * sizeof(float), cudaMemcpyHostToDevice));
}

DeviceLmHead::~DeviceLmHead() {
    for (float* p : {weight_, hidden_, logits_}) {
        if (p) cudaFree(p);
    }
}

DeviceLogits DeviceLmHead::logits(const std::vector<float>& hidden) {
    if (static_cast<int64_t>(hidden.size()) != d_model_) {
        throw std::invalid_argument("DeviceLmHead: the hidden state must hold d_model values");
    }
    ContextHolder& holder = thread_context();
    cudaStream_t stream = static_cast<cudaStream_t>(psx_b200_ctx_stream(holder.ctx));
    // (the copy reads pageable host memory: it has left `hidden` when the call returns)
    if (cudaMemcpyAsync(hidden_, hidden.data(), hidden.size() * sizeof(float), cudaMemcpyHostToDevice, stream) != cudaSuccess) {
        throw std::runtime_error("CUDA error: copying the hidden state");
    }
    const psx_status s = psx_b200_lm_head_logits(holder.ctx, stream, hidden_, 1, d_model_, weight_, vocab_,
                                                 tied_ ? PSX_HEAD_VOCAB_BY_D : PSX_HEAD_D_BY_VOCAB, logits_, vocab_);
    if (s != PSX_OK) raise(s);
    return DeviceLogits{logits_, vocab_, stream};
}

DeviceNextTokenLogitsFn MakeDeviceLmHeadLogits(HiddenStateFn body, std::shared_ptr<DeviceLmHead> head) {
    if (!body || !head) throw std::invalid_argument("MakeDeviceLmHeadLogits: the body and the head must not be empty");
    return [body = std::move(body), head = std::move(head)](const std::vector<int64_t>& tokens) {
        return head->logits(body(tokens));
    };
}

}  // namespace pulsatrix
