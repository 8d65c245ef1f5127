// C entry points around the UNMODIFIED reference library -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// This file contains no reference code: it only calls the reference's public C++ API
// (pulsatrix::Generate, ProcessLogits, top_k, CPUBackend::top_k_rows, set_seed/next_seed,
// ShuffleSampler, PortableRng) so that Python tests and the benchmark's CPU-baseline leg can
// reach it through ctypes.  oracle/Makefile compiles it together with the reference's own
// sources, in place, into oracle/_ref/libpsx_ref.so.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "portable_random.hpp"  // private header of the reference, reached with -I<ref>/src
#include "psx_oracle.h"         // the shared C structs (psxo_config, psxo_step_info, status codes)
#include "pulsatrix/causal_lm.hpp"
#include "pulsatrix/cpu_backend.hpp"
#include "pulsatrix/determinism.hpp"
#include "pulsatrix/generation.hpp"
#include "pulsatrix/sampler.hpp"
#include "pulsatrix/top_k.hpp"

namespace {

pulsatrix::GenerationConfig ToConfig(const psxo_config* c) {
    pulsatrix::GenerationConfig g;
    g.max_new_tokens = c->max_new_tokens;
    g.min_new_tokens = c->min_new_tokens;
    g.eos_token_ids.assign(c->eos_token_ids, c->eos_token_ids + c->num_eos_token_ids);
    g.do_sample = c->do_sample != 0;
    g.temperature = c->temperature;
    g.top_k = c->top_k;
    g.top_p = c->top_p;
    g.min_p = c->min_p;
    g.repetition_penalty = c->repetition_penalty;
    return g;
}

// The reference reports every contract violation as std::invalid_argument; the message tells
// which one (src/generation.cpp:19-38,117-138).
int StatusOf(const std::invalid_argument& e) {
    const std::string what = e.what();
    if (what.find("GenerationConfig") != std::string::npos) return PSXO_BAD_CONFIG;
    if (what.find("prompt is empty") != std::string::npos) return PSXO_EMPTY_PROMPT;
    if (what.find("no logits") != std::string::npos) return PSXO_EMPTY_LOGITS;
    if (what.find("non-finite") != std::string::npos) return PSXO_NON_FINITE;
    if (what.find("every token was removed") != std::string::npos) return PSXO_ALL_REMOVED;
    return 99;
}

void RunRow(const float* logits, int64_t vocab, const int64_t* hist, int64_t hist_len, const psxo_config* c,
            uint64_t seed, psxo_step_info* info) {
    std::memset(info, 0, sizeof(*info));
    info->token = -1;
    info->draw_margin = INFINITY;
    info->top_p_margin = INFINITY;
    pulsatrix::GenerationConfig g = ToConfig(c);
    g.max_new_tokens = 1;
    g.seed = seed;
    const std::vector<int64_t> prompt(hist, hist + hist_len);
    auto model = [&](const std::vector<int64_t>&) { return std::vector<float>(logits, logits + vocab); };
    try {
        const pulsatrix::GenerationResult r = pulsatrix::Generate(model, prompt, g);
        info->token = r.new_tokens.at(0);
        info->log_prob = r.log_probs.at(0);
        info->status = PSXO_OK;
    } catch (const std::invalid_argument& e) {
        info->status = StatusOf(e);
    }
}

}  // namespace

extern "C" {

int psxref_process_logits(float* logits, int64_t vocab, const int64_t* tokens, int64_t num_tokens,
                          int64_t num_new_tokens, const psxo_config* c) {
    std::vector<float> l(logits, logits + vocab);
    const std::vector<int64_t> t(tokens, tokens + num_tokens);
    try {
        pulsatrix::ProcessLogits(l, t, num_new_tokens, ToConfig(c));
    } catch (const std::invalid_argument& e) {
        return StatusOf(e);
    }
    std::copy(l.begin(), l.end(), logits);
    return PSXO_OK;
}

// Independent rows, one Generate(max_new_tokens = 1, seed = seeds[r]) each, fanned over threads.
int psxref_rows(const float* logits, int64_t rows, int64_t vocab, int64_t row_stride, const int64_t* hist,
                const int64_t* offsets, const psxo_config* c, const uint64_t* seeds, int threads,
                psxo_step_info* infos) {
    threads = std::max(1, std::min<int>(threads, rows > 0 ? static_cast<int>(std::min<int64_t>(rows, 1024)) : 1));
    auto work = [&](int t) {
        for (int64_t r = t; r < rows; r += threads) {
            RunRow(logits + r * row_stride, vocab, hist + offsets[r], offsets[r + 1] - offsets[r], c, seeds[r],
                   &infos[r]);
        }
    };
    std::vector<std::thread> pool;
    for (int t = 1; t < threads; ++t) pool.emplace_back(work, t);
    work(0);
    for (auto& th : pool) th.join();
    int worst = PSXO_OK;
    for (int64_t r = 0; r < rows; ++r) {
        if (infos[r].status != PSXO_OK) worst = infos[r].status;
    }
    return worst;
}

// The whole of Generate() with the model given as a table: step s returns logits_steps[s].
int psxref_generate_table(const float* logits_steps, int64_t vocab, const int64_t* prompt, int64_t prompt_len,
                          const psxo_config* c, int32_t has_seed, uint64_t seed, int64_t* tokens_out,
                          float* log_probs_out, int64_t* n_new, int32_t* finished_eos) {
    *n_new = 0;
    *finished_eos = 0;
    pulsatrix::GenerationConfig g = ToConfig(c);
    if (has_seed) g.seed = seed;
    const std::vector<int64_t> p(prompt, prompt + prompt_len);
    int64_t step = 0;
    auto model = [&](const std::vector<int64_t>&) {
        const float* row = logits_steps + (step++) * vocab;
        return std::vector<float>(row, row + vocab);
    };
    try {
        const pulsatrix::GenerationResult r = pulsatrix::Generate(model, p, g);
        std::copy(r.tokens.begin(), r.tokens.end(), tokens_out);
        std::copy(r.log_probs.begin(), r.log_probs.end(), log_probs_out);
        *n_new = static_cast<int64_t>(r.new_tokens.size());
        *finished_eos = r.finish_reason == pulsatrix::FinishReason::Eos ? 1 : 0;
    } catch (const std::invalid_argument& e) {
        return StatusOf(e);
    }
    return PSXO_OK;
}

void psxref_top_k_rows(const float* in, float* values, float* indices, int64_t rows, int64_t cols, int64_t k,
                       int largest) {
    pulsatrix::CPUBackend cpu;
    cpu.top_k_rows(in, values, indices, static_cast<size_t>(rows), static_cast<size_t>(cols),
                   static_cast<size_t>(k), largest != 0);
}

void psxref_softmax_rows(const float* in, float* out, int64_t rows, int64_t cols) {
    pulsatrix::CPUBackend cpu;
    cpu.softmax_rows(in, out, static_cast<size_t>(rows), static_cast<size_t>(cols));
}

void psxref_logsumexp_rows(const float* in, float* out, int64_t rows, int64_t cols) {
    pulsatrix::CPUBackend cpu;
    cpu.logsumexp_rows(in, out, static_cast<size_t>(rows), static_cast<size_t>(cols));
}

void psxref_gather_rows(const float* table, const float* indices, float* out, int64_t count, int64_t dim) {
    pulsatrix::CPUBackend cpu;
    cpu.gather_rows(table, indices, out, static_cast<size_t>(count), static_cast<size_t>(dim));
}

// The core of MultiHeadAttentionModule::forward_cached (src/multihead_attention_module.cpp:562-586) through the
// reference's CPUBackend, call for call: gemm_ex, axpby, attention_mask_fill, softmax_rows, gemm.
void psxref_decode_attention(const float* q, const float* keys, const float* values, const float* key_keep, float* context,
                             int64_t batch, int64_t heads, int64_t kv_heads, int64_t q_len, int64_t head_dim, int64_t cached,
                             int64_t max_len, float scale, int causal, int64_t window) {
    pulsatrix::CPUBackend cpu;
    const int64_t total = cached + q_len, group = heads / kv_heads;
    const auto n = static_cast<size_t>(batch), h = static_cast<size_t>(heads), l = static_cast<size_t>(q_len),
               d = static_cast<size_t>(head_dim), t = static_cast<size_t>(total);
    std::vector<float> scores(n * h * l * t);
    for (int64_t nh = 0; nh < batch * heads; ++nh) {
        const int64_t kv = (nh / heads) * kv_heads + (nh % heads) / group;
        cpu.gemm_ex(q + nh * q_len * head_dim, false, keys + kv * max_len * head_dim, true, scores.data() + nh * q_len * total, l, d, t,
                    0.0f);
    }
    cpu.axpby(scale, scores.data(), 0.0f, nullptr, scores.data(), scores.size());
    if (causal || key_keep != nullptr) {
        cpu.attention_mask_fill(scores.data(), key_keep, n, h, l, t, causal != 0, static_cast<size_t>(cached),
                                static_cast<size_t>(window), std::numeric_limits<float>::lowest());
    }
    cpu.softmax_rows(scores.data(), scores.data(), n * h * l, t);
    for (int64_t nh = 0; nh < batch * heads; ++nh) {
        const int64_t kv = (nh / heads) * kv_heads + (nh % heads) / group;
        cpu.gemm(scores.data() + nh * q_len * total, values + kv * max_len * head_dim, context + nh * q_len * head_dim, l, t, d);
    }
}

// A tiny Hugging Face model of the reference's own fixtures (tests/fixtures/hf_tiny/<name>), decoded
// greedily for `steps` tokens after `prompt`: per step the input of the language-model head (the
// final norm's output at the last position, d floats), the logits the reference's head makes of it
// (vocab floats) and the token; the head's weight matrix (vocab x d when tied to the embedding, else
// the Linear's d x vocab); and what Generate() with the KV cache generates (`generated`, the tokens
// CausalLMTest.GreedyGenerationMatchesTransformers pins).  Buffers are the caller's; 0 on success.
int psxref_tiny_lm(const char* directory, const int64_t* prompt, int64_t prompt_len, int64_t steps, int64_t* d_out,
                   int64_t* vocab_out, int32_t* tied_out, float* weight, int64_t weight_capacity, float* hidden,
                   float* logits, int64_t* tokens, int64_t* generated) {
    try {
        pulsatrix::CPUBackend cpu;
        std::unique_ptr<pulsatrix::CausalLM> model = pulsatrix::LoadCausalLM(directory, &cpu);
        const int64_t d = model->config().hidden_size, vocab = model->config().vocab_size;
        *d_out = d;
        *vocab_out = vocab;
        const bool tied = model->lm_head() == nullptr;
        *tied_out = tied ? 1 : 0;
        pulsatrix::Tensor* w = tied ? model->embed_tokens().named_parameters().front().ref.value
                                    : model->lm_head()->named_parameters().front().ref.value;
        const std::vector<float> w_host = w->to_host_vector();
        if (static_cast<int64_t>(w_host.size()) != d * vocab || d * vocab > weight_capacity) return 3;
        std::memcpy(weight, w_host.data(), w_host.size() * sizeof(float));

        std::vector<int64_t> sequence(prompt, prompt + prompt_len);
        const int64_t last_layer = model->num_layers();
        for (int64_t s = 0; s < steps; ++s) {
            const int64_t length = static_cast<int64_t>(sequence.size());
            std::vector<float> last_hidden;
            model->set_hidden_state_hook([&](int64_t position, const pulsatrix::Tensor& x) {
                if (position == last_layer) {
                    const std::vector<float> all = x.to_host_vector();
                    last_hidden.assign(all.end() - d, all.end());
                }
                return x;
            });
            const std::vector<float> ids(sequence.begin(), sequence.end());
            const std::vector<float> out = model->forward(pulsatrix::Tensor(pulsatrix::Shape({1, length}), &cpu, ids)).to_host_vector();
            model->set_hidden_state_hook({});
            const float* row = out.data() + (length - 1) * vocab;
            std::memcpy(logits + s * vocab, row, static_cast<size_t>(vocab) * sizeof(float));
            const std::vector<float> normed =
                model->norm().forward(pulsatrix::Tensor(pulsatrix::Shape({1, d}), &cpu, last_hidden)).to_host_vector();
            std::memcpy(hidden + s * d, normed.data(), static_cast<size_t>(d) * sizeof(float));
            const int64_t token = std::max_element(row, row + vocab) - row;  // the first maximum
            tokens[s] = token;
            sequence.push_back(token);
        }
        pulsatrix::GenerationConfig g;
        g.max_new_tokens = steps;
        const pulsatrix::GenerationResult r =
            pulsatrix::Generate(model->next_token_logits(prompt_len + steps + 8), std::vector<int64_t>(prompt, prompt + prompt_len), g);
        for (int64_t s = 0; s < steps; ++s) generated[s] = s < static_cast<int64_t>(r.new_tokens.size()) ? r.new_tokens[s] : -1;
        return 0;
    } catch (const std::exception&) {
        return 2;
    }
}

// top_k() on a (rows, cols) CPU tensor: 0 on success, 1 when it throws std::invalid_argument.
int psxref_top_k(const float* in, float* values, float* indices, int64_t rows, int64_t cols, int64_t k,
                 int largest) {
    pulsatrix::CPUBackend cpu;
    try {
        const std::vector<float> data(in, in + rows * cols);
        pulsatrix::Tensor x(pulsatrix::Shape({rows, cols}), &cpu, data);
        const pulsatrix::TopKResult r = pulsatrix::top_k(x, k, largest != 0);
        std::copy(r.values.data(), r.values.data() + rows * k, values);
        std::copy(r.indices.data(), r.indices.data() + rows * k, indices);
    } catch (const std::invalid_argument&) {
        return 1;
    }
    return 0;
}

void psxref_set_seed(uint64_t seed) { pulsatrix::set_seed(seed); }
uint64_t psxref_next_seed(void) { return pulsatrix::next_seed(); }

// ShuffleSampler's visiting order over `epochs` consecutive reset(n) calls: out has epochs*n ids.
void psxref_shuffle_order(unsigned seed, int64_t n, int64_t epochs, int64_t* out) {
    pulsatrix::ShuffleSampler s(seed);
    for (int64_t e = 0; e < epochs; ++e) {
        s.reset(n);
        for (int64_t i = 0; i < n; ++i) out[e * n + i] = s.next().value();
    }
}

// PortableRng streams: n raw words, then n uniforms, then n gaussians from fresh generators.
void psxref_portable_streams(uint64_t seed, int64_t n, uint64_t* words, double* uniforms, double* gaussians) {
    pulsatrix::PortableRng a{seed}, b{seed}, c{seed};
    for (int64_t i = 0; i < n; ++i) {
        words[i] = a.next();
        uniforms[i] = b.uniform();
        gaussians[i] = c.gaussian();
    }
}

}  // extern "C"
