/** @file generation.hpp
 *  Token generation with the sampling step on the GPU.  Same API as the reference's
 *  include/pulsatrix/generation.hpp:25-96 (GenerationConfig, GenerationResult, ProcessLogits,
 *  Generate); the arithmetic of src/generation.cpp:55-164 runs in the sm_100a kernels behind
 *  include/psx_b200.h, bit-compatible with the reference's host code.  The module-stack adapters
 *  (MakeNextTokenLogits, MakeCachedNextTokenLogits) belong to the model side and are not here.
 */
#pragma once

#include <cstdint>
#include <functional>
#include <memory>
#include <optional>
#include <vector>

#include "pulsatrix/export.hpp"

namespace pulsatrix {

/** The model as generation sees it: token sequence in, next-token logits out (host vector). */
using NextTokenLogitsFn = std::function<std::vector<float>(const std::vector<int64_t>& tokens)>;

/** The same for a model whose logits stay on the GPU: returns a device pointer to `vocab` floats
 *  that stays valid until the next call.  Not in the reference (its adapter copies to the host).
 *  `stream` is the CUDA stream (a cudaStream_t) the model produced the logits on: Generate() orders
 *  its kernels after everything the model has enqueued there, so the model need not wait for its
 *  own head.  nullptr says the logits are complete when the model returns (the legacy default
 *  stream, which synchronises with every blocking stream, is not meant by it).  The logits must live
 *  on the device that was current when the calling thread first used this library. */
struct DeviceLogits {
    const float* data = nullptr;
    int64_t vocab = 0;
    void* stream = nullptr;
};
using DeviceNextTokenLogitsFn = std::function<DeviceLogits(const std::vector<int64_t>& tokens)>;

/** Decoding settings; the defaults decode greedily.  Field for field the reference's struct. */
struct GenerationConfig {
    int64_t max_new_tokens = 32;
    int64_t min_new_tokens = 0;          ///< EOS cannot be generated before this many new tokens
    std::vector<int64_t> eos_token_ids;  ///< generation stops after any of these (kept in the output)
    bool do_sample = false;              ///< false: first maximum; true: inverse-CDF draw
    float temperature = 1.0f;            ///< > 0, divides the logits
    int64_t top_k = 0;                   ///< 0 keeps all; ties at the k-th value all stay
    float top_p = 1.0f;                  ///< (0, 1]
    float min_p = 0.0f;                  ///< [0, 1]
    float repetition_penalty = 1.0f;     ///< > 0; applied to every id already in the sequence
    std::optional<uint64_t> seed;        ///< unset: next_seed()
};

enum class FinishReason { Eos, Length };

struct GenerationResult {
    std::vector<int64_t> tokens;      ///< prompt followed by the new tokens
    std::vector<int64_t> new_tokens;  ///< the new tokens only (EOS included if generated)
    std::vector<float> log_probs;     ///< log-softmax of the RAW logits at each new token
    FinishReason finish_reason = FinishReason::Length;
};

/** Repetition penalty, EOS ban before min_new_tokens, then (when sampling) temperature, top-k,
 *  top-p, min-p; removed entries become -infinity.  Runs on the GPU.
 *  @throws std::invalid_argument for an invalid config (same messages as the reference). */
PULSATRIX_API void ProcessLogits(std::vector<float>& logits, const std::vector<int64_t>& tokens,
                                 int64_t num_new_tokens, const GenerationConfig& config);

/** Generates up to max_new_tokens after @p prompt; each step's sampling runs on the GPU and draws
 *  from std::mt19937_64 exactly as the reference does, so a seed gives the reference's tokens.
 *  @throws std::invalid_argument for an empty prompt, an invalid config, empty or non-finite
 *          logits, or when every token was removed. */
[[nodiscard]] PULSATRIX_API GenerationResult Generate(const NextTokenLogitsFn& model,
                                                      const std::vector<int64_t>& prompt,
                                                      const GenerationConfig& config = {});

/** Generate() for a model that leaves its logits on the GPU: no per-token copy of the row. */
[[nodiscard]] PULSATRIX_API GenerationResult Generate(const DeviceNextTokenLogitsFn& model,
                                                      const std::vector<int64_t>& prompt,
                                                      const GenerationConfig& config = {});

/** The language-model head on the GPU: logits = hidden . W^T, what TiedLMHeadModule::forward
 *  (src/tied_lm_head_module.cpp:31-53) or an untied Linear head computes, with the weights resident
 *  on the device and the logits left there.  Every logit is accumulated in ascending feature order
 *  with product and sum each rounded to float, as the reference's CPU backend does
 *  (src/cpu_backend.cpp:188-196): the logits equal the reference's bit for bit.  Not in the
 *  reference as a class of its own (there the head is a Module of the model). */
class PULSATRIX_API DeviceLmHead {
public:
    /** @param weight vocab x d_model row-major when @p tied (the embedding table), else d_model x vocab
     *         (a Linear's weight).
     *  @throws std::invalid_argument when the sizes do not match. */
    DeviceLmHead(const std::vector<float>& weight, int64_t vocab, int64_t d_model, bool tied);
    ~DeviceLmHead();
    DeviceLmHead(const DeviceLmHead&) = delete;
    DeviceLmHead& operator=(const DeviceLmHead&) = delete;
    [[nodiscard]] int64_t vocab() const { return vocab_; }
    [[nodiscard]] int64_t d_model() const { return d_model_; }
    /** The logits of one hidden state (d_model floats, host): copied to the device, multiplied there;
     *  the result stays on the device, on the calling thread's context stream. */
    [[nodiscard]] DeviceLogits logits(const std::vector<float>& hidden);

private:
    int64_t vocab_, d_model_;
    bool tied_;
    float* weight_ = nullptr;
    float* hidden_ = nullptr;
    float* logits_ = nullptr;
};

/** The model up to the head as generation sees it: token sequence in, the final norm's output at
 *  the last position out (d_model floats). */
using HiddenStateFn = std::function<std::vector<float>(const std::vector<int64_t>& tokens)>;

/** A DeviceNextTokenLogitsFn made of a model body and a device head: what replaces the last two
 *  steps of the reference's cached adapter, head and copy to the host (src/generation.cpp:251-256).
 *  The logits never leave the GPU; per token only d_model floats go up and a token id comes back. */
[[nodiscard]] PULSATRIX_API DeviceNextTokenLogitsFn MakeDeviceLmHeadLogits(HiddenStateFn body, std::shared_ptr<DeviceLmHead> head);

}  // namespace pulsatrix
