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
#include <optional>
#include <vector>

#include "pulsatrix/export.hpp"

namespace pulsatrix {

/** The model as generation sees it: token sequence in, next-token logits out (host vector). */
using NextTokenLogitsFn = std::function<std::vector<float>(const std::vector<int64_t>& tokens)>;

/** The same for a model whose logits stay on the GPU: returns a device pointer to `vocab` floats
 *  that stays valid until the next call.  Not in the reference (its adapter copies to the host). */
struct DeviceLogits {
    const float* data = nullptr;
    int64_t vocab = 0;
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

}  // namespace pulsatrix
