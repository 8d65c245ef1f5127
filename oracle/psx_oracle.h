/* CPU oracle for the token-sampling path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the reference's host algorithm, used only as the checker in tests,
 * in the smoke run and in the benchmark's CPU-baseline leg.  Nothing shipped may call it.
 * Every function names the reference lines it follows (paths are relative to the reference
 * project root).  Parity of this file with the reference is pinned by the reference's own
 * golden vectors (tests/generation_test.cpp:27-44, tests/top_k_test.cpp:49-144) and by running
 * the reference itself, compiled from its sources (see oracle/Makefile, target `ref`).
 */
#ifndef PSX_ORACLE_H
#define PSX_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* include/pulsatrix/generation.hpp:29-52, flattened to C. */
typedef struct psxo_config {
    int64_t max_new_tokens;
    int64_t min_new_tokens;
    const int64_t* eos_token_ids;
    int64_t num_eos_token_ids;
    int32_t do_sample;
    float temperature;
    int64_t top_k;
    float top_p;
    float min_p;
    float repetition_penalty;
} psxo_config;

enum {
    PSXO_OK = 0,
    PSXO_BAD_CONFIG = 1,     /* CheckConfig would throw */
    PSXO_EMPTY_PROMPT = 2,   /* "Generate: the prompt is empty" */
    PSXO_EMPTY_LOGITS = 3,   /* "Generate: the model returned no logits" */
    PSXO_NON_FINITE = 4,     /* "Generate: the model returned a non-finite logit" */
    PSXO_ALL_REMOVED = 5     /* "Generate: every token was removed" */
};

/* What one step decided, with the distances the parity report needs. */
typedef struct psxo_step_info {
    int64_t token;
    float log_prob;
    int32_t status;
    int64_t survivors;        /* entries of the processed row that are not -inf */
    double u;                 /* the uniform that was used (0 when greedy) */
    double draw_margin;       /* min |u - CDF edge| around the chosen bucket (inf when greedy) */
    double top_p_margin;      /* min |cum - (1 - top_p)| over the top-p walk (inf when off) */
} psxo_step_info;

/* src/generation.cpp:19-38 */
int psxo_check_config(const psxo_config* c);

/* src/generation.cpp:41-51; out has n doubles */
void psxo_softmax(const float* logits, int64_t n, double* out);

/* src/generation.cpp:55-112.  Returns PSXO_OK or PSXO_BAD_CONFIG.  top_p_margin may be NULL. */
int psxo_process_logits(float* logits, int64_t vocab, const int64_t* tokens, int64_t num_tokens,
                        int64_t num_new_tokens, const psxo_config* c, double* top_p_margin);

/* One iteration of the loop at src/generation.cpp:123-156 with the uniform given by the caller
 * (ignored when do_sample is 0).  `logits` is not modified.  `processed_out` (vocab floats) may
 * be NULL. */
int psxo_step(const float* logits, int64_t vocab, const int64_t* tokens, int64_t num_tokens,
              int64_t num_new_tokens, const psxo_config* c, double u, psxo_step_info* info,
              float* processed_out);

/* std::mt19937_64 as the C++ standard specifies it (src/generation.cpp:120,143 draw from it). */
typedef struct psxo_mt19937_64 {
    uint64_t mt[312];
    int index;
} psxo_mt19937_64;
void psxo_mt_seed(psxo_mt19937_64* g, uint64_t seed);
uint64_t psxo_mt_next(psxo_mt19937_64* g);
/* (engine() >> 11) * 2^-53, src/generation.cpp:143 */
double psxo_mt_uniform(psxo_mt19937_64* g);

/* The whole of Generate() (src/generation.cpp:114-164) for a model given as a table:
 * step s reads logits_steps + s*vocab.  tokens_out receives prompt then new tokens
 * (prompt_len + max_new_tokens capacity); returns the number of new tokens through n_new,
 * *finished_eos = 1 when an EOS id stopped it.  infos (max_new_tokens entries) may be NULL. */
int psxo_generate_table(const float* logits_steps, int64_t vocab, const int64_t* prompt, int64_t prompt_len,
                        const psxo_config* c, uint64_t seed, int64_t* tokens_out, float* log_probs_out,
                        int64_t* n_new, int32_t* finished_eos, psxo_step_info* infos);

/* Independent rows, each one Generate(max_new_tokens = 1) with its own seed: row r reads
 * logits + r*row_stride, history ids hist[offsets[r] .. offsets[r+1]).  Runs rows on `threads`
 * host threads (>= 1).  infos has `rows` entries. */
int psxo_rows(const float* logits, int64_t rows, int64_t vocab, int64_t row_stride, const int64_t* hist,
              const int64_t* offsets, const psxo_config* c, const uint64_t* seeds, int threads,
              psxo_step_info* infos);

/* src/top_k_math.hpp:19-47 by its stated order: NaN above every number, equal values keep the
 * lower column first; `largest == 0` mirrors it.  values/indices are (rows, k). */
void psxo_top_k_rows(const float* in, float* values, float* indices, int64_t rows, int64_t cols, int64_t k,
                     int largest);

/* src/cpu_backend.cpp:292-310,325-338,459-466: the float row primitives beside the path. */
void psxo_softmax_rows(const float* in, float* out, int64_t rows, int64_t cols);
void psxo_logsumexp_rows(const float* in, float* out, int64_t rows, int64_t cols);
void psxo_gather_rows(const float* table, const float* indices, float* out, int64_t count, int64_t dim);

/* MultiHeadAttentionModule::forward_cached, src/multihead_attention_module.cpp:562-586, with the CPU
 * backend's loops: scores by gemm_ex against the cached keys (src/cpu_backend.cpp:186-198), the score scale
 * (axpby, :272-277), attention_mask_fill (:429-443 with src/row_math.hpp:117-127), softmax_rows, context by
 * gemm against the cached values (:110-118).  q, context: (batch, heads, q_len, head_dim); keys, values:
 * (batch, kv_heads, max_len, head_dim) with cached + q_len positions filled; key_keep: (batch, cached +
 * q_len) or NULL. */
void psxo_decode_attention(const float* q, const float* keys, const float* values, const float* key_keep, float* context,
                           int64_t batch, int64_t heads, int64_t kv_heads, int64_t q_len, int64_t head_dim, int64_t cached,
                           int64_t max_len, float scale, int causal, int64_t window);

/* src/determinism.cpp:24-34: the global seed stream. */
void psxo_set_seed(uint64_t seed);
uint64_t psxo_next_seed(void);

/* src/portable_random.hpp:11-29 */
typedef struct psxo_portable_rng {
    uint64_t state;
} psxo_portable_rng;
uint64_t psxo_prng_next(psxo_portable_rng* g);
double psxo_prng_uniform(psxo_portable_rng* g);
double psxo_prng_gaussian(psxo_portable_rng* g);

/* Synthetic workload (not part of the reference): one row of fp32 logits
 *   logit[perm[r]] = (float)(gaussian * sigma - zeta * log(r + 1)),  r = 0 .. vocab-1,
 * with perm a Fisher-Yates permutation of [0, vocab) drawn from a psxo_portable_rng seeded with
 * `seed`, then `history_len` ids uniform in [0, vocab).  history may be NULL. */
void psxo_synth_row(uint64_t seed, int64_t vocab, double sigma, double zeta, float* logits, int64_t history_len,
                    int64_t* history);

#ifdef __cplusplus
}
#endif
#endif
