/* CPU oracle for the token-sampling path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * See psx_oracle.h.  Plain C99 + libm + pthreads.  Each function cites the reference lines it
 * restates (paths relative to the reference project root).
 */
#include "psx_oracle.h"

#include <float.h>
#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

#define NEG_INF (-INFINITY)

/* ---- src/generation.cpp:19-38 ------------------------------------------------------------ */
int psxo_check_config(const psxo_config* c) {
    if (c->max_new_tokens < 0 || c->min_new_tokens < 0) return PSXO_BAD_CONFIG;
    if (!(c->temperature > 0.0f) || isinf(c->temperature)) return PSXO_BAD_CONFIG;
    if (c->top_k < 0) return PSXO_BAD_CONFIG;
    if (!(c->top_p > 0.0f && c->top_p <= 1.0f)) return PSXO_BAD_CONFIG;
    if (!(c->min_p >= 0.0f && c->min_p <= 1.0f)) return PSXO_BAD_CONFIG;
    if (!(c->repetition_penalty > 0.0f) || isinf(c->repetition_penalty)) return PSXO_BAD_CONFIG;
    return PSXO_OK;
}

/* ---- src/generation.cpp:41-51 ------------------------------------------------------------
 * The max is taken over floats; each term is exp((double)l - max); the sum runs in index
 * order; -inf entries contribute an exact 0. */
void psxo_softmax(const float* logits, int64_t n, double* out) {
    float mx = logits[0];
    for (int64_t i = 1; i < n; ++i) {
        if (logits[i] > mx) mx = logits[i];
    }
    double sum = 0.0;
    for (int64_t i = 0; i < n; ++i) {
        out[i] = (logits[i] == NEG_INF) ? 0.0 : exp((double)logits[i] - mx);
        sum += out[i];
    }
    for (int64_t i = 0; i < n; ++i) out[i] /= sum;
}

/* k-th largest (1-based) of a scratch copy: what std::nth_element(greater) leaves at k-1
 * (src/generation.cpp:82-84).  Three-way quickselect; the value is unique whatever the method. */
static float kth_largest(float* a, int64_t n, int64_t k) {
    int64_t lo = 0, hi = n - 1, want = k - 1;
    uint64_t lcg = 0x2545F4914F6CDD1DULL;
    while (lo < hi) {
        lcg = lcg * 6364136223846793005ULL + 1442695040888963407ULL;
        const float pivot = a[lo + (int64_t)((lcg >> 33) % (uint64_t)(hi - lo + 1))];
        int64_t lt = lo, i = lo, gt = hi; /* [lo,lt) > pivot, [lt,i) == pivot, (gt,hi] < pivot */
        while (i <= gt) {
            if (a[i] > pivot) {
                float t = a[i]; a[i] = a[lt]; a[lt] = t; ++lt; ++i;
            } else if (a[i] < pivot) {
                float t = a[i]; a[i] = a[gt]; a[gt] = t; --gt;
            } else {
                ++i;
            }
        }
        if (want < lt) hi = lt - 1;
        else if (want > gt) lo = gt + 1;
        else return pivot;
    }
    return a[lo];
}

/* Ascending order of the row with equal values keeping the lower index first: the result of
 * std::stable_sort(iota, by logits[a] < logits[b]) at src/generation.cpp:93-95.  Stable LSD
 * radix sort on an order-preserving key; -0.0 and +0.0 compare equal in the reference, so both
 * get the same key. */
static uint32_t ascending_key(float x) {
    union { float f; uint32_t u; } v;
    v.f = x + 0.0f; /* -0.0 -> +0.0 */
    return (v.u & 0x80000000u) ? ~v.u : (v.u | 0x80000000u);
}

static void stable_ascending_order(const float* logits, int64_t n, uint32_t* order) {
    uint32_t* keys = (uint32_t*)malloc((size_t)n * sizeof(uint32_t));
    uint32_t* tmp = (uint32_t*)malloc((size_t)n * sizeof(uint32_t));
    for (int64_t i = 0; i < n; ++i) {
        keys[i] = ascending_key(logits[i]);
        order[i] = (uint32_t)i;
    }
    uint32_t* src = order;
    uint32_t* dst = tmp;
    for (int pass = 0; pass < 3; ++pass) {
        const int shift = pass * 11;
        const uint32_t mask = pass == 2 ? 0x3FFu : 0x7FFu;
        size_t count[2049];
        memset(count, 0, sizeof(count));
        for (int64_t i = 0; i < n; ++i) ++count[((keys[src[i]] >> shift) & mask) + 1];
        for (int b = 0; b < 2048; ++b) count[b + 1] += count[b];
        for (int64_t i = 0; i < n; ++i) dst[count[(keys[src[i]] >> shift) & mask]++] = src[i];
        uint32_t* t = src; src = dst; dst = t;
    }
    if (src != order) memcpy(order, src, (size_t)n * sizeof(uint32_t));
    free(keys);
    free(tmp);
}

/* ---- src/generation.cpp:55-112 ----------------------------------------------------------- */
int psxo_process_logits(float* logits, int64_t vocab, const int64_t* tokens, int64_t num_tokens,
                        int64_t num_new_tokens, const psxo_config* c, double* top_p_margin) {
    if (top_p_margin) *top_p_margin = INFINITY;
    if (psxo_check_config(c) != PSXO_OK) return PSXO_BAD_CONFIG;
    /* :59-68 repetition penalty on every id of the sequence that is inside the vocabulary */
    if (c->repetition_penalty != 1.0f) {
        unsigned char* seen = (unsigned char*)calloc((size_t)(vocab > 0 ? vocab : 1), 1);
        for (int64_t j = 0; j < num_tokens; ++j) {
            if (tokens[j] >= 0 && tokens[j] < vocab) seen[tokens[j]] = 1;
        }
        for (int64_t i = 0; i < vocab; ++i) {
            if (!seen[i]) continue;
            logits[i] = logits[i] < 0.0f ? logits[i] * c->repetition_penalty : logits[i] / c->repetition_penalty;
        }
        free(seen);
    }
    /* :69-73 EOS ban before min_new_tokens */
    if (num_new_tokens < c->min_new_tokens) {
        for (int64_t j = 0; j < c->num_eos_token_ids; ++j) {
            const int64_t e = c->eos_token_ids[j];
            if (e >= 0 && e < vocab) logits[e] = NEG_INF;
        }
    }
    /* :74-76 */
    if (!c->do_sample) return PSXO_OK;
    /* :77-79 temperature, a float divide */
    if (c->temperature != 1.0f) {
        for (int64_t i = 0; i < vocab; ++i) logits[i] /= c->temperature;
    }
    /* :80-88 top-k keeps everything >= the k-th largest value */
    if (c->top_k > 0 && c->top_k < vocab) {
        float* scratch = (float*)malloc((size_t)vocab * sizeof(float));
        memcpy(scratch, logits, (size_t)vocab * sizeof(float));
        const float kth = kth_largest(scratch, vocab, c->top_k);
        free(scratch);
        for (int64_t i = 0; i < vocab; ++i) {
            if (logits[i] < kth) logits[i] = NEG_INF;
        }
    }
    /* :89-103 top-p: ascending cumulative probability, the largest entry always stays */
    if (c->top_p < 1.0f) {
        double* p = (double*)malloc((size_t)vocab * sizeof(double));
        uint32_t* order = (uint32_t*)malloc((size_t)vocab * sizeof(uint32_t));
        psxo_softmax(logits, vocab, p);
        stable_ascending_order(logits, vocab, order);
        const double limit = 1.0 - (double)c->top_p;
        double cumulative = 0.0;
        for (int64_t r = 0; r + 1 < vocab; ++r) {
            cumulative += p[order[r]];
            if (top_p_margin && p[order[r]] > 0.0) {
                const double d = fabs(cumulative - limit);
                if (d < *top_p_margin) *top_p_margin = d;
            }
            if (cumulative <= limit) logits[order[r]] = NEG_INF;
        }
        free(p);
        free(order);
    }
    /* :104-111 min-p relative to the most likely token, which itself always stays */
    if (c->min_p > 0.0f) {
        double* p = (double*)malloc((size_t)vocab * sizeof(double));
        psxo_softmax(logits, vocab, p);
        int64_t best = 0;
        for (int64_t i = 1; i < vocab; ++i) {
            if (p[i] > p[best]) best = i;
        }
        const double top = p[best];
        for (int64_t i = 0; i < vocab; ++i) {
            if (i != best && p[i] < c->min_p * top) logits[i] = NEG_INF;
        }
        free(p);
    }
    return PSXO_OK;
}

/* ---- src/generation.cpp:123-156, one iteration ------------------------------------------- */
int psxo_step(const float* logits, int64_t vocab, const int64_t* tokens, int64_t num_tokens,
              int64_t num_new_tokens, const psxo_config* c, double u, psxo_step_info* info,
              float* processed_out) {
    memset(info, 0, sizeof(*info));
    info->token = -1;
    info->draw_margin = INFINITY;
    info->top_p_margin = INFINITY;
    int rc = psxo_check_config(c);
    if (rc == PSXO_OK && vocab <= 0) rc = PSXO_EMPTY_LOGITS; /* :125-127 */
    if (rc == PSXO_OK) {
        for (int64_t i = 0; i < vocab; ++i) { /* :128-132 */
            if (!isfinite(logits[i])) { rc = PSXO_NON_FINITE; break; }
        }
    }
    if (rc != PSXO_OK) { info->status = rc; return rc; }

    double* raw = (double*)malloc((size_t)vocab * sizeof(double));
    float* work = (float*)malloc((size_t)vocab * sizeof(float));
    psxo_softmax(logits, vocab, raw); /* :133, before any processing */
    memcpy(work, logits, (size_t)vocab * sizeof(float));
    psxo_process_logits(work, vocab, tokens, num_tokens, num_new_tokens, c, &info->top_p_margin); /* :134 */

    int64_t best = 0, alive = 0; /* :135 first maximum */
    for (int64_t i = 0; i < vocab; ++i) {
        if (work[i] > work[best]) best = i;
        if (work[i] != NEG_INF) ++alive;
    }
    info->survivors = alive;
    if (work[best] == NEG_INF) { /* :136-138 */
        rc = PSXO_ALL_REMOVED;
    } else {
        int64_t chosen = best;
        if (c->do_sample) { /* :140-152 inverse CDF in index order over the non-zero entries */
            double* p = (double*)malloc((size_t)vocab * sizeof(double));
            psxo_softmax(work, vocab, p);
            double cumulative = 0.0, before = 0.0;
            for (int64_t i = 0; i < vocab; ++i) {
                if (p[i] == 0.0) continue;
                before = cumulative;
                cumulative += p[i];
                chosen = i;
                if (u < cumulative) break;
            }
            info->u = u;
            const double lo = fabs(u - before), hi = fabs(u - cumulative);
            info->draw_margin = before == 0.0 ? hi : (lo < hi ? lo : hi);
            free(p);
        }
        info->token = chosen;
        info->log_prob = (float)log(raw[chosen]); /* :156 */
    }
    if (processed_out) memcpy(processed_out, work, (size_t)vocab * sizeof(float));
    free(raw);
    free(work);
    info->status = rc;
    return rc;
}

/* ---- std::mt19937_64 (ISO C++ [rand.predef]: w=64 n=312 m=156 r=31) ---------------------- */
void psxo_mt_seed(psxo_mt19937_64* g, uint64_t seed) {
    g->mt[0] = seed;
    for (int i = 1; i < 312; ++i) {
        g->mt[i] = 6364136223846793005ULL * (g->mt[i - 1] ^ (g->mt[i - 1] >> 62)) + (uint64_t)i;
    }
    g->index = 312;
}

uint64_t psxo_mt_next(psxo_mt19937_64* g) {
    if (g->index >= 312) {
        for (int i = 0; i < 312; ++i) {
            const uint64_t x = (g->mt[i] & 0xFFFFFFFF80000000ULL) | (g->mt[(i + 1) % 312] & 0x7FFFFFFFULL);
            g->mt[i] = g->mt[(i + 156) % 312] ^ (x >> 1) ^ ((x & 1ULL) ? 0xB5026F5AA96619E9ULL : 0ULL);
        }
        g->index = 0;
    }
    uint64_t y = g->mt[g->index++];
    y ^= (y >> 29) & 0x5555555555555555ULL;
    y ^= (y << 17) & 0x71D67FFFEDA60000ULL;
    y ^= (y << 37) & 0xFFF7EEE000000000ULL;
    y ^= (y >> 43);
    return y;
}

double psxo_mt_uniform(psxo_mt19937_64* g) { return (double)(psxo_mt_next(g) >> 11) * 0x1.0p-53; }

/* ---- src/generation.cpp:114-164 with the model given as a table of rows ------------------- */
int psxo_generate_table(const float* logits_steps, int64_t vocab, const int64_t* prompt, int64_t prompt_len,
                        const psxo_config* c, uint64_t seed, int64_t* tokens_out, float* log_probs_out,
                        int64_t* n_new, int32_t* finished_eos, psxo_step_info* infos) {
    *n_new = 0;
    *finished_eos = 0;
    if (psxo_check_config(c) != PSXO_OK) return PSXO_BAD_CONFIG;
    if (prompt_len <= 0) return PSXO_EMPTY_PROMPT; /* :117-119 */
    psxo_mt19937_64 engine;
    psxo_mt_seed(&engine, seed); /* :120 one engine per call */
    memcpy(tokens_out, prompt, (size_t)prompt_len * sizeof(int64_t));
    int64_t len = prompt_len;
    for (int64_t step = 0; step < c->max_new_tokens; ++step) {
        psxo_step_info local;
        psxo_step_info* info = infos ? &infos[step] : &local;
        /* The reference validates and processes before it draws, so the engine only advances
         * on a step that reaches the draw (:143). */
        psxo_mt19937_64 probe = engine;
        const double u = c->do_sample ? psxo_mt_uniform(&probe) : 0.0;
        const int rc = psxo_step(logits_steps + step * vocab, vocab, tokens_out, len, step, c, u, info, NULL);
        if (rc != PSXO_OK) return rc;
        if (c->do_sample) engine = probe;
        tokens_out[len++] = info->token;
        log_probs_out[step] = info->log_prob;
        *n_new = step + 1;
        for (int64_t j = 0; j < c->num_eos_token_ids; ++j) { /* :157-160 */
            if (c->eos_token_ids[j] == info->token) { *finished_eos = 1; return PSXO_OK; }
        }
    }
    return PSXO_OK;
}

/* ---- independent rows ---------------------------------------------------------------------- */
typedef struct rows_job {
    const float* logits; int64_t rows, vocab, row_stride;
    const int64_t* hist; const int64_t* offsets;
    const psxo_config* c; const uint64_t* seeds;
    psxo_step_info* infos;
    int thread, threads;
} rows_job;

static void* rows_worker(void* arg) {
    rows_job* j = (rows_job*)arg;
    for (int64_t r = j->thread; r < j->rows; r += j->threads) {
        const int64_t h0 = j->offsets[r], h1 = j->offsets[r + 1];
        if (h1 <= h0) { /* Generate() rejects an empty prompt, src/generation.cpp:117-119 */
            memset(&j->infos[r], 0, sizeof(psxo_step_info));
            j->infos[r].token = -1;
            j->infos[r].status = PSXO_EMPTY_PROMPT;
            continue;
        }
        psxo_mt19937_64 engine;
        psxo_mt_seed(&engine, j->seeds[r]);
        const double u = j->c->do_sample ? psxo_mt_uniform(&engine) : 0.0;
        psxo_step(j->logits + r * j->row_stride, j->vocab, j->hist + h0, h1 - h0, 0, j->c, u, &j->infos[r], NULL);
    }
    return NULL;
}

int psxo_rows(const float* logits, int64_t rows, int64_t vocab, int64_t row_stride, const int64_t* hist,
              const int64_t* offsets, const psxo_config* c, const uint64_t* seeds, int threads,
              psxo_step_info* infos) {
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    if (threads > rows) threads = rows > 0 ? (int)rows : 1;
    pthread_t tid[256];
    rows_job jobs[256];
    for (int t = 0; t < threads; ++t) {
        rows_job j = {logits, rows, vocab, row_stride, hist, offsets, c, seeds, infos, t, threads};
        jobs[t] = j;
        if (t > 0) pthread_create(&tid[t], NULL, rows_worker, &jobs[t]);
    }
    rows_worker(&jobs[0]);
    for (int t = 1; t < threads; ++t) pthread_join(tid[t], NULL);
    int worst = PSXO_OK;
    for (int64_t r = 0; r < rows; ++r) {
        if (infos[r].status != PSXO_OK) worst = infos[r].status;
    }
    return worst;
}

/* ---- src/top_k_math.hpp:19-47 by its stated order ------------------------------------------ */
typedef struct rank_item {
    uint32_t key; /* larger key ranks first */
    uint32_t col;
} rank_item;

static uint32_t rank_key(float x, int largest) {
    uint32_t k = (x != x) ? 0xFFFFFFFFu : ascending_key(x); /* NaN above every number (:19) */
    return largest ? k : ~k;                                /* :22-24 mirrored */
}

static int rank_cmp(const void* a, const void* b) {
    const rank_item* x = (const rank_item*)a;
    const rank_item* y = (const rank_item*)b;
    if (x->key != y->key) return x->key > y->key ? -1 : 1;
    return x->col < y->col ? -1 : (x->col > y->col ? 1 : 0); /* ties keep scan order */
}

void psxo_top_k_rows(const float* in, float* values, float* indices, int64_t rows, int64_t cols, int64_t k,
                     int largest) {
    rank_item* items = (rank_item*)malloc((size_t)cols * sizeof(rank_item));
    for (int64_t r = 0; r < rows; ++r) {
        const float* row = in + r * cols;
        for (int64_t j = 0; j < cols; ++j) {
            items[j].key = rank_key(row[j], largest);
            items[j].col = (uint32_t)j;
        }
        qsort(items, (size_t)cols, sizeof(rank_item), rank_cmp);
        for (int64_t j = 0; j < k; ++j) {
            values[r * k + j] = row[items[j].col];
            indices[r * k + j] = (float)items[j].col;
        }
    }
    free(items);
}

/* ---- src/cpu_backend.cpp:292-310 (softmax_rows), :325-338 (logsumexp_rows), :459-466 (gather_rows) ---- */
void psxo_softmax_rows(const float* in, float* out, int64_t rows, int64_t cols) {
    for (int64_t r = 0; r < rows; ++r) {
        const float* x = in + r * cols;
        float* y = out + r * cols;
        float row_max = x[0];
        for (int64_t j = 1; j < cols; ++j) row_max = x[j] > row_max ? x[j] : row_max; /* std::max(a, b): b when a < b */
        float exp_sum = 0.0f;
        for (int64_t j = 0; j < cols; ++j) {
            const float e = expf(x[j] - row_max);
            y[j] = e;
            exp_sum += e;
        }
        for (int64_t j = 0; j < cols; ++j) y[j] /= exp_sum;
    }
}

void psxo_logsumexp_rows(const float* in, float* out, int64_t rows, int64_t cols) {
    for (int64_t r = 0; r < rows; ++r) {
        const float* x = in + r * cols;
        float row_max = x[0];
        for (int64_t j = 1; j < cols; ++j) row_max = x[j] > row_max ? x[j] : row_max;
        float exp_sum = 0.0f;
        for (int64_t j = 0; j < cols; ++j) exp_sum += expf(x[j] - row_max);
        out[r] = row_max + logf(exp_sum);
    }
}

void psxo_gather_rows(const float* table, const float* indices, float* out, int64_t count, int64_t dim) {
    for (int64_t i = 0; i < count; ++i) {
        const float* row = table + (size_t)indices[i] * (size_t)dim;
        for (int64_t d = 0; d < dim; ++d) out[i * dim + d] = row[d];
    }
}

/* ---- src/determinism.cpp:14-34 --------------------------------------------------------------- */
static uint64_t g_seed = 0, g_counter = 0;

static uint64_t splitmix_finalize(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

void psxo_set_seed(uint64_t seed) { g_seed = seed; g_counter = 0; }

uint64_t psxo_next_seed(void) {
    const uint64_t index = g_counter++;
    return splitmix_finalize(g_seed + 0x9E3779B97F4A7C15ULL * (index + 1));
}

/* ---- src/portable_random.hpp:11-29 ----------------------------------------------------------- */
uint64_t psxo_prng_next(psxo_portable_rng* g) {
    g->state += 0x9E3779B97F4A7C15ULL;
    return splitmix_finalize(g->state);
}

double psxo_prng_uniform(psxo_portable_rng* g) {
    return ((double)(psxo_prng_next(g) >> 11) + 0.5) / (double)(1ULL << 53);
}

double psxo_prng_gaussian(psxo_portable_rng* g) {
    const double two_pi = 6.28318530717958647692;
    const double a = psxo_prng_uniform(g);
    const double b = psxo_prng_uniform(g);
    return sqrt(-2.0 * log(a)) * cos(two_pi * b);
}

/* ---- synthetic workload (not in the reference) ------------------------------------------------ */
void psxo_synth_row(uint64_t seed, int64_t vocab, double sigma, double zeta, float* logits, int64_t history_len,
                    int64_t* history) {
    psxo_portable_rng g = {seed};
    uint32_t* perm = (uint32_t*)malloc((size_t)vocab * sizeof(uint32_t));
    for (int64_t i = 0; i < vocab; ++i) perm[i] = (uint32_t)i;
    for (int64_t i = vocab - 1; i > 0; --i) {
        const int64_t j = (int64_t)(psxo_prng_next(&g) % (uint64_t)(i + 1));
        const uint32_t t = perm[i]; perm[i] = perm[j]; perm[j] = t;
    }
    for (int64_t r = 0; r < vocab; ++r) {
        logits[perm[r]] = (float)(psxo_prng_gaussian(&g) * sigma - zeta * log((double)(r + 1)));
    }
    for (int64_t j = 0; j < history_len; ++j) {
        history[j] = (int64_t)(psxo_prng_next(&g) % (uint64_t)vocab);
    }
    free(perm);
}

/* src/multihead_attention_module.cpp:562-586 over the CPU backend's loops (see psx_oracle.h). */
void psxo_decode_attention(const float* q, const float* keys, const float* values, const float* key_keep, float* context,
                           int64_t batch, int64_t heads, int64_t kv_heads, int64_t q_len, int64_t head_dim, int64_t cached,
                           int64_t max_len, float scale, int causal, int64_t window) {
    const int64_t total = cached + q_len, group = heads / kv_heads;
    float* scores = (float*)malloc((size_t)(q_len * total) * sizeof(float));
    for (int64_t nh = 0; nh < batch * heads; ++nh) {
        const int64_t b = nh / heads, kv = b * kv_heads + (nh % heads) / group; /* :563 */
        const float* a = q + nh * q_len * head_dim;
        const float* k = keys + kv * max_len * head_dim;
        const float* v = values + kv * max_len * head_dim;
        for (int64_t i = 0; i < q_len; ++i) {
            for (int64_t j = 0; j < total; ++j) { /* gemm_ex, B transposed: src/cpu_backend.cpp:188-196 */
                float acc = 0.0f;
                for (int64_t p = 0; p < head_dim; ++p) acc += a[i * head_dim + p] * k[j * head_dim + p];
                scores[i * total + j] = acc;
            }
        }
        for (int64_t x = 0; x < q_len * total; ++x) scores[x] = scale * scores[x]; /* axpby with beta == 0: :274-276 */
        for (int64_t i = 0; i < q_len; ++i) { /* attention_mask_fill: :429-443, src/row_math.hpp:117-127 */
            for (int64_t j = 0; j < total; ++j) {
                int masked = 0;
                if (causal && j > i + cached) masked = 1;
                if (causal && window > 0 && j + window <= i + cached) masked = 1;
                if (!masked && key_keep != NULL && key_keep[b * total + j] == 0.0f) masked = 1;
                if (masked) scores[i * total + j] = -FLT_MAX; /* std::numeric_limits<float>::lowest() */
            }
        }
        psxo_softmax_rows(scores, scores, q_len, total); /* :578 */
        for (int64_t i = 0; i < q_len; ++i) { /* gemm: :110-118 (one accumulator per output, products in order) */
            for (int64_t d = 0; d < head_dim; ++d) {
                float acc = 0.0f;
                for (int64_t j = 0; j < total; ++j) acc += scores[i * total + j] * v[j * head_dim + d];
                context[(nh * q_len + i) * head_dim + d] = acc;
            }
        }
    }
    free(scores);
}
