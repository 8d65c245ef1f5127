/* psx_b200.h -- C ABI of the B200 (sm_100a) token-sampling library.
 *
 * A drop-in for one path of pulsatrix: logits processing + draw (ProcessLogits/Generate) and the
 * top-k selection primitive (DeviceBackend::top_k_rows).  Plain C types only: raw device or host
 * pointers, sizes, a CUDA stream passed as void*.  Each entry point names the reference interface
 * it replaces (paths relative to the pulsatrix project root).
 *
 * Conventions
 *   - Every function returns a psx_status (0 = ok).  psx_b200_last_error() gives the message of
 *     the calling thread's last failure.  There is no CPU fallback: without a CUDA device every
 *     compute call fails with PSX_ERR_CUDA.
 *   - A psx_ctx belongs to one device and one host thread at a time (like the reference's
 *     DeviceBackend, include/pulsatrix/cuda_backend.hpp:159-166).  It owns scratch memory that
 *     grows on demand; growing synchronises the device, steady-state calls do not allocate.
 *   - Device entry points are asynchronous on `stream` (a cudaStream_t; NULL is CUDA's default
 *     stream, as everywhere in CUDA); outputs are valid once that stream has been synchronised.
 *     Host entry points run on the context's own stream and synchronise before returning.
 */
#ifndef PSX_B200_H
#define PSX_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define PSX_API __attribute__((visibility("default")))
#else
#define PSX_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum psx_status {
    PSX_OK = 0,
    PSX_ERR_BAD_ARGUMENT = 1, /* the reference would throw std::invalid_argument (bad config, sizes) */
    PSX_ERR_CUDA = 2,         /* a CUDA call failed; the reference throws std::runtime_error */
    PSX_ERR_ROW_FAILED = 3,   /* host entry points only: some row's status is not PSX_ROW_OK */
    PSX_ERR_UNSUPPORTED = 4   /* a shape or setting outside what the kernels handle */
} psx_status;

/* Per-row outcome written to the `row_status` output of the sampling calls. */
typedef enum psx_row_status {
    PSX_ROW_OK = 0,
    PSX_ROW_NON_FINITE = 4,  /* "Generate: the model returned a non-finite logit" (src/generation.cpp:128-132) */
    PSX_ROW_ALL_REMOVED = 5, /* "Generate: every token was removed" (src/generation.cpp:136-138) */
    PSX_ROW_TOO_WIDE = 16,   /* more tokens survive the filters (or tie at a cut) than the device
                                path holds; nothing was drawn for this row.  Only where the whole row is
                                not at hand (the vocabulary-sharded merge): with the row on the GPU such a
                                row is decided from the row itself */
    PSX_ROW_DEVICE_TIMEOUT = 32 /* a bounded device-side wait (a bulk copy of a piece of the row into
                                shared memory) ran out; nothing was drawn for this row */
} psx_row_status;

/* GenerationConfig (include/pulsatrix/generation.hpp:29-52) without the loop fields, plus the
 * `num_new_tokens` argument of ProcessLogits (generation.hpp:83).  eos_token_ids is a HOST
 * pointer; it is copied during the call. */
typedef struct psx_sampling_config {
    int64_t min_new_tokens;
    int64_t num_new_tokens;
    const int64_t* eos_token_ids;
    int64_t num_eos_token_ids;
    int32_t do_sample;   /* 0: greedy (argmax, lower index wins); 1: sample */
    float temperature;   /* > 0, finite */
    int64_t top_k;       /* >= 0; 0 or >= vocab keeps all */
    float top_p;         /* (0, 1] */
    float min_p;         /* [0, 1] */
    float repetition_penalty; /* > 0, finite; 1 is off */
} psx_sampling_config;

/* Optional per-row diagnostics (device or host array of `rows` entries, may be NULL). */
typedef struct psx_row_diag {
    int32_t candidates;   /* entries the row pass handed to the survivor stage */
    int32_t survivors;    /* tokens left after top-k / top-p / min-p */
    double draw_margin;   /* min |u - edge| over the two CDF edges of the chosen bucket */
    double top_p_margin;  /* min |cumulative - (1 - top_p)| seen by the top-p walk */
} psx_row_diag;

typedef struct psx_ctx psx_ctx;

/* Library version, "major.minor.patch". */
PSX_API const char* psx_b200_version(void);
/* Message of the calling thread's most recent failure ("" if none). */
PSX_API const char* psx_b200_last_error(void);

/* Creates a context on CUDA device `device` (stream, scratch).  Replaces what the reference's
 * CUDABackend constructor sets up (src/cuda_backend.cu:24-29). */
PSX_API psx_status psx_b200_ctx_create(int device, psx_ctx** out);
PSX_API void psx_b200_ctx_destroy(psx_ctx* ctx);
/* The context's own non-blocking stream (a cudaStream_t), for callers that want one. */
PSX_API void* psx_b200_ctx_stream(psx_ctx* ctx);
/* cudaStreamSynchronize on `stream`. */
PSX_API psx_status psx_b200_sync(psx_ctx* ctx, void* stream);
/* Number of kernels this context has launched since it was created. */
PSX_API uint64_t psx_b200_launch_count(const psx_ctx* ctx);

/* Per-kernel device timing for benchmarks.  While enabled, every psx_b200_sample_rows call
 * brackets its row pass and its survivor stage with CUDA events on the launching stream.
 * psx_b200_ctx_read_timing synchronises those events, adds the elapsed milliseconds of all calls
 * since the last read into the two totals, reports the number of calls, and clears the record.
 * No counterpart in the reference. */
PSX_API psx_status psx_b200_ctx_enable_timing(psx_ctx* ctx, int enable);
PSX_API psx_status psx_b200_ctx_read_timing(psx_ctx* ctx, double* row_pass_ms, double* survivor_stage_ms,
                                            uint64_t* calls);

/* A promise about the calls that follow on this context (default 0: no promise).  ready != 0 says
 * that the inputs of a call (logits, history ids and offsets) are complete in device memory when
 * the call is made: they are not still being written by a kernel enqueued just before it on the
 * same stream that announces its completion early (programmatic dependent launch).  The row pass
 * then starts reading while the kernel before it in the stream -- usually the survivor stage of
 * the previous call -- is still running; it never writes before that kernel has finished.
 * Without the promise it waits for the kernel before it first.  No counterpart in the reference. */
PSX_API psx_status psx_b200_ctx_inputs_are_ready(psx_ctx* ctx, int ready);

/* How long a kernel of this context waits for one of its own asynchronous copies (a chunk of a row
 * on its way into shared memory) before it gives up: default one second.  A row whose wait ran out
 * reports PSX_ROW_DEVICE_TIMEOUT, nothing is drawn for it, and the context stays usable.  No
 * counterpart in the reference. */
PSX_API psx_status psx_b200_ctx_set_wait_limit(psx_ctx* ctx, uint64_t nanoseconds);
/* Test hook, never set it in production: while enabled, the row pass announces 16 bytes more per
 * copy than the copy delivers, so that its wait for the copy runs out (with no copy in flight)
 * and every row reports PSX_ROW_DEVICE_TIMEOUT.  It exists so that the give-up path of the bounded
 * wait can be tested without a fault.  No counterpart in the reference. */
PSX_API psx_status psx_b200_test_short_copy(psx_ctx* ctx, int enable);

/* Batched sampling step on device-resident logits: for every row, what one iteration of
 * Generate()'s loop computes (src/generation.cpp:124-156) -- finite check, raw log-softmax,
 * ProcessLogits (src/generation.cpp:55-112: repetition penalty, EOS ban, temperature, top-k,
 * top-p, min-p), then argmax or the inverse-CDF draw against `uniforms[row]`, and the chosen
 * token's log-probability under the unprocessed logits.  The reference has no batched or
 * device entry; this is what CUDA-resident callers of Generate() bind instead of copying the
 * row to the host (src/generation.cpp:248-256).
 *
 *   logits        device, rows x vocab fp32, row r at logits + r*row_stride (row_stride >= vocab)
 *   history_ids   device int64, the token sequence of every row back to back (prompt + generated)
 *   history_offsets device int64[rows+1]; row r owns history_ids[offsets[r] .. offsets[r+1])
 *                 (both may be NULL when repetition_penalty == 1)
 *   uniforms      device double[rows] in [0,1): the draw of each row, from the caller's
 *                 generator (psx_uniforms_mt19937_64 below reproduces the reference's); may be
 *                 NULL when do_sample == 0
 *   tokens        device int64[rows] out (-1 on a failed row)
 *   log_probs     device float[rows] out
 *   row_status    device int32[rows] out, a psx_row_status each
 *   diag          device psx_row_diag[rows] out, or NULL
 */
PSX_API psx_status psx_b200_sample_rows(psx_ctx* ctx, void* stream, const float* logits, int64_t rows, int64_t vocab,
                                int64_t row_stride, const int64_t* history_ids, const int64_t* history_offsets,
                                const psx_sampling_config* config, const double* uniforms, int64_t* tokens,
                                float* log_probs, int32_t* row_status, psx_row_diag* diag);

/* Only the first kernel of psx_b200_sample_rows (the pass that reads the logits), leaving its
 * output in the context's scratch: for benchmarks and profilers that time that kernel alone.
 * No counterpart in the reference. */
PSX_API psx_status psx_b200_row_pass_only(psx_ctx* ctx, void* stream, const float* logits, int64_t rows,
                                          int64_t vocab, int64_t row_stride, const int64_t* history_ids,
                                          const int64_t* history_offsets, const psx_sampling_config* config);

/* Benchmark aid: a kernel that only reads `bytes` bytes at `data` (16-byte aligned, device) with
 * 128-bit streaming loads and writes nothing (`sink`: one device float it practically never
 * touches).  Timed beside the row pass, it shows what reading a batch of that size can reach at
 * all.  No counterpart in the reference. */
PSX_API psx_status psx_b200_read_only_pass(void* stream, const void* data, size_t bytes, float* sink);

/* The same step as psx_b200_sample_rows for callers that must not allocate device memory: a
 * decode loop inside a serving process whose own pool already owns the GPU's memory (a cudaMalloc
 * from a plug-in would fail or stall), or a latency-critical loop that cannot afford cudaMalloc's
 * device-wide synchronisation.  It takes no context and calls no cudaMalloc / cudaFree: the
 * scratch between its kernels is a fixed array inside the library image on every GPU (about
 * 8.1 MiB).  Limits: rows * ceil(vocab / 16384) <= 1024 and at most 256 banned EOS ids, else
 * PSX_ERR_UNSUPPORTED.  The
 * first call on a device looks up that array's address and sets the kernels up: make it at
 * start-up, before any stream capture on that device and before the host process's own pool
 * takes the rest of the GPU's memory (the array and the kernels' code are placed on the device
 * when the first call loads them).  All calls share the array: calls that overlap on
 * the GPU race, so keep them stream-ordered per device.  Same inputs, outputs and statuses as
 * psx_b200_sample_rows (no diagnostics).  This entry point has no counterpart in the reference. */
PSX_API psx_status psx_b200_sample_rows_static(void* stream, const float* logits, int64_t rows, int64_t vocab,
                                               int64_t row_stride, const int64_t* history_ids,
                                               const int64_t* history_offsets, const psx_sampling_config* config,
                                               const double* uniforms, int64_t* tokens, float* log_probs,
                                               int32_t* row_status);

/* ProcessLogits (include/pulsatrix/generation.hpp:83, src/generation.cpp:55-112) for a batch of
 * device rows, in place: repetition penalty, EOS ban before min_new_tokens, and -- when sampling
 * -- temperature, top-k, top-p and min-p; removed entries become -infinity.  row_status (device,
 * may be NULL) receives PSX_ROW_OK, PSX_ROW_ALL_REMOVED (the row is all -infinity, as the
 * reference would leave it) or PSX_ROW_TOO_WIDE (the row is left unchanged).  Unlike Generate(),
 * and like the reference's ProcessLogits, non-finite input is not looked for.
 * psx_b200_process_logits_host does the same for host rows (copy in, process, copy back, sync). */
PSX_API psx_status psx_b200_process_logits(psx_ctx* ctx, void* stream, float* logits, int64_t rows, int64_t vocab,
                                           int64_t row_stride, const int64_t* history_ids,
                                           const int64_t* history_offsets, const psx_sampling_config* config,
                                           int32_t* row_status);
PSX_API psx_status psx_b200_process_logits_host(psx_ctx* ctx, float* logits, int64_t rows, int64_t vocab,
                                                int64_t row_stride, const int64_t* history_ids,
                                                const int64_t* history_offsets, const psx_sampling_config* config,
                                                int32_t* row_status);

/* The same step for callers that hold everything on the host, as the reference's
 * NextTokenLogitsFn does (include/pulsatrix/generation.hpp:25): copies inputs to the device,
 * runs psx_b200_sample_rows, copies results back and synchronises.  Returns
 * PSX_ERR_ROW_FAILED when any row_status is non-zero (outputs are still filled in). */
PSX_API psx_status psx_b200_sample_rows_host(psx_ctx* ctx, const float* logits, int64_t rows, int64_t vocab,
                                     int64_t row_stride, const int64_t* history_ids,
                                     const int64_t* history_offsets, const psx_sampling_config* config,
                                     const double* uniforms, int64_t* tokens, float* log_probs,
                                     int32_t* row_status, psx_row_diag* diag);

/* Vocabulary-sharded step, part 1 of 2 (no counterpart in the reference, which is single
 * device): this GPU holds columns [shard_begin, shard_begin + shard_cols) of every row.  Writes
 * one fixed-size record per row into `records` (device, rows * psx_b200_shard_record_bytes(config)
 * bytes): the shard's partial max / sum-exp and its local candidates with global column ids.
 * The caller all-gathers the records of all shards (NCCL) and passes them to part 2. */
PSX_API size_t psx_b200_shard_record_bytes(const psx_sampling_config* config);
PSX_API psx_status psx_b200_shard_scan(psx_ctx* ctx, void* stream, const float* shard_logits, int64_t rows,
                               int64_t shard_cols, int64_t row_stride, int64_t shard_begin, int64_t vocab,
                               const int64_t* history_ids, const int64_t* history_offsets,
                               const psx_sampling_config* config, void* records);
/* Part 2: merges `num_shards` gathered record sets (shard s at gathered + s*rows*record_bytes,
 * all in this GPU's own memory) and draws; every GPU that runs it gets the same result.  The
 * records carry the raw logits of their candidates, so the logits are not read again.
 * Sampling needs 0 < top_k < vocab here (greedy needs nothing).  Outputs as above. */
PSX_API psx_status psx_b200_shard_merge(psx_ctx* ctx, void* stream, const void* gathered, int32_t num_shards,
                                int64_t rows, int64_t vocab, const psx_sampling_config* config,
                                const double* uniforms, int64_t* tokens, float* log_probs, int32_t* row_status,
                                psx_row_diag* diag);

/* Part 2 for a subset of the rows: merges rows row_begin .. row_begin + row_count - 1 only, so that
 * the ranks can share the rows out among themselves and exchange the 16 bytes per row of results
 * afterwards.  `gathered` and `uniforms` are indexed by the absolute row as above; the outputs hold
 * the merged rows only, row_begin's at index 0.  No counterpart in the reference. */
PSX_API psx_status psx_b200_shard_merge_rows(psx_ctx* ctx, void* stream, const void* gathered, int32_t num_shards,
                                     int64_t rows, int64_t row_begin, int64_t row_count, int64_t vocab,
                                     const psx_sampling_config* config, const double* uniforms, int64_t* tokens,
                                     float* log_probs, int32_t* row_status, psx_row_diag* diag);

/* The vocabulary-sharded step without a library collective (no counterpart in the reference): the
 * ranks (one process per GPU, up to 8 GPUs of one box) write their records straight into the memory
 * of the rank that decides the row, over NVLink, and every rank's results straight into every
 * rank's memory; counters in the same memory say when a row's records, and a rank's results, are
 * complete.  Rank r decides rows r * ceil(rows / world) onwards.
 *
 *   psx_b200_exchange_create   allocates this rank's exchange buffer (device memory of ctx's GPU,
 *                              zeroed) for steps of `rows` rows under settings whose record size is
 *                              that of `config`, and writes its CUDA IPC handle
 *                              (psx_b200_exchange_handle_bytes() bytes) to `handle`;
 *   psx_b200_exchange_open     takes the handles of all ranks (world of them, in rank order, e.g.
 *                              all-gathered once through the caller's process group) and maps the
 *                              peers' buffers;
 *   psx_b200_exchange_sample   one step: row pass over this rank's columns, records to their ranks,
 *                              the draw for this rank's rows, results to every rank.  Asynchronous on
 *                              `stream`; every rank must call it the same number of times.  When the
 *                              stream has run, psx_b200_exchange_results (called after the step was
 *                              enqueued) points at `world` blocks of rows_per_rank rows each (rank
 *                              r's rows in block r): rows_per_rank tokens (int64), then as many
 *                              log-probs (float), then as many statuses (int32).  Two steps are in
 *                              flight at a time and the results alternate between two places: a step's
 *                              stay where they are until the step after the next one.  Arguments as
 *                              psx_b200_shard_scan / psx_b200_shard_merge.
 *   psx_b200_exchange_destroy  unmaps and frees; the caller makes sure (a barrier of its process
 *                              group) that no rank is still inside a step.
 *
 * Every device-side wait for another rank is bounded (one second unless changed): a row whose
 * records do not arrive, and the rows of a rank whose results do not, report
 * PSX_ROW_DEVICE_TIMEOUT, and the context stays usable.  psx_b200_exchange_test_wait sets that
 * bound and makes this rank's rows wait for `extra_arrivals` records more than will ever come:
 * it exists so that the give-up path can be tested without a rank that fails. */
typedef struct psx_exchange psx_exchange;
PSX_API size_t psx_b200_exchange_handle_bytes(void);
PSX_API psx_status psx_b200_exchange_create(psx_ctx* ctx, int32_t world, int32_t rank, int64_t rows,
                                            const psx_sampling_config* config, psx_exchange** out, void* handle);
PSX_API psx_status psx_b200_exchange_open(psx_exchange* exchange, const void* handles);
PSX_API void psx_b200_exchange_destroy(psx_exchange* exchange);
PSX_API psx_status psx_b200_exchange_sample(psx_exchange* exchange, void* stream, const float* shard_logits,
                                            int64_t shard_cols, int64_t row_stride, int64_t shard_begin, int64_t vocab,
                                            const int64_t* history_ids, const int64_t* history_offsets,
                                            const psx_sampling_config* config, const double* uniforms);
PSX_API psx_status psx_b200_exchange_results(const psx_exchange* exchange, const void** results, int64_t* rows_per_rank);
PSX_API psx_status psx_b200_exchange_test_wait(psx_exchange* exchange, uint64_t wait_limit_ns, uint32_t extra_arrivals);

/* Replaces DeviceBackend::top_k_rows (include/pulsatrix/device_backend.hpp:828-837; CUDA
 * implementation src/cuda_backend.cu:851-860, kernel src/gpu_kernels.cuh:1256-1262): per row of
 * a row-major (rows, cols) device matrix, the k largest (or smallest) values in rank order and
 * their column indices as whole-number floats.  NaN ranks above every number; equal values keep
 * the lower column first.  Requires 1 <= k <= cols <= 2^24 (top_k() validates the same,
 * src/top_k.cpp:10-21).  Up to k = 4096 the k winners are selected and sorted in shared memory;
 * beyond that the rows are sorted whole in the context's scratch memory.  Asynchronous on
 * `stream`. */
PSX_API psx_status psx_b200_top_k_rows(psx_ctx* ctx, void* stream, const float* in, float* values, float* indices,
                               size_t rows, size_t cols, size_t k, int largest);

/* The language-model head on the device: logits[m][j] = sum_p hidden[m][p] * w_j[p], what
 * TiedLMHeadModule::forward computes with gemm_ex(hidden, E^T) (src/tied_lm_head_module.cpp:31-53;
 * an untied head is a bias-free Linear: gemm(hidden, W), src/linear_module.cpp) right before
 * Generate() samples (src/generation.cpp:251-256 -- where the reference copies the row to the host).
 * hidden: device, rows x d fp32, contiguous.  weight: device fp32, vocab x d (PSX_HEAD_VOCAB_BY_D, the
 * tied embedding) or d x vocab (PSX_HEAD_D_BY_VOCAB, a Linear's weight).  Every logit is one float
 * accumulator that takes its products in ascending p, product and sum each rounded, as the
 * reference's CPU backend forms it (src/cpu_backend.cpp:188-196): the logits are the reference's bit
 * for bit.  psx_b200_lm_head_logits writes them to `logits` (row m at logits + m * row_stride);
 * psx_b200_lm_head_sample_rows keeps them in the context's scratch and samples them at once with
 * psx_b200_sample_rows (same remaining arguments, same outputs): the row never leaves the device. */
enum { PSX_HEAD_VOCAB_BY_D = 0, PSX_HEAD_D_BY_VOCAB = 1 };
PSX_API psx_status psx_b200_lm_head_logits(psx_ctx* ctx, void* stream, const float* hidden, int64_t rows, int64_t d,
                                           const float* weight, int64_t vocab, int32_t weight_layout, float* logits,
                                           int64_t row_stride);
PSX_API psx_status psx_b200_lm_head_sample_rows(psx_ctx* ctx, void* stream, const float* hidden, int64_t rows, int64_t d,
                                                const float* weight, int64_t vocab, int32_t weight_layout,
                                                const int64_t* history_ids, const int64_t* history_offsets,
                                                const psx_sampling_config* config, const double* uniforms,
                                                int64_t* tokens, float* log_probs, int32_t* row_status,
                                                psx_row_diag* diag);

/* Attention of the new positions over the KV cache: the core of MultiHeadAttentionModule::forward_cached
 * (src/multihead_attention_module.cpp:562-586) -- per (batch, head) scores = q . K^T (gemm_ex), times
 * `scale` (axpby; the module's score_scale(), 1 / sqrt(head_dim) by default, :190-192), masked entries set
 * to the lowest float (attention_mask_fill; src/row_math.hpp:117-127: with `causal`, key j is masked for
 * new position i when j > i + cached, or, with window > 0, when j + window <= i + cached; a key whose
 * key_keep entry is 0 is masked), softmax over the cached positions (softmax_rows), context = P . V (gemm)
 * -- in one pass over the cache.  q and context: (batch, heads, q_len, head_dim); keys and values: the
 * cache, (batch, kv_heads, max_len, head_dim), holding positions 0 .. cached + q_len - 1 (the new keys and
 * values already appended, :554-559); query head h reads kv head h / (heads / kv_heads) in place;
 * key_keep: (batch, cached + q_len) or null.  All device pointers, stream-asynchronous.  status (device,
 * may be null): bit 0 is set if a bounded device-side wait for a copy ran out.  Float sums in another
 * order than the reference's loops: within its 1e-4 CPU/GPU equivalence tolerance, not bit for bit.
 * Limits: (heads / kv_heads) * q_len <= 8, head_dim a multiple of 4 up to 256 (else PSX_ERR_UNSUPPORTED). */
PSX_API psx_status psx_b200_decode_attention(psx_ctx* ctx, void* stream, const float* q, const float* keys, const float* values,
                                             const float* key_keep, float* context, int64_t batch, int64_t heads,
                                             int64_t kv_heads, int64_t q_len, int64_t head_dim, int64_t cached, int64_t max_len,
                                             float scale, int32_t causal, int64_t window, int32_t* status);

/* Replace DeviceBackend::softmax_rows, logsumexp_rows and gather_rows
 * (include/pulsatrix/device_backend.hpp:456,465,596; CUDA implementations src/cuda_backend.cu with
 * the kernels src/gpu_kernels.cuh:315-365,665; CPU semantics src/cpu_backend.cpp:292-338,459-466)
 * for row-major device matrices.  softmax: out[r][j] = exp(in[r][j] - max_r) / sum, out may alias
 * in; logsumexp: out[r] = max_r + log(sum_j exp(in[r][j] - max_r)); both in float like the
 * reference (sums in a fixed tree: equal to the reference's sequential sums to rounding, its own
 * CPU/GPU tolerance is 1e-4).  gather: out[i][:] = table[indices[i]][:] with whole-number float
 * indices, bit-exact.  Asynchronous on `stream`. */
PSX_API psx_status psx_b200_softmax_rows(psx_ctx* ctx, void* stream, const float* in, float* out, size_t rows, size_t cols);
PSX_API psx_status psx_b200_logsumexp_rows(psx_ctx* ctx, void* stream, const float* in, float* out, size_t rows, size_t cols);
PSX_API psx_status psx_b200_gather_rows(psx_ctx* ctx, void* stream, const float* table, const float* indices, float* out,
                                        size_t count, size_t dim);

/* Host helpers: the uniform streams the reference draws from.
 * psx_uniforms_mt19937_64: out[i] = (std::mt19937_64(seeds[i])() >> 11) * 2^-53, the first draw
 * of Generate() for that seed (src/generation.cpp:120,143).
 * psx_uniforms_portable: out[i] = PortableRng{seeds[i]}.uniform() (src/portable_random.hpp:23). */
PSX_API void psx_uniforms_mt19937_64(const uint64_t* seeds, int64_t n, double* out);
PSX_API void psx_uniforms_portable(const uint64_t* seeds, int64_t n, double* out);

#ifdef __cplusplus
}
#endif
#endif /* PSX_B200_H */
