// psx_b200_sample_rows_static: the batched sampling step for callers that must not allocate.
//
// Who cannot allocate: a decode loop that lives inside a serving process whose own memory pool
// already owns (nearly) all of the GPU's memory, so that a cudaMalloc from a plug-in either fails
// or takes memory the pool believes it has; and any latency-critical loop for which cudaMalloc is
// off limits because it synchronises the whole device and stalls every other stream.  The regular
// entry point (psx_b200_sample_rows) grows a context's scratch with cudaMalloc the first time it
// sees a bigger batch; this one never does.  Its scratch -- the row pass's per-part records and
// candidate lists that the survivor stage reads -- is a fixed array that is part of the loaded
// library image on every GPU (kStaticParts parts, about 8.1 MiB, held until the process exits).
//
// Consequences the caller must know:
//   * rows * parts-per-row may not exceed kStaticParts (a part is 16384 logits of one row; a
//     64 x 151,936 batch is 640 parts); bigger batches and more than kStaticBanned EOS ids are
//     refused with PSX_ERR_UNSUPPORTED, nothing is launched;
//   * the first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and lifts the two kernels' shared-memory limits; make that first call
//     at start-up: before any stream capture on that device, and before the host process's own
//     pool takes the rest of the GPU's memory -- under CUDA's lazy module loading the array's
//     8.1 MiB and the kernels' code are placed on the device when the first call loads them;
//   * every call uses the same array.  Nothing in it has to start at zero: the row pass rewrites
//     every record and every list count of the batch before the survivor stage reads them, and
//     list slots beyond a count are never used, so stale contents of an earlier call are
//     harmless.  But two calls that overlap on the GPU (different streams, or different host
//     threads) race on it: keep calls stream-ordered one after another per device.
#include <mutex>
#include <string>

#include "../../include/psx_b200.h"
#include "merge_rows.cuh"
#include "sample_plan.cuh"
#include "scan_rows.cuh"

namespace {

constexpr int kStaticParts = 1024;  // (row, part) pairs one call may produce
constexpr int kStaticBanned = 256;  // EOS ids one call may ban
constexpr int kMaxDevices = 64;

struct StaticScratch {
    psx::PartStats stats[kStaticParts];
    uint32_t part_counts[kStaticParts];
    uint2 candidates[(size_t)kStaticParts * psx::kPartCap];
    int64_t banned[kStaticBanned];
};

// Lives in device memory of every GPU that loads the library.  In host code this name is only a
// handle for cudaGetSymbolAddress; kernels get the looked-up address.
static __device__ __align__(256) unsigned char g_scratch[sizeof(StaticScratch)];

struct DeviceSetup {
    bool done = false;
    StaticScratch* scratch = nullptr;
};
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;

}  // namespace

// Stores the calling thread's error message where psx_b200_last_error() finds it (c_abi.cu).
namespace psx_internal {
psx_status set_error(psx_status code, const std::string& message);
}

#define PSX_STATIC_CUDA(call)                                                                                  \
    do {                                                                                                       \
        const cudaError_t psx_cuda_result = (call);                                                            \
        if (psx_cuda_result != cudaSuccess) {                                                                  \
            return psx_internal::set_error(PSX_ERR_CUDA, std::string("CUDA error: ") +                         \
                                                             cudaGetErrorString(psx_cuda_result) + " at " __FILE__ \
                                                             ":" + std::to_string(__LINE__));                  \
        }                                                                                                      \
    } while (0)

extern "C" psx_status psx_b200_sample_rows_static(void* stream_ptr, const float* logits, int64_t rows, int64_t vocab,
                                                  int64_t row_stride, const int64_t* history_ids,
                                                  const int64_t* history_offsets, const psx_sampling_config* c,
                                                  const double* uniforms, int64_t* tokens, float* log_probs,
                                                  int32_t* row_status) {
    using psx_internal::set_error;
    // ---- the reference's argument checks (src/generation.cpp:19-38) -------------------------------
    if (!c) return set_error(PSX_ERR_BAD_ARGUMENT, "psx_b200: config is null");
    if (c->min_new_tokens < 0) {
        return set_error(PSX_ERR_BAD_ARGUMENT, "GenerationConfig: max_new_tokens and min_new_tokens must not be negative");
    }
    if (!(c->temperature > 0.0f) || c->temperature > 3.4028235e38f) {
        return set_error(PSX_ERR_BAD_ARGUMENT, "GenerationConfig: temperature must be positive and finite");
    }
    if (c->top_k < 0) return set_error(PSX_ERR_BAD_ARGUMENT, "GenerationConfig: top_k must not be negative");
    if (!(c->top_p > 0.0f && c->top_p <= 1.0f)) return set_error(PSX_ERR_BAD_ARGUMENT, "GenerationConfig: top_p must be in (0, 1]");
    if (!(c->min_p >= 0.0f && c->min_p <= 1.0f)) return set_error(PSX_ERR_BAD_ARGUMENT, "GenerationConfig: min_p must be in [0, 1]");
    if (!(c->repetition_penalty > 0.0f) || c->repetition_penalty > 3.4028235e38f) {
        return set_error(PSX_ERR_BAD_ARGUMENT, "GenerationConfig: repetition_penalty must be positive and finite");
    }
    if (rows < 0) return set_error(PSX_ERR_BAD_ARGUMENT, "psx_b200: rows must not be negative");
    if (vocab <= 0) return set_error(PSX_ERR_BAD_ARGUMENT, "Generate: the model returned no logits");
    if (vocab > (int64_t)psx::kColumnMask) return set_error(PSX_ERR_UNSUPPORTED, "psx_b200: vocabulary exceeds 2^30 - 1 columns");
    if (row_stride < vocab) return set_error(PSX_ERR_BAD_ARGUMENT, "psx_b200: row_stride is smaller than the row");
    if (rows == 0) return PSX_OK;
    if (!logits || !tokens || !log_probs || !row_status) return set_error(PSX_ERR_BAD_ARGUMENT, "psx_b200: null pointer");
    const bool sample = c->do_sample != 0;
    if (sample && !uniforms) return set_error(PSX_ERR_BAD_ARGUMENT, "psx_b200: sampling needs uniforms");
    const bool penalty = c->repetition_penalty != 1.0f;
    if (penalty && (!history_ids || !history_offsets)) {
        return set_error(PSX_ERR_BAD_ARGUMENT, "psx_b200: a repetition penalty needs history_ids and history_offsets");
    }
    const bool ban = c->num_new_tokens < c->min_new_tokens && c->num_eos_token_ids > 0;
    if (c->num_eos_token_ids < 0 || (c->num_eos_token_ids > 0 && !c->eos_token_ids)) {
        return set_error(PSX_ERR_BAD_ARGUMENT, "psx_b200: eos_token_ids is null");
    }

    // ---- once per device: the array's device address, the SM count, the kernels' shared-memory opt-ins --------
    int device = 0;
    PSX_STATIC_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return set_error(PSX_ERR_UNSUPPORTED, "psx_b200: device index too large");
    StaticScratch* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        DeviceSetup& setup = g_setup[device];
        if (!setup.done) {
            void* address = nullptr;
            PSX_STATIC_CUDA(cudaGetSymbolAddress(&address, g_scratch));  // for the device that is current
            // Host-side function attributes, no memory: the limits are lifted to the device's maximum
            // once, and nobody lowers them again.
            PSX_STATIC_CUDA(psx::configure_scan_rows());
            PSX_STATIC_CUDA(psx::configure_merge_rows());
            setup.scratch = static_cast<StaticScratch*>(address);
            setup.done = true;
        }
        scratch = setup.scratch;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);

    // ---- the same plan as psx_b200_sample_rows, within the fixed limits ----------------------------------------
    const psx::Plan plan = psx::make_plan(logits, vocab, row_stride, vocab, c);
    if (rows * plan.parts > kStaticParts) {
        return set_error(PSX_ERR_UNSUPPORTED,
                         "psx_b200_sample_rows_static: the batch needs " + std::to_string(rows * plan.parts) +
                             " parts (rows x ceil(vocab / 16384)); the built-in scratch holds " + std::to_string(kStaticParts) + " -- use psx_b200_sample_rows or a smaller batch");
    }
    if (ban && c->num_eos_token_ids > kStaticBanned) {
        return set_error(PSX_ERR_UNSUPPORTED, "psx_b200_sample_rows_static: at most " + std::to_string(kStaticBanned) +
                                                  " EOS ids can be banned");
    }

    // ---- the same two kernels as psx_b200_sample_rows, pointed at the built-in scratch ----------------------
    psx::ScanParams sp{};
    sp.logits = logits;
    sp.row_stride = row_stride;
    sp.rows = rows;
    sp.cols = vocab;
    sp.col_begin = 0;
    sp.vocab = vocab;
    sp.history_ids = history_ids;
    sp.history_offsets = history_offsets;
    psx::fill_scan_settings(sp, c, plan);
    if (ban) {
        PSX_STATIC_CUDA(cudaMemcpyAsync(scratch->banned, c->eos_token_ids, (size_t)c->num_eos_token_ids * sizeof(int64_t),
                                        cudaMemcpyHostToDevice, stream));
        sp.banned_ids = scratch->banned;
        sp.num_banned = (int32_t)c->num_eos_token_ids;
    }
    sp.stats = scratch->stats;
    sp.part_counts = scratch->part_counts;
    sp.candidates = scratch->candidates;
    if (!plan.lists_cannot_bound) PSX_STATIC_CUDA(psx::launch_scan_rows(sp, plan.nucleus, stream));

    psx::MergeParams mp{};
    psx::fill_merge_params(mp, sp, plan, c, rows, vocab, uniforms, tokens, log_probs, row_status, nullptr, logits, row_stride);
    PSX_STATIC_CUDA(psx::launch_merge_rows(mp, stream));
    return PSX_OK;
}
