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
//     that device current); make that first call before starting any stream capture on that device;
//   * every call uses the same array.  Nothing in it has to start at zero: the row pass rewrites
//     every record and every list count of the batch before the survivor stage reads them, and
//     list slots beyond a count are never used, so stale contents of an earlier call are
//     harmless.  But two calls that overlap on the GPU (different streams, or different host
//     threads) race on it: keep calls stream-ordered one after another per device.
#include <mutex>
#include <string>

#include "../../include/psx_b200.h"
#include "merge_rows.cuh"
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

constexpr int kSortCapacity = 1024, kGatherCapacity = 4096;          // as the regular top-k / greedy plan
constexpr int kSortCapacityWide = 4096, kGatherCapacityWide = 8192;  // sampling without a top-k

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

    // ---- the fixed limits ------------------------------------------------------------------------------
    const bool aligned = (reinterpret_cast<uintptr_t>(logits) % 16 == 0) && (row_stride % 4 == 0);
    const int64_t vectors = (vocab + 3 + (aligned ? 0 : 3)) / 4;
    const int64_t parts = (vectors + psx::kPartVecs - 1) / psx::kPartVecs;
    if (rows * parts > kStaticParts) {
        return set_error(PSX_ERR_UNSUPPORTED,
                         "psx_b200_sample_rows_static: the batch needs " + std::to_string(rows * parts) +
                             " parts (rows x ceil(vocab / 16384)); the built-in scratch holds " +
                             std::to_string(kStaticParts) + " -- use psx_b200_sample_rows or a smaller batch");
    }
    if (ban && c->num_eos_token_ids > kStaticBanned) {
        return set_error(PSX_ERR_UNSUPPORTED, "psx_b200_sample_rows_static: at most " + std::to_string(kStaticBanned) +
                                                  " EOS ids can be banned");
    }

    // ---- once per device: the array's device address, the kernels' shared-memory opt-ins -------------------
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
            setup.scratch = static_cast<StaticScratch*>(address);
            setup.done = true;
        }
        scratch = setup.scratch;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    // Shared-memory opt-ins of the two kernels (host-side function attributes, no memory): set on
    // every call, because the regular entry points adjust the same attributes to their own needs.
    PSX_STATIC_CUDA(psx::configure_scan_rows());
    PSX_STATIC_CUDA(psx::configure_merge_rows());

    // ---- the same two kernels as psx_b200_sample_rows, pointed at the built-in scratch ----------------------
    const bool top_k_on = sample && c->top_k > 0 && c->top_k < vocab;
    const bool apply_temperature = sample && c->temperature != 1.0f;
    const bool nucleus = sample && !top_k_on;
    psx::ScanParams sp{};
    sp.logits = logits;
    sp.row_stride = row_stride;
    sp.rows = rows;
    sp.cols = vocab;
    sp.col_begin = 0;
    sp.vocab = vocab;
    sp.history_ids = history_ids;
    sp.history_offsets = history_offsets;
    sp.apply_penalty = penalty ? 1 : 0;
    sp.penalty = c->repetition_penalty;
    sp.apply_temperature = apply_temperature ? 1 : 0;
    sp.temperature = c->temperature;
    const double log2e = 1.4426950408889634073599246810019;
    sp.log2e_over_t = (float)(apply_temperature ? log2e / (double)c->temperature : log2e);
    sp.k_need = !sample ? 1 : top_k_on ? (int)(c->top_k < (1 << 20) ? c->top_k : (1 << 20)) : 160;
    if (vectors * 4 <= psx::kPartCap) sp.k_need = 1 << 30;  // small rows are handed on whole
    sp.parts = (int)parts;
    sp.vecs_per_part = (int)((vectors + parts - 1) / parts);
    sp.debug_skip = 0;
    sp.num_banned = 0;
    sp.banned_ids = nullptr;
    if (ban) {
        PSX_STATIC_CUDA(cudaMemcpyAsync(scratch->banned, c->eos_token_ids, (size_t)c->num_eos_token_ids * sizeof(int64_t),
                                        cudaMemcpyHostToDevice, stream));
        sp.banned_ids = scratch->banned;
        sp.num_banned = (int32_t)c->num_eos_token_ids;
    }
    sp.stats = scratch->stats;
    sp.part_counts = scratch->part_counts;
    sp.candidates = scratch->candidates;
    PSX_STATIC_CUDA(psx::launch_scan_rows(sp, nucleus, stream));

    psx::MergeParams mp{};
    mp.stats = sp.stats;
    mp.part_counts = sp.part_counts;
    mp.candidates = sp.candidates;
    mp.parts = sp.parts;
    mp.part_cap = psx::kPartCap;
    mp.slot_shift = psx::merge_slot_shift(sp.parts, psx::kPartCap,
                                          sp.k_need >= psx::kPartCap ? psx::kPartCap : sp.k_need + sp.k_need / 4 + 24);
    mp.stats_part_stride = sizeof(psx::PartStats);
    mp.stats_row_stride = mp.stats_part_stride * sp.parts;
    mp.count_part_stride = sizeof(uint32_t);
    mp.count_row_stride = mp.count_part_stride * sp.parts;
    mp.cand_part_stride = sizeof(uint2) * psx::kPartCap;
    mp.cand_row_stride = mp.cand_part_stride * sp.parts;
    mp.rows = rows;
    mp.vocab = vocab;
    mp.do_sample = sample ? 1 : 0;
    mp.apply_temperature = apply_temperature ? 1 : 0;
    mp.temperature = c->temperature;
    mp.penalty = c->repetition_penalty;
    mp.top_k = c->top_k;
    mp.top_p = c->top_p;
    mp.min_p = c->min_p;
    mp.uniforms = uniforms;
    mp.tokens = tokens;
    mp.log_probs = log_probs;
    mp.row_status = row_status;
    mp.diag = nullptr;
    mp.sort_capacity = nucleus ? kSortCapacityWide : kSortCapacity;
    mp.gather_capacity = nucleus ? kGatherCapacityWide : kGatherCapacity;
    PSX_STATIC_CUDA(psx::launch_merge_rows(mp, stream));
    return PSX_OK;
}
