// The boundary against the reference's REAL classes -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// This file contains no reference code.  It is compiled together with the reference's own
// src/cuda_backend.cu (nvcc, in place, objects only under oracle/_ref/) and defines
//     class B200Backend : public pulsatrix::CUDABackend      (the reference's class, from its header)
// whose top_k_rows forwards to psx_b200_top_k_rows of libpsx_b200.so -- the binding a maintainer
// would add to src/cuda_backend.cu:851-860 -- so that the reference's own top_k()
// (src/top_k.cpp:9-34) and its TopKRowsMatchCPUBitExactly case
// (tests/backend_primitive_equivalence_cases.hpp:345-375) run through the new kernel, and the
// reference's unmodified kernel (src/gpu_kernels.cuh:1256-1262) can be timed beside it on the same
// GPU.  libpsx_b200.so is opened with dlopen(RTLD_LOCAL): it carries its own restatement of the
// pulsatrix:: classes, which must not meet the reference's in one symbol table.
#include <dlfcn.h>

#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

#include "pulsatrix/cpu_backend.hpp"
#include "pulsatrix/cuda_backend.hpp"
#include "pulsatrix/top_k.hpp"

namespace {

struct psx_ctx;
using ctx_create_fn = int (*)(int, psx_ctx**);
using ctx_destroy_fn = void (*)(psx_ctx*);
using ctx_stream_fn = void* (*)(psx_ctx*);
using sync_fn = int (*)(psx_ctx*, void*);
using last_error_fn = const char* (*)();
using top_k_rows_fn = int (*)(psx_ctx*, void*, const float*, float*, float*, size_t, size_t, size_t, int);

class B200Backend : public pulsatrix::CUDABackend {
public:
    explicit B200Backend(const char* library) {
        handle_ = dlopen(library, RTLD_NOW | RTLD_LOCAL);
        if (!handle_) throw std::runtime_error(std::string("dlopen: ") + dlerror());
        create_ = reinterpret_cast<ctx_create_fn>(dlsym(handle_, "psx_b200_ctx_create"));
        destroy_ = reinterpret_cast<ctx_destroy_fn>(dlsym(handle_, "psx_b200_ctx_destroy"));
        stream_of_ = reinterpret_cast<ctx_stream_fn>(dlsym(handle_, "psx_b200_ctx_stream"));
        sync_ = reinterpret_cast<sync_fn>(dlsym(handle_, "psx_b200_sync"));
        last_error_ = reinterpret_cast<last_error_fn>(dlsym(handle_, "psx_b200_last_error"));
        top_k_rows_ = reinterpret_cast<top_k_rows_fn>(dlsym(handle_, "psx_b200_top_k_rows"));
        if (!create_ || !destroy_ || !stream_of_ || !sync_ || !last_error_ || !top_k_rows_) {
            throw std::runtime_error("libpsx_b200.so lacks an entry point");
        }
        if (create_(0, &psx_) != 0) throw std::runtime_error(last_error_());
    }
    ~B200Backend() override {
        if (psx_) destroy_(psx_);
    }
    // The one override: what replaces src/cuda_backend.cu:851-860.
    void top_k_rows(const float* in, float* values, float* indices, size_t rows, size_t cols, size_t k,
                    bool largest) override {
        if (rows == 0) return;
        void* stream = stream_of_(psx_);
        const int s = top_k_rows_(psx_, stream, in, values, indices, rows, cols, k, largest ? 1 : 0);
        if (s == 1) throw std::invalid_argument(last_error_());
        if (s != 0) throw std::runtime_error(last_error_());
        if (sync_(psx_, stream) != 0) throw std::runtime_error(last_error_());  // every backend op synchronises
    }

private:
    void* handle_ = nullptr;
    psx_ctx* psx_ = nullptr;
    ctx_create_fn create_ = nullptr;
    ctx_destroy_fn destroy_ = nullptr;
    ctx_stream_fn stream_of_ = nullptr;
    sync_fn sync_ = nullptr;
    last_error_fn last_error_ = nullptr;
    top_k_rows_fn top_k_rows_ = nullptr;
};

void Say(char* message, int length, const std::string& text) {
    if (message && length > 0) std::snprintf(message, static_cast<size_t>(length), "%s", text.c_str());
}

bool SameFloat(float a, float b) { return a == b || (std::isnan(a) && std::isnan(b)); }

struct DeviceArray {
    pulsatrix::DeviceBackend& backend;
    float* ptr;
    size_t count;
    DeviceArray(pulsatrix::DeviceBackend& b, const std::vector<float>& host)
        : backend(b), ptr(static_cast<float*>(b.allocate(host.size() * sizeof(float)))), count(host.size()) {
        backend.copy(ptr, host.data(), host.size() * sizeof(float), pulsatrix::CopyDirection::HostToDevice);
    }
    ~DeviceArray() { backend.free(ptr); }
    std::vector<float> host() const {
        std::vector<float> out(count);
        backend.copy(out.data(), ptr, count * sizeof(float), pulsatrix::CopyDirection::DeviceToHost);
        return out;
    }
};

}  // namespace

extern "C" {

// The inputs and the checks of the reference's TopKRowsMatchCPUBitExactly
// (tests/backend_primitive_equivalence_cases.hpp:345-375), through B200Backend.  0 when everything
// matched the reference's CPUBackend bit for bit; otherwise 1 and what differed in `message`.
int psxrefcuda_top_k_rows_match_cpu(const char* library, char* message, int length) {
    try {
        B200Backend gpu(library);
        pulsatrix::CPUBackend cpu;
        const size_t rows = 300, cols = 129;
        std::vector<float> in(rows * cols);
        std::mt19937 rng(41);
        for (auto& x : in) x = static_cast<float>(static_cast<int>(rng() % 9) - 4) * 0.5f;
        in[3] = std::nanf("");
        in[cols + 7] = INFINITY;
        in[2 * cols + 1] = -INFINITY;
        DeviceArray din(gpu, in);
        for (bool largest : {true, false}) {
            for (size_t k : {size_t{1}, size_t{7}, cols}) {
                std::vector<float> cpu_values(rows * k), cpu_indices(rows * k);
                cpu.top_k_rows(in.data(), cpu_values.data(), cpu_indices.data(), rows, cols, k, largest);
                DeviceArray dvalues(gpu, std::vector<float>(rows * k, 0.0f)), dindices(gpu, std::vector<float>(rows * k, 0.0f));
                gpu.top_k_rows(din.ptr, dvalues.ptr, dindices.ptr, rows, cols, k, largest);
                const std::vector<float> gpu_values = dvalues.host(), gpu_indices = dindices.host();
                for (size_t i = 0; i < cpu_values.size(); ++i) {
                    if (cpu_indices[i] != gpu_indices[i] || !SameFloat(cpu_values[i], gpu_values[i])) {
                        Say(message, length, "largest=" + std::to_string(largest) + " k=" + std::to_string(k) +
                                                 " flat index " + std::to_string(i));
                        return 1;
                    }
                }
            }
        }
        return 0;
    } catch (const std::exception& e) {
        Say(message, length, e.what());
        return 2;
    }
}

// The reference's own top_k() (src/top_k.cpp:9-34) on a (rows, cols) tensor that lives on
// B200Backend (library given) or on the reference's unmodified CUDABackend (library null).
// 0 ok; 1 std::invalid_argument; 2 anything else (text in `message`).
int psxrefcuda_top_k(const char* library, const float* in, int64_t rows, int64_t cols, int64_t k, int largest,
                     float* values, float* indices, char* message, int length) {
    try {
        std::unique_ptr<pulsatrix::CUDABackend> gpu;
        if (library) gpu.reset(new B200Backend(library)); else gpu.reset(new pulsatrix::CUDABackend());
        const std::vector<float> data(in, in + rows * cols);
        pulsatrix::Tensor x(pulsatrix::Shape({rows, cols}), gpu.get(), data);
        const pulsatrix::TopKResult r = pulsatrix::top_k(x, k, largest != 0);
        const std::vector<float> v = r.values.to_host_vector(), i = r.indices.to_host_vector();
        std::memcpy(values, v.data(), v.size() * sizeof(float));
        std::memcpy(indices, i.data(), i.size() * sizeof(float));
        return 0;
    } catch (const std::invalid_argument& e) {
        Say(message, length, e.what());
        return 1;
    } catch (const std::exception& e) {
        Say(message, length, e.what());
        return 2;
    }
}

// Microseconds per DeviceBackend::top_k_rows call (each call synchronises, as every op of the
// reference's backend does) on seeded normal data: the reference's own kernel (library null) or the
// override.  Negative on failure.
double psxrefcuda_time_top_k_rows(const char* library, int64_t rows, int64_t cols, int64_t k, int repeats) {
    try {
        std::unique_ptr<pulsatrix::CUDABackend> gpu;
        if (library) gpu.reset(new B200Backend(library)); else gpu.reset(new pulsatrix::CUDABackend());
        std::vector<float> in(static_cast<size_t>(rows * cols));
        std::mt19937 rng(7);
        std::normal_distribution<float> normal(0.0f, 1.0f);
        for (auto& x : in) x = normal(rng);
        DeviceArray din(*gpu, in);
        DeviceArray dvalues(*gpu, std::vector<float>(static_cast<size_t>(rows * k), 0.0f));
        DeviceArray dindices(*gpu, std::vector<float>(static_cast<size_t>(rows * k), 0.0f));
        gpu->top_k_rows(din.ptr, dvalues.ptr, dindices.ptr, rows, cols, k, true);  // warm-up
        const auto begin = std::chrono::steady_clock::now();
        for (int r = 0; r < repeats; ++r) gpu->top_k_rows(din.ptr, dvalues.ptr, dindices.ptr, rows, cols, k, true);
        const auto end = std::chrono::steady_clock::now();
        return std::chrono::duration<double, std::micro>(end - begin).count() / repeats;
    } catch (const std::exception&) {
        return -1.0;
    }
}

}  // extern "C"
