// The reference's own tests for this path, restated against the C++ host API of this library
// (tests/generation_test.cpp:66-245, tests/top_k_test.cpp:49-144, tests/sampler_test.cpp:20-77,
// tests/determinism_test.cpp:41-53 of the reference).  No test framework is available offline,
// so a few macros stand in.  `host_api_test --host-only` runs what needs no GPU.
#include <cuda_runtime.h>

#include <algorithm>
#include <memory>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <limits>
#include <map>
#include <numeric>
#include <set>
#include <stdexcept>
#include <string>
#include <vector>

#include "pulsatrix/determinism.hpp"
#include "pulsatrix/generation.hpp"
#include "pulsatrix/sampler.hpp"
#include "pulsatrix/top_k.hpp"

using namespace pulsatrix;

static int g_failures = 0, g_checks = 0;
#define CHECK(cond)                                                                 \
    do {                                                                            \
        ++g_checks;                                                                 \
        if (!(cond)) {                                                              \
            ++g_failures;                                                           \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);           \
        }                                                                           \
    } while (0)
#define CHECK_THROWS(expr, type)                                                    \
    do {                                                                            \
        ++g_checks;                                                                 \
        bool caught = false;                                                        \
        try { (void)(expr); } catch (const type&) { caught = true; } catch (...) {} \
        if (!caught) {                                                              \
            ++g_failures;                                                           \
            std::printf("FAILED %s:%d: %s did not throw %s\n", __FILE__, __LINE__, #expr, #type); \
        }                                                                           \
    } while (0)

constexpr float kInf = std::numeric_limits<float>::infinity();
constexpr float kNaN = std::numeric_limits<float>::quiet_NaN();

// ---- host-only: seed stream and index samplers ------------------------------------------------------

static void test_seed_stream() {
    set_seed(5);
    const uint64_t a = next_seed(), b = next_seed();
    CHECK(a != b);
    set_seed(5);
    CHECK(next_seed() == a && next_seed() == b);
    set_seed(6);
    CHECK(next_seed() != a);
    CHECK(global_seed() == 6);
    CHECK(deterministic());
    CHECK_THROWS(check_deterministic_allowed("atomic add"), std::logic_error);
    set_deterministic(false);
    check_deterministic_allowed("atomic add");
    set_deterministic(true);
}

static void test_samplers() {
    SequentialSampler seq;
    seq.reset(4);
    for (int64_t i = 0; i < 4; ++i) CHECK(seq.next() == i);
    CHECK(!seq.next().has_value());
    seq.reset(0);
    CHECK(!seq.next().has_value());

    ShuffleSampler a(123), b(123), c(124);
    auto epoch = [](ShuffleSampler& s, int64_t n) {
        std::vector<int64_t> order;
        s.reset(n);
        while (auto i = s.next()) order.push_back(*i);
        return order;
    };
    const auto a1 = epoch(a, 50), b1 = epoch(b, 50), c1 = epoch(c, 50);
    CHECK(a1 == b1);                                  // same seed, same order
    CHECK(a1 != c1);                                  // another seed, another order
    std::vector<int64_t> sorted = a1;
    std::sort(sorted.begin(), sorted.end());
    std::vector<int64_t> all(50);
    std::iota(all.begin(), all.end(), 0);
    CHECK(sorted == all);                             // a permutation
    const auto a2 = epoch(a, 50);
    CHECK(a2 != a1);                                  // a new epoch is a new permutation
    CHECK(epoch(b, 50) == a2);                        // ... the same one for the same seed
    // The engine is std::mt19937 and the shuffle std::shuffle, as in the reference.
    std::mt19937 rng(123);
    std::vector<int64_t> expect(50);
    std::iota(expect.begin(), expect.end(), 0);
    std::shuffle(expect.begin(), expect.end(), rng);
    CHECK(a1 == expect);
}

// ---- generation ------------------------------------------------------------------------------------

static const std::vector<float> kLogits{1.25f, -0.5f, 2.0f, 0.75f, -1.5f, 0.25f, 3.0f, -0.25f, 1.5f, 0.5f, -1.0f, 2.5f};
static const std::vector<int64_t> kTokens{3, 5, 5, 9};

static void expect_logits(const std::vector<float>& actual, const std::vector<float>& expected) {
    CHECK(actual.size() == expected.size());
    for (size_t i = 0; i < expected.size() && i < actual.size(); ++i) {
        if (std::isinf(expected[i])) CHECK(actual[i] == expected[i]);
        else CHECK(std::fabs(actual[i] - expected[i]) <= 1e-5f);
    }
}

static std::vector<float> processed(const GenerationConfig& c, int64_t num_new = 0) {
    std::vector<float> l = kLogits;
    ProcessLogits(l, kTokens, num_new, c);
    return l;
}

// The Hugging Face vectors of the reference's GenerationTest.LogitProcessingMatchesHuggingFace.
static void test_logit_processing_matches_hugging_face() {
    GenerationConfig c;
    c.repetition_penalty = 1.3f;
    expect_logits(processed(c), {1.25f, -0.5f, 2.0f, 0.576923072f, -1.5f, 0.192307696f, 3.0f, -0.25f, 1.5f, 0.384615391f, -1.0f, 2.5f});
    c = {};
    c.do_sample = true;
    c.temperature = 0.7f;
    c.top_k = 4;
    expect_logits(processed(c), {-kInf, -kInf, 2.85714293f, -kInf, -kInf, -kInf, 4.28571415f, -kInf, 2.14285707f, -kInf, -kInf, 3.57142854f});
    c = {};
    c.do_sample = true;
    c.top_p = 0.8f;
    expect_logits(processed(c), {-kInf, -kInf, 2.0f, -kInf, -kInf, -kInf, 3.0f, -kInf, 1.5f, -kInf, -kInf, 2.5f});
    c = {};
    c.do_sample = true;
    c.min_p = 0.1f;
    expect_logits(processed(c), {1.25f, -kInf, 2.0f, 0.75f, -kInf, -kInf, 3.0f, -kInf, 1.5f, -kInf, -kInf, 2.5f});
    c = {};
    c.min_new_tokens = 2;
    c.eos_token_ids = {6};
    expect_logits(processed(c, 1), {1.25f, -0.5f, 2.0f, 0.75f, -1.5f, 0.25f, -kInf, -0.25f, 1.5f, 0.5f, -1.0f, 2.5f});
    expect_logits(processed(c, 2), kLogits);
    c = {};
    c.do_sample = true;
    c.repetition_penalty = 1.2f;
    c.temperature = 0.8f;
    c.top_k = 6;
    c.top_p = 0.9f;
    c.min_p = 0.05f;
    expect_logits(processed(c), {-kInf, -kInf, 2.5f, -kInf, -kInf, -kInf, 3.75f, -kInf, 1.875f, -kInf, -kInf, 3.125f});
    c.do_sample = false;  // greedy ignores the sampling settings
    c.repetition_penalty = 1.0f;
    expect_logits(processed(c), kLogits);
}

// A bigram model: the next token is (last + 1) mod 5 with high probability.
static std::vector<float> bigram(const std::vector<int64_t>& tokens) {
    std::vector<float> l(5, 0.0f);
    l[static_cast<size_t>((tokens.back() + 1) % 5)] = 4.0f;
    return l;
}

static void test_greedy_follows_the_model_and_stops_at_eos() {
    GenerationConfig c;
    c.max_new_tokens = 10;
    c.eos_token_ids = {4};
    GenerationResult r = Generate(NextTokenLogitsFn(bigram), {1}, c);
    CHECK((r.new_tokens == std::vector<int64_t>{2, 3, 4}));
    CHECK((r.tokens == std::vector<int64_t>{1, 2, 3, 4}));
    CHECK(r.finish_reason == FinishReason::Eos);
    CHECK(r.log_probs.size() == 3u);
    CHECK(std::fabs(r.log_probs[0] - (4.0f - std::log(std::exp(4.0f) + 4.0f))) <= 1e-6f);
    c.eos_token_ids = {};
    c.max_new_tokens = 7;
    r = Generate(NextTokenLogitsFn(bigram), {1}, c);
    CHECK(r.new_tokens.size() == 7u);
    CHECK(r.finish_reason == FinishReason::Length);
    CHECK(r.new_tokens.back() == 3);  // 2 3 4 0 1 2 3
}

static void test_min_new_tokens_holds_off_eos() {
    GenerationConfig c;
    c.max_new_tokens = 10;
    c.eos_token_ids = {2};
    CHECK((Generate(NextTokenLogitsFn(bigram), {1}, c).new_tokens == std::vector<int64_t>{2}));
    c.min_new_tokens = 3;
    const GenerationResult r = Generate(NextTokenLogitsFn(bigram), {1}, c);
    CHECK(r.new_tokens.size() >= 4u);
    CHECK(r.new_tokens[0] != 2);
    CHECK(r.new_tokens[0] == 0);  // EOS banned: everything else ties, the lowest index wins
    CHECK(r.finish_reason == FinishReason::Eos);
}

static void test_sampling_is_seeded_and_follows_the_distribution(int draws) {
    const std::vector<float> fixed{0.0f, 1.0f, 2.0f, -1.0f};
    NextTokenLogitsFn model = [&](const std::vector<int64_t>&) { return fixed; };
    GenerationConfig c;
    c.do_sample = true;
    c.temperature = 0.5f;  // p ~ exp(2 * logit)
    c.max_new_tokens = draws;
    c.seed = 17;
    GenerationResult r = Generate(model, {0}, c);
    std::map<int64_t, int> counts;
    for (int64_t t : r.new_tokens) ++counts[t];
    double z = 0.0;
    for (float l : fixed) z += std::exp(2.0 * l);
    for (int64_t t = 0; t < 4; ++t) {
        const double p = std::exp(2.0 * fixed[static_cast<size_t>(t)]) / z;
        CHECK(std::fabs(counts[t] / static_cast<double>(draws) - p) <= 0.015);
    }
    c.max_new_tokens = 50;
    CHECK(Generate(model, {0}, c).new_tokens == Generate(model, {0}, c).new_tokens);
    GenerationConfig other = c;
    other.seed = 18;
    CHECK(Generate(model, {0}, c).new_tokens != Generate(model, {0}, other).new_tokens);
    c.seed.reset();  // without a seed, set_seed() makes it reproducible
    set_seed(5);
    const auto first = Generate(model, {0}, c).new_tokens;
    set_seed(5);
    CHECK(Generate(model, {0}, c).new_tokens == first);
    c.top_k = 1;  // top_k = 1 makes sampling greedy
    for (int64_t t : Generate(model, {0}, c).new_tokens) CHECK(t == 2);
}

static void test_rejects_bad_input() {
    NextTokenLogitsFn model = bigram;
    GenerationConfig c;
    CHECK_THROWS(Generate(model, {}, c), std::invalid_argument);
    c.temperature = 0.0f;
    CHECK_THROWS(Generate(model, {1}, c), std::invalid_argument);
    c = {};
    c.top_p = 0.0f;
    CHECK_THROWS(Generate(model, {1}, c), std::invalid_argument);
    c = {};
    c.top_k = -1;
    CHECK_THROWS(Generate(model, {1}, c), std::invalid_argument);
    c = {};
    c.max_new_tokens = -1;
    CHECK_THROWS(Generate(model, {1}, c), std::invalid_argument);
    NextTokenLogitsFn nan_model = [](const std::vector<int64_t>&) { return std::vector<float>{0.0f, std::nanf("")}; };
    CHECK_THROWS(Generate(nan_model, {1}, GenerationConfig{}), std::invalid_argument);
    NextTokenLogitsFn empty_model = [](const std::vector<int64_t>&) { return std::vector<float>{}; };
    CHECK_THROWS(Generate(empty_model, {1}, GenerationConfig{}), std::invalid_argument);
    GenerationConfig banned;  // EOS is the whole vocabulary and min_new_tokens holds it off
    banned.min_new_tokens = 1;
    banned.eos_token_ids = {0, 1, 2, 3, 4};
    CHECK_THROWS(Generate(model, {1}, banned), std::invalid_argument);
    std::vector<float> l = kLogits;
    GenerationConfig bad;
    bad.min_p = 2.0f;
    CHECK_THROWS(ProcessLogits(l, kTokens, 0, bad), std::invalid_argument);
}

// The device-logits overload gives the same text as the host one.
static void test_device_logits_overload_matches(CUDABackend& gpu) {
    const int64_t vocab = 5000;
    std::vector<float> table(static_cast<size_t>(vocab));
    uint32_t s = 7;
    for (auto& x : table) { s = s * 1664525u + 1013904223u; x = static_cast<float>((s >> 8) % 2000) * 0.005f - 5.0f; }
    Tensor device_row(Shape({vocab}), &gpu, table);
    NextTokenLogitsFn host_model = [&](const std::vector<int64_t>& t) {
        std::vector<float> row = table;
        row[static_cast<size_t>(t.back() % vocab)] += 3.0f;  // depends on the sequence
        return row;
    };
    Tensor scratch(Shape({vocab}), &gpu);
    DeviceNextTokenLogitsFn device_model = [&](const std::vector<int64_t>& t) {
        const std::vector<float> row = host_model(t);
        gpu.copy(scratch.data(), row.data(), row.size() * sizeof(float), CopyDirection::HostToDevice);
        return DeviceLogits{scratch.data(), vocab};
    };
    GenerationConfig c;
    c.do_sample = true;
    c.temperature = 0.9f;
    c.top_k = 40;
    c.top_p = 0.95f;
    c.repetition_penalty = 1.3f;
    c.max_new_tokens = 64;
    c.seed = 3;
    const GenerationResult a = Generate(host_model, {1, 2, 3}, c), b = Generate(device_model, {1, 2, 3}, c);
    CHECK(a.new_tokens == b.new_tokens);
    CHECK(a.log_probs == b.log_probs);
}

// A model that produces its logits asynchronously on a stream of its own and does not wait for them:
// Generate() must order its kernels after that stream's work (DeviceLogits::stream).
static void test_device_logits_from_another_stream(CUDABackend& gpu) {
    const int64_t vocab = 200000;  // a copy long enough to still be in flight when the model returns
    float* pinned = nullptr;
    CHECK(cudaMallocHost(&pinned, static_cast<size_t>(vocab) * sizeof(float)) == cudaSuccess);
    cudaStream_t producer = nullptr;
    CHECK(cudaStreamCreateWithFlags(&producer, cudaStreamNonBlocking) == cudaSuccess);
    Tensor row(Shape({vocab}), &gpu, std::vector<float>(static_cast<size_t>(vocab), -50.0f));  // stale contents
    auto fill = [&](const std::vector<int64_t>& t) {
        for (int64_t i = 0; i < vocab; ++i) pinned[i] = static_cast<float>((i * 7919 + t.back() * 104729) % 1000) * 0.01f;
    };
    NextTokenLogitsFn host_model = [&](const std::vector<int64_t>& t) {
        fill(t);
        return std::vector<float>(pinned, pinned + vocab);
    };
    DeviceNextTokenLogitsFn device_model = [&](const std::vector<int64_t>& t) {
        cudaStreamSynchronize(producer);  // (the pinned buffer is free again)
        fill(t);
        cudaMemcpyAsync(row.data(), pinned, static_cast<size_t>(vocab) * sizeof(float), cudaMemcpyHostToDevice, producer);
        return DeviceLogits{row.data(), vocab, producer};  // not waited for
    };
    GenerationConfig c;
    c.max_new_tokens = 12;
    c.repetition_penalty = 1.5f;
    const GenerationResult a = Generate(host_model, {5, 6}, c), b = Generate(device_model, {5, 6}, c);
    CHECK(a.new_tokens == b.new_tokens);
    CHECK(a.log_probs == b.log_probs);
    cudaStreamSynchronize(producer);
    cudaStreamDestroy(producer);
    cudaFreeHost(pinned);
}

// The head on the device: Generate(MakeDeviceLmHeadLogits(body, head)) gives the tokens and log-probs
// of a host model whose head is the reference's loop (one float accumulator per logit, ascending
// feature order, product and sum each rounded: src/cpu_backend.cpp:188-196).
static void test_device_lm_head(bool tied) {
    const int64_t vocab = 3001, d = 97;
    std::vector<float> weight(static_cast<size_t>(vocab * d));
    uint32_t s = tied ? 11u : 23u;
    for (auto& x : weight) { s = s * 1664525u + 1013904223u; x = static_cast<float>(static_cast<int>((s >> 9) % 2001) - 1000) * 0.001f; }
    HiddenStateFn body = [&](const std::vector<int64_t>& t) {
        std::vector<float> h(static_cast<size_t>(d));
        uint32_t r = static_cast<uint32_t>(t.back() * 2654435761u + t.size() * 40503u);
        for (auto& x : h) { r = r * 1664525u + 1013904223u; x = static_cast<float>(static_cast<int>((r >> 10) % 4001) - 2000) * 0.002f; }
        return h;
    };
    NextTokenLogitsFn host_model = [&](const std::vector<int64_t>& t) {
        const std::vector<float> h = body(t);
        std::vector<float> logits(static_cast<size_t>(vocab));
        for (int64_t j = 0; j < vocab; ++j) {
            volatile float acc = 0.0f;  // (volatile: every product and every sum is rounded to float, never fused)
            for (int64_t p = 0; p < d; ++p) {
                const float w = tied ? weight[static_cast<size_t>(j * d + p)] : weight[static_cast<size_t>(p * vocab + j)];
                volatile float product = h[static_cast<size_t>(p)] * w;
                acc = acc + product;
            }
            logits[static_cast<size_t>(j)] = acc;
        }
        return logits;
    };
    auto head = std::make_shared<DeviceLmHead>(weight, vocab, d, tied);
    const DeviceNextTokenLogitsFn device_model = MakeDeviceLmHeadLogits(body, head);
    GenerationConfig greedy;
    greedy.max_new_tokens = 24;
    greedy.repetition_penalty = 1.2f;
    GenerationConfig sampled = greedy;
    sampled.do_sample = true;
    sampled.temperature = 0.7f;
    sampled.top_k = 30;
    sampled.top_p = 0.9f;
    sampled.seed = 9;
    for (const GenerationConfig& c : {greedy, sampled}) {
        const GenerationResult a = Generate(host_model, {3, 1, 4}, c), b = Generate(device_model, {3, 1, 4}, c);
        CHECK(a.new_tokens == b.new_tokens);
        CHECK(a.log_probs == b.log_probs);
    }
    CHECK_THROWS(DeviceLmHead(weight, vocab, d + 1, tied), std::invalid_argument);
    CHECK_THROWS((void)head->logits(std::vector<float>(5)), std::invalid_argument);
}

// ---- top-k -------------------------------------------------------------------------------------------

static std::vector<float> tie_heavy_values(size_t n, uint32_t seed) {  // coarse values: ties are common
    std::vector<float> v(n);
    for (auto& x : v) {
        seed = seed * 1664525u + 1013904223u;
        x = static_cast<float>(static_cast<int>((seed >> 16) % 9) - 4) * 0.5f;
    }
    return v;
}

static std::vector<int64_t> reference_order(const std::vector<float>& row, bool largest) {
    auto greater = [](float a, float b) { return (std::isnan(a) && !std::isnan(b)) || a > b; };
    std::vector<int64_t> order(row.size());
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int64_t i, int64_t j) {
        return largest ? greater(row[static_cast<size_t>(i)], row[static_cast<size_t>(j)])
                       : greater(row[static_cast<size_t>(j)], row[static_cast<size_t>(i)]);
    });
    return order;
}

static void test_top_k(CUDABackend& gpu) {
    {
        Tensor x(Shape({8}), &gpu, {3, 1, 4, 1, 5, 9, 2, 6});
        TopKResult r = top_k(x, 3);
        CHECK(r.values.shape() == Shape({3}));
        CHECK((r.values.to_host_vector() == std::vector<float>{9, 6, 5}));
        CHECK((r.indices.to_host_vector() == std::vector<float>{5, 7, 4}));
        r = top_k(x, 3, /*largest=*/false);
        CHECK((r.values.to_host_vector() == std::vector<float>{1, 1, 2}));
        CHECK((r.indices.to_host_vector() == std::vector<float>{1, 3, 6}));
        CHECK(r.values.device() == x.device());
    }
    {
        Tensor x(Shape({5}), &gpu, {2, 7, 2, 7, 2});
        TopKResult r = top_k(x, 4);
        CHECK((r.values.to_host_vector() == std::vector<float>{7, 7, 2, 2}));
        CHECK((r.indices.to_host_vector() == std::vector<float>{1, 3, 0, 2}));
    }
    {
        Tensor x(Shape({5}), &gpu, {1.0f, kNaN, kInf, -kInf, kNaN});
        TopKResult largest = top_k(x, 3);
        CHECK((largest.indices.to_host_vector() == std::vector<float>{1, 4, 2}));
        const auto v = largest.values.to_host_vector();
        CHECK(std::isnan(v[0]) && std::isnan(v[1]) && v[2] == kInf);
        TopKResult smallest = top_k(x, 3, false);
        CHECK((smallest.values.to_host_vector() == std::vector<float>{-kInf, 1.0f, kInf}));
        CHECK((smallest.indices.to_host_vector() == std::vector<float>{3, 0, 2}));
    }
    {
        Tensor x(Shape({2, 3, 5}), &gpu, tie_heavy_values(30, 3));
        TopKResult r = top_k(x, 2);
        CHECK(r.values.shape() == Shape({2, 3, 2}) && r.indices.shape() == Shape({2, 3, 2}));
    }
    {
        constexpr int64_t rows = 37, cols = 53;
        std::vector<float> v = tie_heavy_values(rows * cols, 11);
        v[5] = kNaN;
        v[cols + 9] = -kInf;
        Tensor x(Shape({rows, cols}), &gpu, v);
        for (bool largest : {true, false}) {
            for (int64_t k : {int64_t{1}, int64_t{4}, int64_t{17}, cols}) {
                TopKResult r = top_k(x, k, largest);
                const auto idx = r.indices.to_host_vector(), val = r.values.to_host_vector();
                for (int64_t row = 0; row < rows; ++row) {
                    const std::vector<float> rv(v.begin() + row * cols, v.begin() + (row + 1) * cols);
                    const auto order = reference_order(rv, largest);
                    for (int64_t j = 0; j < k; ++j) {
                        CHECK(idx[static_cast<size_t>(row * k + j)] == static_cast<float>(order[static_cast<size_t>(j)]));
                        const float e = rv[static_cast<size_t>(order[static_cast<size_t>(j)])], a = val[static_cast<size_t>(row * k + j)];
                        CHECK(a == e || (std::isnan(a) && std::isnan(e)));
                    }
                }
            }
        }
    }
    {
        Tensor x(Shape({2, 4}), &gpu, {1, 2, 3, 4, 5, 6, 7, 8});
        CHECK_THROWS(top_k(x, 0), std::invalid_argument);
        CHECK_THROWS(top_k(x, -1), std::invalid_argument);
        CHECK_THROWS(top_k(x, 5), std::invalid_argument);
        Tensor empty(Shape({0}), &gpu);
        CHECK_THROWS(top_k(empty, 1), std::invalid_argument);
    }
}

// `--print-streams`: the seed stream and a shuffle order, for comparison with the reference's.
static int print_streams() {
    set_seed(5);
    std::printf("seeds");
    for (int i = 0; i < 5; ++i) std::printf(" %llu", static_cast<unsigned long long>(next_seed()));
    std::printf("\nshuffle");
    ShuffleSampler s(41);
    for (int epoch = 0; epoch < 2; ++epoch) {
        s.reset(12);
        while (auto i = s.next()) std::printf(" %lld", static_cast<long long>(*i));
    }
    std::printf("\n");
    return 0;
}

int main(int argc, char** argv) {
    if (argc > 1 && std::strcmp(argv[1], "--print-streams") == 0) return print_streams();
    const bool host_only = argc > 1 && std::strcmp(argv[1], "--host-only") == 0;
    const int draws = argc > 2 ? std::atoi(argv[2]) : 40000;
    test_seed_stream();
    test_samplers();
    if (!host_only) {
        try {
            CUDABackend gpu(0);
            test_logit_processing_matches_hugging_face();
            test_greedy_follows_the_model_and_stops_at_eos();
            test_min_new_tokens_holds_off_eos();
            test_sampling_is_seeded_and_follows_the_distribution(draws);
            test_rejects_bad_input();
            test_device_logits_overload_matches(gpu);
            test_device_logits_from_another_stream(gpu);
            test_device_lm_head(true);
            test_device_lm_head(false);
            test_top_k(gpu);
        } catch (const std::exception& e) {
            ++g_failures;
            std::printf("FAILED: unexpected exception: %s\n", e.what());
        }
    }
    std::printf("%s: %d checks, %d failures\n", host_only ? "host-only" : "all", g_checks, g_failures);
    return g_failures == 0 ? 0 : 1;
}
