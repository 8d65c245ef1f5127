// Global seed stream (API of include/pulsatrix/determinism.hpp; behaviour of the reference's
// src/determinism.cpp:24-47).
#include "pulsatrix/determinism.hpp"

#include <atomic>
#include <stdexcept>
#include <string>

namespace pulsatrix {
namespace {

std::atomic<uint64_t> seed_value{0};
std::atomic<uint64_t> seeds_drawn{0};
std::atomic<bool> deterministic_mode{true};

// SplitMix64's output function: a bijection on 64 bits that decorrelates neighbouring inputs.
uint64_t scramble(uint64_t z) {
    z ^= z >> 30;
    z *= 0xBF58476D1CE4E5B9ULL;
    z ^= z >> 27;
    z *= 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

}  // namespace

void set_seed(uint64_t seed) {
    seed_value.store(seed);
    seeds_drawn.store(0);
}

uint64_t global_seed() { return seed_value.load(); }

uint64_t next_seed() {
    const uint64_t n = seeds_drawn.fetch_add(1) + 1;
    return scramble(seed_value.load() + n * 0x9E3779B97F4A7C15ULL);
}

void set_deterministic(bool enabled) { deterministic_mode.store(enabled); }

bool deterministic() { return deterministic_mode.load(); }

void check_deterministic_allowed(const char* operation) {
    if (!deterministic()) return;
    throw std::logic_error(std::string(operation) + " is nondeterministic; call set_deterministic(false) to allow it");
}

}  // namespace pulsatrix
