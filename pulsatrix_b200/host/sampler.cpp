// DataLoader index samplers (API of include/pulsatrix/sampler.hpp; behaviour of the reference's
// src/sampler.cpp:10-38: a std::mt19937 that persists across epochs, std::iota + std::shuffle).
#include "pulsatrix/sampler.hpp"

#include <algorithm>
#include <numeric>

namespace pulsatrix {

void SequentialSampler::reset(int64_t dataset_size) {
    size_ = dataset_size < 0 ? 0 : dataset_size;
    position_ = 0;
}

std::optional<int64_t> SequentialSampler::next() {
    if (position_ < size_) return position_++;
    return std::nullopt;
}

ShuffleSampler::ShuffleSampler(unsigned seed) : seed_(seed), rng_(seed) {}

void ShuffleSampler::reset(int64_t dataset_size) {
    indices_.assign(static_cast<size_t>(dataset_size < 0 ? 0 : dataset_size), 0);
    std::iota(indices_.begin(), indices_.end(), int64_t{0});
    std::shuffle(indices_.begin(), indices_.end(), rng_);  // the engine is NOT reseeded: every epoch differs
    position_ = 0;
}

std::optional<int64_t> ShuffleSampler::next() {
    if (position_ < indices_.size()) return indices_[position_++];
    return std::nullopt;
}

}  // namespace pulsatrix
