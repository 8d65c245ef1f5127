/** @file sampler.hpp
 *  The DataLoader's index samplers, API-compatible with the reference's
 *  include/pulsatrix/sampler.hpp:20-67 (behaviour of src/sampler.cpp:10-38).  Host-only; not part of
 *  the GPU sampling path -- kept because callers of the generation API also link against it.
 */
#pragma once

#include <cstdint>
#include <optional>
#include <random>
#include <vector>

#include "pulsatrix/export.hpp"

namespace pulsatrix {

/** Order in which one epoch visits the indices [0, dataset_size). reset() starts an epoch,
 *  next() yields one index per call and std::nullopt once all have been produced. */
class PULSATRIX_API Sampler {
public:
    virtual ~Sampler() = default;
    virtual void reset(int64_t dataset_size) = 0;
    [[nodiscard]] virtual std::optional<int64_t> next() = 0;
};

/** 0, 1, 2, ... */
class PULSATRIX_API SequentialSampler : public Sampler {
public:
    void reset(int64_t dataset_size) override;
    [[nodiscard]] std::optional<int64_t> next() override;

private:
    int64_t size_ = 0;
    int64_t position_ = 0;
};

/** A fresh std::shuffle permutation per epoch from one std::mt19937 seeded at construction, so
 *  a seed fixes the whole sequence of epochs and no two epochs repeat the same order. */
class PULSATRIX_API ShuffleSampler : public Sampler {
public:
    explicit ShuffleSampler(unsigned seed);
    void reset(int64_t dataset_size) override;
    [[nodiscard]] std::optional<int64_t> next() override;

private:
    unsigned seed_;
    std::mt19937 rng_;
    std::vector<int64_t> indices_;
    size_t position_ = 0;
};

}  // namespace pulsatrix
