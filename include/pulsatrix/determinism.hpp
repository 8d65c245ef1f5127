/** @file determinism.hpp
 *  Global seed stream of the library, API-compatible with the reference's
 *  include/pulsatrix/determinism.hpp (implementation restated from src/determinism.cpp:24-47).
 *  Host-only: Generate() draws its engine seed from next_seed() when the config carries none.
 */
#pragma once

#include <cstdint>

#include "pulsatrix/export.hpp"

namespace pulsatrix {

/** Sets the global seed and restarts the stream of derived seeds. Call before other threads
 *  construct seeded components. */
PULSATRIX_API void set_seed(uint64_t seed);
PULSATRIX_API uint64_t global_seed();
/** The next seed of the stream: a SplitMix64 finalizer over seed + golden-ratio * (index + 1),
 *  so consecutive seeds give unrelated streams and set_seed() makes the sequence reproducible. */
PULSATRIX_API uint64_t next_seed();
/** Deterministic mode is on by default. */
PULSATRIX_API void set_deterministic(bool enabled);
PULSATRIX_API bool deterministic();
/** Throws std::logic_error naming @p operation while deterministic mode is on. */
PULSATRIX_API void check_deterministic_allowed(const char* operation);

}  // namespace pulsatrix
