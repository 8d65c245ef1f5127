/** @file top_k.hpp
 *  top_k(): selection along a tensor's last dimension, API-compatible with the reference's
 *  include/pulsatrix/top_k.hpp:14-36 (validation of src/top_k.cpp:9-34, order of
 *  src/top_k_math.hpp:19-47), executed by the backend's top_k_rows on the GPU.
 */
#pragma once

#include <cstdint>

#include "pulsatrix/device_backend.hpp"

namespace pulsatrix {

struct TopKResult {
    Tensor values;   ///< (..., k): each row's k best values, best first
    Tensor indices;  ///< (..., k): their positions in the row, as whole-number floats
};

/** The k largest (or smallest) entries of every row along the last dimension, in rank order:
 *  NaN above every number, equal values by ascending index; identical bits on every backend.
 *  @throws std::invalid_argument if input is empty or rank 0, k is outside [1, last dimension],
 *          or the last dimension exceeds 2^24. */
[[nodiscard]] PULSATRIX_API TopKResult top_k(const Tensor& input, int64_t k, bool largest = true);

}  // namespace pulsatrix
