/** @file export.hpp  Symbol visibility of the C++ host layer (the library is built with hidden
 *  visibility; what a caller links against is marked PULSATRIX_API). */
#pragma once

#if defined(__GNUC__)
#define PULSATRIX_API __attribute__((visibility("default")))
#else
#define PULSATRIX_API
#endif
