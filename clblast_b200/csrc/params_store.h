// Internal view of the tuning-parameter store.
#pragma once

#include <cstddef>

namespace b200 {

// Current GemmRoutine/XGEMM_MIN_INDIRECT_SIZE for (device, precision); 0 unless overridden.
size_t min_indirect_size(int device, int precision);

}  // namespace b200
