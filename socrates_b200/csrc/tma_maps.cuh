// Tensor maps for TMA, shared by the kernels that use it.
#pragma once

#include <cuda.h>

namespace sb {

// Tensor map of a row-major bfloat16 matrix [rows, cols] with boxes of {64 columns,
// box_rows rows} and 128-byte swizzle.  Maps are pure functions of their arguments and are
// cached (defined in gemm_tcgen05.cu).  False if the driver refuses the map.
bool get_map(CUtensorMap* out, const void* ptr, int rows, int cols, int box_rows);

}  // namespace sb
