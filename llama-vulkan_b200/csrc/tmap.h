// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled through the runtime's
// driver entry point, so the library does not link libcuda).
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace lv {

// [rows][row_bytes / 8] view of a quantised matrix in 8-byte elements; a box is box_rows rows
// of seg_bytes bytes.  row_bytes and seg_bytes must be multiples of 16.
int make_weight_map(CUtensorMap* out, const void* base, uint32_t rows, uint32_t row_bytes, uint32_t box_rows, uint32_t seg_bytes);

}  // namespace lv
