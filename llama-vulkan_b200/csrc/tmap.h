// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled through the runtime's
// driver entry point, so the library does not link libcuda).
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace lv {

// [rows][row_bytes / 8] view of a quantised matrix in 8-byte elements; a box is box_rows rows
// of seg_bytes bytes.  row_bytes and seg_bytes must be multiples of 16.
int make_weight_map(CUtensorMap* out, const void* base, uint32_t rows, uint32_t row_bytes, uint32_t box_rows, uint32_t seg_bytes);

// Tiled view of `rank` (<= 5) dimensions over 8-byte elements: dims[0] is the contiguous one, strides[i] (bytes, multiples
// of 16) belongs to dims[i + 1]; box[i] <= 256.  No swizzle; out-of-range elements read as zero.
int make_tiled_map(CUtensorMap* out, const void* base, uint32_t rank, const uint64_t* dims, const uint64_t* strides, const uint32_t* box);

}  // namespace lv
