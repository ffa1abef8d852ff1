// Host-side construction of TMA tensor maps (driver entry point fetched through the runtime, so
// the library does not link against libcuda).
#pragma once

#include <cuda.h>
#include <cstdint>

#include "df8_internal.cuh"

namespace df8 {

// Tensor map of a row-major [rows, cols] byte matrix (row pitch `pitch_bytes`, a multiple of 16),
// loaded in boxes of [box_rows, box_cols] bytes with a shared-memory swizzle of `swizzle_bytes`
// (0 = none, 32, 64 or 128; box_cols must not exceed it).  Out-of-range parts of a box read as zero.
df8_status make_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                           uint32_t box_rows, uint32_t box_cols, int swizzle_bytes);

}  // namespace df8
