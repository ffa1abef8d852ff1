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

// Tensor map of a row-major [rows, cols] fp32 matrix with a row pitch of `pitch_bytes` (a multiple of 16), moved
// in boxes of [box_rows, box_cols] floats; box_cols * 4 must not exceed swizzle_bytes when a swizzle is used.
df8_status make_tmap_2d_f32(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                            uint32_t box_rows, uint32_t box_cols, int swizzle_bytes);

// Tensor map of a byte matrix [rows, slabs * slab_cols] whose columns are stored as `slabs` separate row-major
// [rows, slab_cols] slabs, `slab_stride_bytes` apart (the layout an all-gather of per-rank column slices leaves):
// coordinates (column inside the slab, row, slab), boxes of [1, box_rows, box_cols] bytes.
df8_status make_tmap_3d_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t slab_cols, uint64_t slabs,
                           uint64_t pitch_bytes, uint64_t slab_stride_bytes, uint32_t box_rows, uint32_t box_cols,
                           int swizzle_bytes);

}  // namespace df8
