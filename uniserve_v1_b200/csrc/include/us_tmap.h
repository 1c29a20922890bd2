// Host-side construction of TMA tensor maps.  The driver entry point is looked
// up at run time (cudaGetDriverEntryPoint), so the library links against the
// CUDA runtime only.
#pragma once
#include <cuda.h>
#include <stdint.h>

enum UsTmapDtype : int { US_TMAP_BF16 = 0, US_TMAP_F16 = 1, US_TMAP_U8 = 2, US_TMAP_F32 = 3 };
enum UsTmapSwizzle : int { US_SWZ_NONE = 0, US_SWZ_32 = 1, US_SWZ_64 = 2, US_SWZ_128 = 3 };

// dims/box are innermost first; strides_bytes has rank-1 entries (the innermost
// stride is the element size).  Returns 0 on success.
int us_tmap_encode(CUtensorMap* out, const void* base, int dtype, int rank, const uint64_t* dims,
                   const uint64_t* strides_bytes, const uint32_t* box, int swizzle);

// Row-major 2-D matrix [rows, cols] with `ld` elements between rows; box is
// [box_rows, box_cols].
int us_tmap_2d(CUtensorMap* out, const void* base, int dtype, uint64_t rows, uint64_t cols,
               uint64_t ld, uint32_t box_rows, uint32_t box_cols, int swizzle);

// Batched row-major matrices [batch, rows, cols] (contiguous), box [1, box_rows, box_cols].
int us_tmap_3d(CUtensorMap* out, const void* base, int dtype, uint64_t batch, uint64_t rows,
               uint64_t cols, uint64_t ld, uint64_t batch_stride, uint32_t box_rows,
               uint32_t box_cols, int swizzle);
