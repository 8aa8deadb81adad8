// Host-side construction (and caching) of TMA tensor maps.  The driver entry point is looked up through the
// runtime (cudaGetDriverEntryPoint), so the library has no link-time dependency on libcuda and still loads on
// a machine without a GPU.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tmaps {

bool available();

// [planes][rows][Dh] bf16 buffer (a state's K or V planes): box = 64 elements x box_rows rows x 1 plane,
// 128-byte swizzle.  Rows past `rows` inside a box read as zeros and never bleed into the next plane.
bool plane_map(CUtensorMap* out, const void* base, int planes, int rows, int Dh, int box_rows = 64);

// [rows][cols] bf16 matrix whose rows are row_stride elements apart (a multiple of 8): box = 64 elements x box_rows
// rows, 128-byte swizzle, addressed with coordinates (column, row, 0).  Rows past `rows` read as zeros.
bool matrix_map(CUtensorMap* out, const void* base, int rows, int cols, long long row_stride, int box_rows);

// [B][L][heads][Dh] bf16 activations with element strides (batch, token): box = 64 elements x 1 head x
// box_rows tokens x 1 batch row, 128-byte swizzle.
bool token_map(CUtensorMap* out, const void* base, int B, int L, int heads, int Dh, long long bs, long long rs,
               int box_rows);

}  // namespace tmaps
