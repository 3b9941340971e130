// TMA tensor maps over row-major bfloat16 matrices, shared by the kernels that load through them.
#pragma once
#include <cuda.h>

namespace kb {

// A [rows, cols] bfloat16 matrix whose rows are `pitch_elems` elements apart, seen in boxes of
// box_rows x 64 elements (128 bytes) under the 128-byte swizzle; elements outside the matrix read
// as zero. Returns 0, or 1 after storing a message.
int encode_map_bf16(CUtensorMap* map, const void* base, unsigned long long rows, unsigned long long cols,
                    unsigned long long pitch_elems, unsigned box_rows);

// A dense [rows, cols] bfloat16 matrix (cols a multiple of 64) seen as three dimensions: 64 elements,
// rows, chunks of 64 columns. A box of box_rows rows lands in shared memory chunk by chunk:
// [cols / 64][box_rows][128 bytes] under the 128-byte swizzle, one copy for rows of any width.
// Coordinates are (0, row, 0).
// `box_chunks` (0: all of them) chunks a box; the third coordinate is then the first chunk wanted.
int encode_map_bf16_chunks(CUtensorMap* map, const void* base, unsigned long long rows, unsigned cols, unsigned box_rows,
                           unsigned box_chunks = 0);

}  // namespace kb
