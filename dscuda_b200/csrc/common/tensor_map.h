// Host-side construction of TMA tensor maps for 2-D bf16 views with 128-byte
// swizzle.  The driver entry point is looked up at run time, so the library
// does not link against libcuda.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace dscuda {

// View of `rows` x `cols` bf16 elements whose rows are `row_stride_elements`
// apart; the box is `box_rows` x 64 elements (128 bytes wide), swizzled.
// Out-of-range elements are read as zero.  Throws on bad alignment.
CUtensorMap make_bf16_tile_map(const void* base, std::uint64_t rows, std::uint64_t cols, std::uint64_t row_stride_elements,
                               std::uint32_t box_rows);

// The same rows seen as [chunk][row][64 elements]: `chunks` consecutive 64-column chunks of a row are
// 128 bytes apart, rows `row_stride_elements` apart.  One load of a box {64, box_rows, box_chunks} at
// coordinates {0, row, chunk} lands in shared memory chunk after chunk, each a [box_rows x 128 byte]
// swizzled tile, i.e. what `box_chunks` loads through the 2-D view would have produced.
CUtensorMap make_bf16_chunked_map(const void* base, std::uint64_t rows, std::uint32_t chunks, std::uint64_t row_stride_elements,
                                  std::uint32_t box_rows, std::uint32_t box_chunks);

// A plain (unswizzled) view of `rows` rows of `row_words` 64-bit words each, rows contiguous.  One load of
// a box {box_words, box_rows} at {word, row} lands in shared memory row after row, box_words * 8 bytes each.
CUtensorMap make_u64_rows_map(const void* base, std::uint64_t rows, std::uint32_t row_words, std::uint32_t box_words, std::uint32_t box_rows);

}  // namespace dscuda
