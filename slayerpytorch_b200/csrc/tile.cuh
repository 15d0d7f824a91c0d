// 32-row x 32-step fp32 tile owned by one warp, shared by the two spike recurrences.
//
// The recurrences are sequential in time and independent across rows, so inside a tile lane
// l walks row l.  Global memory, however, is only efficient when a warp touches contiguous
// time samples of ONE row.  The tile in shared memory is the transposition point: it is
// filled and drained row by row (lane = time sample, 128 contiguous bytes per access) and
// walked column-wise (lane = row, one 16-byte chunk of four time samples per access).
//
// Layout: row r occupies 32 consecutive words; its eight 16-byte chunks are permuted by
// XOR-ing the chunk index with (r & 7).  This is the 128-byte swizzle pattern of the tensor
// memory unit, so a tile written by a bulk tensor copy and one written by the plain-load
// path look the same.  Both access patterns are bank-conflict free:
//   - row-wise:    fixed r, lane = column: 32 distinct words of one 128-byte row;
//   - column-wise: lane = r, fixed chunk c: each group of eight lanes covers eight distinct
//                  physical chunks = all 32 banks.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace sb200 {

constexpr int kTile = 32;                 // rows per warp = time steps per tile
constexpr int kTileWords = kTile * kTile;

// word offset of (row r, column c)
__device__ __forceinline__ int tile_word(int r, int c)
{
    return r * kTile + ((((c >> 2) ^ (r & 7)) << 2) | (c & 3));
}

// word offset of the 16-byte chunk holding columns 4*chunk .. 4*chunk+3 of row r
__device__ __forceinline__ int tile_chunk(int r, int chunk)
{
    return r * kTile + ((chunk ^ (r & 7)) << 2);
}

// Fill the warp's tile from rows [row0, row0+32) x columns [t0, t0+32) of a [rows, T]
// array; everything outside the array reads as zero.  All 32 loads are issued before the
// first shared-memory store so that they are in flight together.
__device__ __forceinline__ void tile_load(float *tile, const float *g,
                                          int64_t row0, int64_t rows, int t0, int T, int lane)
{
    const int c = t0 + lane;
    const bool col_ok = c < T;
    const int64_t nrow = rows - row0;      // > 0
    const float *p = g + row0 * (int64_t)T + c;
    float v[kTile];
#pragma unroll
    for (int r = 0; r < kTile; ++r)
        v[r] = (col_ok && r < nrow) ? p[(int64_t)r * T] : 0.0f;
#pragma unroll
    for (int r = 0; r < kTile; ++r) tile[tile_word(r, lane)] = v[r];
}

// Drain the warp's tile to the same region of a [rows, T] array.
__device__ __forceinline__ void tile_store(const float *tile, float *g,
                                           int64_t row0, int64_t rows, int t0, int T, int lane)
{
    const int c = t0 + lane;
    if (c >= T) return;
    const int64_t nrow = rows - row0;
    float *p = g + row0 * (int64_t)T + c;
#pragma unroll
    for (int r = 0; r < kTile; ++r)
        if (r < nrow) p[(int64_t)r * T] = tile[tile_word(r, lane)];
}

// Write a 0/value image of per-row bit masks (lane r holds the 32 time bits of row r).
__device__ __forceinline__ void mask_store(unsigned mask, float value, float *g,
                                           int64_t row0, int64_t rows, int t0, int T, int lane)
{
    const int c = t0 + lane;
    const int64_t nrow = rows - row0;
    float *p = g + row0 * (int64_t)T + c;
#pragma unroll
    for (int r = 0; r < kTile; ++r) {
        const unsigned m = __shfl_sync(0xffffffffu, mask, r);
        if (c < T && r < nrow) p[(int64_t)r * T] = ((m >> lane) & 1u) ? value : 0.0f;
    }
}

}  // namespace sb200
