// 32-row x 32-step fp32 tile owned by one warp, shared by the two spike recurrences.
//
// The recurrences are sequential in time and independent across rows, so inside a tile lane
// l walks row l.  Global memory, however, is only efficient when a warp touches contiguous
// time samples of one row.  The tile in shared memory is the transposition point: it is
// filled and drained along rows (contiguous global segments) and walked column-wise (lane =
// row, one 16-byte chunk of four time samples per access).
//
// Layout: row r occupies 32 consecutive words; its eight 16-byte chunks are permuted by
// XOR-ing the chunk index with (r & 7) - the 128-byte swizzle pattern of the tensor memory
// unit.  Both access patterns are bank-conflict free:
//   - along rows:  lanes cover consecutive words / 8-byte pairs / 16-byte chunks of a row;
//   - column-wise: lane = r, fixed chunk c: each group of eight lanes covers eight distinct
//                  physical chunks = all 32 banks.
//
// Fills are asynchronous (cp.async) so that a warp can prefetch its next tile while it walks
// the current one.  V is the access width in floats (4, 2 or 1), chosen by the host from the
// alignment of the rows: V = 4 needs T % 4 == 0 and 16-byte aligned bases, V = 2 needs
// T % 2 == 0 and 8-byte aligned bases.  Because T % V == 0, a V-wide unit is either wholly
// inside its row or wholly outside, so zero fill and clipped stores stay exact.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <initializer_list>

#include "common.cuh"

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

template <int BYTES>
__device__ __forceinline__ void cp_async(void *smem_dst, const void *gmem_src, bool valid)
{
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int src_bytes = valid ? BYTES : 0;        // 0 source bytes = fill with zeros
    if (BYTES == 16)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(src_bytes) : "memory");
    else if (BYTES == 8)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(src_bytes) : "memory");
    else
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(src_bytes) : "memory");
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }

template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// Start filling the warp's tile from rows [row0, row0+32) x columns [t0, t0+32) of a
// [rows, T] array; everything outside the array is filled with zeros.  The caller commits
// the copy group and waits for it.
template <int V>
__device__ __forceinline__ void tile_prefetch(float *tile, const float *g,
                                              int64_t row0, int64_t rows, int t0, int T, int lane)
{
    constexpr int LPR = kTile / V;            // lanes per row
    constexpr int RPI = 32 / LPR;             // rows per instruction
    const int c = (lane % LPR) * V;           // first column of this lane's unit
    const int rsub = lane / LPR;
    const bool col_ok = t0 + c < T;
    const int64_t nrow = rows - row0;
#pragma unroll
    for (int i = 0; i < kTile / RPI; ++i) {
        const int r = i * RPI + rsub;
        const bool ok = col_ok && r < nrow;
        const float *src = ok ? g + (row0 + r) * (int64_t)T + t0 + c : g;
        cp_async<4 * V>(tile + tile_word(r, c), src, ok);
    }
}

template <int V> struct vec_t;
template <> struct vec_t<4> { typedef float4 type; };
template <> struct vec_t<2> { typedef float2 type; };
template <> struct vec_t<1> { typedef float type; };

// Drain the warp's tile to the same region of a [rows, T] array.
template <int V>
__device__ __forceinline__ void tile_store(const float *tile, float *g,
                                           int64_t row0, int64_t rows, int t0, int T, int lane)
{
    typedef typename vec_t<V>::type vec;
    constexpr int LPR = kTile / V;
    constexpr int RPI = 32 / LPR;
    const int c = (lane % LPR) * V;
    const int rsub = lane / LPR;
    if (t0 + c >= T) return;
    const int64_t nrow = rows - row0;
#pragma unroll
    for (int i = 0; i < kTile / RPI; ++i) {
        const int r = i * RPI + rsub;
        if (r < nrow)
            *reinterpret_cast<vec *>(g + (row0 + r) * (int64_t)T + t0 + c) =
                *reinterpret_cast<const vec *>(tile + tile_word(r, c));
    }
}

__device__ __forceinline__ float bit_value(unsigned m, int bit, float value) { return ((m >> bit) & 1u) ? value : 0.0f; }

// Write a 0/value image of per-row bit masks (lane r holds the 32 time bits of row r).
template <int V>
__device__ __forceinline__ void mask_store(unsigned mask, float value, float *g,
                                           int64_t row0, int64_t rows, int t0, int T, int lane)
{
    constexpr int LPR = kTile / V;
    constexpr int RPI = 32 / LPR;
    const int c = (lane % LPR) * V;
    const int rsub = lane / LPR;
    const int64_t nrow = rows - row0;
    const bool col_ok = t0 + c < T;
#pragma unroll
    for (int i = 0; i < kTile / RPI; ++i) {
        const int r = i * RPI + rsub;
        const unsigned m = __shfl_sync(0xffffffffu, mask, r);
        if (col_ok && r < nrow) {
            float *p = g + (row0 + r) * (int64_t)T + t0 + c;
            if (V == 4)
                *reinterpret_cast<float4 *>(p) = make_float4(bit_value(m, c, value), bit_value(m, c + 1, value),
                                                             bit_value(m, c + 2, value), bit_value(m, c + 3, value));
            else if (V == 2)
                *reinterpret_cast<float2 *>(p) = make_float2(bit_value(m, c, value), bit_value(m, c + 1, value));
            else
                *p = bit_value(m, c, value);
        }
    }
}

// Launch shape of the warp-per-32-rows kernels: warps per CTA and a grid that gives every SM
// the same number of resident warps (as many as shared memory allows, at most 32), each warp
// then strides over the row blocks.  Small problems get smaller CTAs so that all SMs take part.
inline void spike_launch_shape(int64_t nblocks, size_t smem_per_warp, int &warps, int &grid)
{
    const int sms = sm_count();
    // CTA size that packs the most warps into one SM's shared memory (ties: the larger CTA)
    const size_t budget = 216 * 1024;
    int best_total = 0;
    warps = 8;
    for (int w = 8; w >= 3; --w) {
        const size_t per_cta = (size_t)w * smem_per_warp + 2048;       // tiles + barriers/taps/reserve
        int ctas = (int)(budget / per_cta);
        if (ctas * w > 32) ctas = 32 / w;
        if (ctas * w > best_total) { best_total = ctas * w; warps = w; }
    }
    // small problems: smaller CTAs so that every SM takes part
    while (warps > 1 && (nblocks + warps - 1) / warps < 2 * (int64_t)sms) warps >>= 1;
    int64_t ctas_per_sm = (int64_t)(budget / ((size_t)warps * smem_per_warp + 2048));
    if (ctas_per_sm * warps > 32) ctas_per_sm = 32 / warps;
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    int64_t g = (nblocks + warps - 1) / warps;
    if (g > ctas_per_sm * sms) g = ctas_per_sm * sms;
    grid = (int)g;
}

// Access width the host may use for a set of [rows, T] arrays.
inline int tile_vec_width(int64_t T, std::initializer_list<const void *> ptrs)
{
    uintptr_t bits = 0;
    for (const void *p : ptrs) bits |= reinterpret_cast<uintptr_t>(p);
    if (T % 4 == 0 && (bits & 15u) == 0) return 4;
    if (T % 2 == 0 && (bits & 7u) == 0) return 2;
    return 1;
}

}  // namespace sb200
