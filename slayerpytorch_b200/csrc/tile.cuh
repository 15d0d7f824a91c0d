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

// ---------------------------------------------------------------------------------------
// Row-skewed tiles.  A row of T samples starts wherever (row * T) falls; when T is not a
// multiple of 8 most rows start in the middle of a 32-byte sector (and, when T is not a
// multiple of 4, off a 16-byte boundary), and tiles cut at the same time index for every row
// then cost half-used sectors or narrow accesses.  Rows are independent, so each lane may run
// its row a few steps behind the others: row r's tiles start at time 32*j - a_r with
// a_r = (base/4 + row*T) mod 8, which puts every tile on a 32-byte boundary of memory.  Then
// all chunks move as 16-byte vectors whatever T is; only the (at most two) chunks that
// straddle the ends of a row are moved sample by sample.  Columns before the row start are
// filled with `pad` (the recurrences choose a value that keeps their state untouched), columns
// past the row end with zeros, and neither is ever stored.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ int row_skew(int skew0, int r, int T) { return (skew0 + r * (T & 7)) & 7; }

// skew of the first row of a block of 32 rows; phase = (base address / 4) mod 8
__device__ __forceinline__ int block_skew(int64_t row0, int T, unsigned phase)
{
    return (int)((phase + (unsigned)((uint64_t)row0 * (uint64_t)T)) & 7u);
}

__device__ __forceinline__ void tile_prefetch_skew(float *tile, const float *g, int64_t row0, int64_t rows,
                                                   int j, int T, int lane, int skew0, float pad)
{
    const int c = (lane & 7) * 4;
    const int rsub = lane >> 3;
    const int64_t nrow = rows - row0;
#pragma unroll
    for (int i = 0; i < kTile / 4; ++i) {
        const int r = i * 4 + rsub;
        const int t = kTile * j - row_skew(skew0, r, T) + c;      // time of the chunk's first sample
        float *dst = tile + tile_word(r, c);
        const float *src = g + (row0 + r) * (int64_t)T + t;
        if (r >= nrow || t >= T) {
            cp_async<16>(dst, g, false);
        } else if (t >= 0 && t + 4 <= T) {
            cp_async<16>(dst, src, true);
        } else if (t + 4 <= 0) {
            *reinterpret_cast<float4 *>(dst) = make_float4(pad, pad, pad, pad);
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (t + e < 0) dst[e] = pad;
                else cp_async<4>(dst + e, (t + e < T) ? src + e : g, t + e < T);
            }
        }
    }
}

__device__ __forceinline__ void tile_store_skew(const float *tile, float *g, int64_t row0, int64_t rows,
                                                int j, int T, int lane, int skew0)
{
    const int c = (lane & 7) * 4;
    const int rsub = lane >> 3;
    const int64_t nrow = rows - row0;
#pragma unroll
    for (int i = 0; i < kTile / 4; ++i) {
        const int r = i * 4 + rsub;
        const int t = kTile * j - row_skew(skew0, r, T) + c;
        if (r >= nrow || t >= T || t + 4 <= 0) continue;
        const float4 v = *reinterpret_cast<const float4 *>(tile + tile_word(r, c));
        float *dst = g + (row0 + r) * (int64_t)T + t;
        if (t >= 0 && t + 4 <= T) {
            *reinterpret_cast<float4 *>(dst) = v;
        } else {
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (t + k >= 0 && t + k < T) dst[k] = e[k];
        }
    }
}

// Three tiles of the same rows and steps to three arrays of the same shape: the row, its skew,
// the bounds and the offset are worked out once per pass and shared by the three stores.
__device__ __forceinline__ void tile_store3_skew(const float *tile_a, const float *tile_b, const float *tile_c,
                                                 float *ga, float *gb, float *gc, int64_t row0, int64_t rows,
                                                 int j, int T, int lane, int skew0)
{
    const int c = (lane & 7) * 4;
    const int rsub = lane >> 3;
    const int64_t nrow = rows - row0;
#pragma unroll
    for (int i = 0; i < kTile / 4; ++i) {
        const int r = i * 4 + rsub;
        const int t = kTile * j - row_skew(skew0, r, T) + c;
        if (r >= nrow || t >= T || t + 4 <= 0) continue;
        const int w = tile_word(r, c);
        const int64_t off = (row0 + r) * (int64_t)T + t;
        const float4 va = *reinterpret_cast<const float4 *>(tile_a + w);
        const float4 vb = *reinterpret_cast<const float4 *>(tile_b + w);
        const float4 vc = *reinterpret_cast<const float4 *>(tile_c + w);
        if (t >= 0 && t + 4 <= T) {
            *reinterpret_cast<float4 *>(ga + off) = va;
            *reinterpret_cast<float4 *>(gb + off) = vb;
            *reinterpret_cast<float4 *>(gc + off) = vc;
        } else {
            const float ea[4] = {va.x, va.y, va.z, va.w};
            const float eb[4] = {vb.x, vb.y, vb.z, vb.w};
            const float ec[4] = {vc.x, vc.y, vc.z, vc.w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (t + k >= 0 && t + k < T) {
                    ga[off + k] = ea[k];
                    gb[off + k] = eb[k];
                    gc[off + k] = ec[k];
                }
        }
    }
}

// number of 32-step tiles that cover a row of T samples for every skew (0..7)
__host__ __device__ inline int skew_tiles(int T) { return (T + 7 + kTile - 1) / kTile; }

// ---------------------------------------------------------------------------------------
// Wide row-skewed tiles: 64 time steps = two 32-step halves, each laid out like the tile
// above, `half` h at word offset h * kTileWords.  DRAM throughput on this part depends on how
// many contiguous bytes of a row one request covers: 128 bytes per row (a 32-step tile)
// sustain about three quarters of what 256 bytes do.  So the fills and drains below cover a
// whole 256-byte row segment per group of 16 lanes, two rows per instruction; the walk still
// sees two ordinary 32-step tiles.
// ---------------------------------------------------------------------------------------
constexpr int kWide = 2 * kTile;                // time steps per wide tile
constexpr int kWideWords = 2 * kTileWords;

// number of wide tiles that cover a row of T samples for every skew (0..7)
__host__ __device__ inline int skew_wide_tiles(int T) { return (T + 7 + kWide - 1) / kWide; }

template <bool SKEW = true>
__device__ __forceinline__ void wide_prefetch_skew(float *tile, const float *g, int64_t row0, int64_t rows,
                                                   int j, int T, int lane, int skew0, float pad)
{
    const int c16 = lane & 15;                  // 16-byte chunk of the 256-byte row segment
    const int rsub = lane >> 4;
    float *half = tile + (c16 >> 3) * kTileWords;
    const int c = (c16 & 7) * 4;                // column inside the half
    const int64_t nrow = rows - row0;
#pragma unroll
    for (int i = 0; i < kTile / 2; ++i) {
        const int r = i * 2 + rsub;
        const int t = kWide * j - (SKEW ? row_skew(skew0, r, T) : 0) + c16 * 4;      // time of the chunk's first sample
        float *dst = half + tile_word(r, c);
        const float *src = g + (row0 + r) * (int64_t)T + t;
        if (r >= nrow || t >= T) {
            cp_async<16>(dst, g, false);
        } else if (t >= 0 && t + 4 <= T) {
            cp_async<16>(dst, src, true);
        } else if (t + 4 <= 0) {
            *reinterpret_cast<float4 *>(dst) = make_float4(pad, pad, pad, pad);
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (t + e < 0) dst[e] = pad;
                else cp_async<4>(dst + e, (t + e < T) ? src + e : g, t + e < T);
            }
        }
    }
}

// Store four samples starting at time t of a row (clipped to [0, T)).
__device__ __forceinline__ void store_clipped4(float *row, int t, int T, const float4 &v)
{
    if (t >= T || t + 4 <= 0) return;
    if (t >= 0 && t + 4 <= T) {
        *reinterpret_cast<float4 *>(row + t) = v;
    } else {
        const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (t + k >= 0 && t + k < T) row[t + k] = e[k];
    }
}

template <bool SKEW = true>
__device__ __forceinline__ void wide_store_skew(const float *tile, float *g, int64_t row0, int64_t rows,
                                                int j, int T, int lane, int skew0)
{
    const int c16 = lane & 15;
    const int rsub = lane >> 4;
    const float *half = tile + (c16 >> 3) * kTileWords;
    const int c = (c16 & 7) * 4;
    const int64_t nrow = rows - row0;
#pragma unroll
    for (int i = 0; i < kTile / 2; ++i) {
        const int r = i * 2 + rsub;
        if (r >= nrow) continue;
        const int t = kWide * j - (SKEW ? row_skew(skew0, r, T) : 0) + c16 * 4;
        store_clipped4(g + (row0 + r) * (int64_t)T, t, T, *reinterpret_cast<const float4 *>(half + tile_word(r, c)));
    }
}

// Spike samples of a wide tile kept as bit masks: masks[h * 32 + r] bit i = row r spiked at
// step i of half h.  They are expanded to `value` / 0 on their way to global memory.
template <bool SKEW = true>
__device__ __forceinline__ void wide_store_spikes_skew(const unsigned *masks, float *g, int64_t row0, int64_t rows,
                                                       int j, int T, int lane, int skew0, float value)
{
    const int c16 = lane & 15;
    const int rsub = lane >> 4;
    const unsigned *half = masks + (c16 >> 3) * kTile;
    const int sh = (c16 & 7) * 4;
    const int64_t nrow = rows - row0;
#pragma unroll
    for (int i = 0; i < kTile / 2; ++i) {
        const int r = i * 2 + rsub;
        if (r >= nrow) continue;
        const int t = kWide * j - (SKEW ? row_skew(skew0, r, T) : 0) + c16 * 4;
        const unsigned m = half[r] >> sh;
        store_clipped4(g + (row0 + r) * (int64_t)T, t, T,
                       make_float4((m & 1u) ? value : 0.0f, (m & 2u) ? value : 0.0f,
                                   (m & 4u) ? value : 0.0f, (m & 8u) ? value : 0.0f));
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

// true if every array starts on a 16-byte boundary (what the row-skewed tiles need)
inline bool all_aligned16(std::initializer_list<const void *> ptrs)
{
    uintptr_t bits = 0;
    for (const void *p : ptrs) bits |= reinterpret_cast<uintptr_t>(p);
    return (bits & 15u) == 0;
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
