// Temporal FIR filter along the last axis and its adjoint:
//   conv: out[r,t] = Ts * sum_{i<K, t-i>=0} in[r,t-i] * f[i]      (psp, forward)
//   corr: out[r,t] = Ts * sum_{i<K, t+i<T}  in[r,t+i] * f[i]      (psp, backward)
// Each output is one fp32 fused-multiply-add chain over the taps in ascending order starting
// from +0, scaled by Ts once at the end - the same sequence of roundings as a thread-per-
// output loop, so results are reproducible bit for bit whatever the tiling.  Samples outside
// the row enter the chain as +0, which leaves the accumulator unchanged for finite taps.
//
// Three kernels compute the same bits.  fir_kernel, described next, is the scalar form;
// fir_flow_kernel (further down, the default) is the same arithmetic without a CTA-wide barrier
// per tile.  fir2_kernel packs two rows per lane into two-wide FMAs, skips the zeros of spike
// tensors and can read bit-packed spike tensors; slayer_b200_set_fir_packed(1) selects it for
// conv / corr, and slayer_b200_conv_packed always runs it.
//
// Cost: 8 algorithmic bytes and 2K flops per element.  For K above ~47 taps the fp32 FMA
// pipes, not HBM, bound the kernel, so the design goal is to keep those pipes fed:
//   - persistent CTAs walk [32 rows x nseg*16 samples] tiles; the input tile (plus a halo of
//     K-1 samples) is staged in shared memory with cp.async, double buffered, so the copy of
//     the next tile overlaps the arithmetic of the current one;
//   - lane l of every warp owns row l, a warp owns 16-sample segments of the tile, and a
//     thread keeps 16 accumulators plus a 20-sample sliding input window in registers;
//   - per group of 4 taps a thread issues 64 FMAs, one 128-bit load of new window samples and
//     one 128-bit broadcast load of taps (shared-memory bandwidth is the second scarcest
//     resource, which is why a thread produces 16 outputs and not fewer);
//   - the window rotates through a ring of six register quads by unrolling, and the loads for
//     the next group target the quad that is not in use, so no moves are spent on it;
//   - results go from registers straight to global memory (64 contiguous bytes per thread).
// The row stride of the tile is = 4 (mod 8) words, which makes the per-row 128-bit loads of a
// warp conflict free.
#include <atomic>
#include <type_traits>
#include <cfloat>

#include "common.cuh"
#include "fir_sparse.cuh"
#include "tile.cuh"
#include "tma.cuh"

namespace sb200 {

constexpr int kFirRows = 32;        // rows per tile (= lanes)
constexpr int kFirSeg = 16;         // outputs per thread per segment
constexpr int kFirWin = kFirSeg + 4;           // samples one group of four taps reads
constexpr int kFirRing = kFirWin + 4;          // register ring: the window plus the quad being loaded
constexpr int kFirPhases = kFirRing / 4;       // 6
constexpr int kFirMaxWarps = 16;
constexpr int kFirStageWords = 16;      // packed input: words of one row that a tile (at most 432 samples) can touch
constexpr int kFirTileWordsPerRow = 432;  // 2 buffers x 32 rows x 432 words = 108 KB: two CTAs per SM

// 128-bit load from a 32-bit shared-memory address (explicit state space: the address
// arithmetic stays 32-bit and constant offsets fold into the instruction)
__device__ __forceinline__ float4 ld4(unsigned saddr)
{
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(saddr));
    return v;
}

// acc = a * b + acc, one fused multiply-add that accumulates in place (denormals flushed, as
// in the rest of this translation unit)
__device__ __forceinline__ void fma_acc(float &acc, float a, float b)
{
    asm("fma.rn.ftz.f32 %0, %1, %2, %0;" : "+f"(acc) : "f"(a), "f"(b));
}

// The sliding input window lives in a ring of six register quads: five hold the 20 samples
// the current group of four taps reads, the sixth receives the quad the NEXT group needs, so
// that load never targets registers that are still being read and costs no register moves.
// After each group the window moves by four samples; the mapping from logical window position
// q to ring register rotates with the phase PH = group mod 6 instead of the data moving:
//   conv (window moves toward older samples):  ring = (q - 4*PH) mod 24
//   corr (window moves toward newer samples):  ring = (q + 4*PH) mod 24
// The incoming quad is logical position -4 (conv) or 20 (corr) of the current phase.
template <int DIR, int PH>
__device__ __forceinline__ constexpr int win_reg(int q)
{
    return DIR < 0 ? (q + 4 * kFirRing - 4 * PH) % kFirRing : (q + 4 * PH) % kFirRing;
}

__device__ __forceinline__ void put4(float (&w)[kFirRing], int base, const float4 &v)
{
    w[base] = v.x; w[base + 1] = v.y; w[base + 2] = v.z; w[base + 3] = v.w;
}

// acc[m] += sum_{ii<NT} W[m + off(ii)] * f[ii], ascending ii, W = logical window of phase PH.
// conv: sample for (m, ii) is W[m + 4 - ii];  corr: W[m + ii].
template <int DIR, int PH, int NT>
__device__ __forceinline__ void fir_group(float (&acc)[kFirSeg], const float (&w)[kFirRing], const float4 &f)
{
    const float fv[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
    for (int ii = 0; ii < NT; ++ii) {
#pragma unroll
        for (int m = 0; m < kFirSeg; ++m)
            fma_acc(acc[m], w[win_reg<DIR, PH>(DIR < 0 ? m + 4 - ii : m + ii)], fv[ii]);
    }
}

template <int DIR, int PH>
__device__ __forceinline__ void fir_group_n(float (&acc)[kFirSeg], const float (&w)[kFirRing], const float4 &f, int ntaps)
{
    switch (ntaps) {
        case 1: fir_group<DIR, PH, 1>(acc, w, f); break;
        case 2: fir_group<DIR, PH, 2>(acc, w, f); break;
        case 3: fir_group<DIR, PH, 3>(acc, w, f); break;
        default: fir_group<DIR, PH, 4>(acc, w, f); break;
    }
}

// One group in phase PH.  Before its arithmetic it starts the loads the group after it needs:
// the sample quad that enters the window (into the free ring quad) and the next four taps
// (into the tap quad the previous group has finished with).
// fp / xp are the addresses phase 0 of the current run of phases uses (taps of its group, sample
// quad it fetches); phase PH reads at constant offsets from them, which go into the load
// instructions as immediates.
template <int OFF>
__device__ __forceinline__ float4 ld4o(unsigned saddr)
{
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4+%5];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(saddr), "n"(OFF));
    return v;
}

template <int DIR, int PH>
__device__ __forceinline__ void fir_step(float (&acc)[kFirSeg], float (&w)[kFirRing], float4 (&f)[2],
                                         unsigned fp, unsigned xp)
{
    put4(w, win_reg<DIR, PH>(DIR < 0 ? -4 + kFirRing : kFirWin), ld4o<(DIR < 0 ? -16 : 16) * PH>(xp));
    f[(PH + 1) & 1] = ld4o<16 * (PH + 1)>(fp);
    fir_group<DIR, PH, 4>(acc, w, f[PH & 1]);
}

// The last `left` (< 6) full groups and the partial group of `tail` taps, phases from PH on.
// f[PH & 1] already holds the taps of the first remaining group.
template <int DIR, int PH>
__device__ __forceinline__ void fir_rest(float (&acc)[kFirSeg], float (&w)[kFirRing], float4 (&f)[2],
                                         unsigned fp, unsigned xp, int left, int tail)
{
    if (left == 0) {
        if (tail) fir_group_n<DIR, PH>(acc, w, f[PH & 1], tail);
        return;
    }
    fir_step<DIR, PH>(acc, w, f, fp, xp);
    if constexpr (PH + 1 < kFirPhases) fir_rest<DIR, PH + 1>(acc, w, f, fp, xp, left - 1, tail);
}

// The partial group of `tail` taps when the groups end in front of phase PH.
template <int DIR, int PH>
__device__ __forceinline__ void fir_tail(float (&acc)[kFirSeg], float (&w)[kFirRing], float4 (&f)[2], int tail)
{
    if (tail) fir_group_n<DIR, PH>(acc, w, f[PH & 1], tail);
}

struct FirShape {
    int nseg;       // 16-sample segments per tile
    int halo;       // extra input samples staged per row (multiple of 4, >= K-1 plus slack)
    int SX;         // row stride of the input tile in words
    int ttiles;     // tiles along time
    int nwarps;     // warps per CTA
};

// DIR = -1: conv, DIR = +1: corr.  V: global access width in floats (4, 2 or 1; T % V == 0
// and bases aligned to 4*V bytes).
template <int DIR, int V>
__global__ void __launch_bounds__(kFirMaxWarps * 32)
fir_kernel(float *__restrict__ out, const float *__restrict__ in, const float *__restrict__ filt,
           int64_t rows, int T, int K, float Ts, FirShape sh, int64_t ntiles, const int *skip_flag)
{
    if (skip_flag != nullptr && *skip_flag != 0) return;      // the event-driven kernel has this call
    extern __shared__ __align__(16) float smem[];
    const int Tt = sh.nseg * kFirSeg;
    const int WX = Tt + sh.halo;
    const int KP = ((K + 3) & ~3) + 4;       // taps, zero padded; one spare quad for the look-ahead load
    float *fs = smem;
    float *xbuf = fs + KP;                   // 2 x [kFirRows x SX]
    const int tile_words = kFirRows * sh.SX;

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;

    for (int i = threadIdx.x; i < KP; i += blockDim.x) fs[i] = i < K ? filt[i] : 0.0f;

    // asynchronous copy of one input tile: warp w fills rows w, w+nwarps, ... from contiguous
    // global segments; samples outside the row (or rows outside the array) become zeros.
    // With 16-byte accesses a lane copies at most four chunks per row, and which of them lie
    // inside [0, T) is the same for every row of the tile, so that is worked out once per tile
    // and a row costs one pointer plus, per chunk, one 64-bit add and the copy itself.
    const unsigned xbuf_saddr = (unsigned)__cvta_generic_to_shared(xbuf);
    auto fill = [&](int buf, int64_t tile) {
        float *xs = xbuf + buf * tile_words;
        const int64_t rb = tile / sh.ttiles;
        const int t0 = (int)(tile - rb * sh.ttiles) * Tt;
        const int64_t row0 = rb * kFirRows;
        const int64_t nrow = rows - row0;
        const int g0 = DIR < 0 ? t0 - sh.halo : t0;      // global time of tile position 0
        if constexpr (V == 4) {
            constexpr int kChunks = (kFirTileWordsPerRow + 127) / 128;     // 4
            int goff[kChunks], nbytes[kChunks];          // source offset in the row; 16, 0 (zero fill) or -1 (no chunk)
#pragma unroll
            for (int k = 0; k < kChunks; ++k) {
                const int pcol = lane * 4 + 128 * k;
                const int gt = g0 + pcol;
                const bool ok = gt >= 0 && gt < T;
                goff[k] = ok ? gt : 0;
                nbytes[k] = pcol < WX ? (ok ? 16 : 0) : -1;
            }
            for (int r = warp; r < kFirRows; r += nwarps) {
                const bool row_ok = r < nrow;
                const float *src = in + (row0 + (row_ok ? r : 0)) * (int64_t)T;
                const unsigned dst = xbuf_saddr + 4u * (unsigned)(buf * tile_words + r * sh.SX + lane * 4);
#pragma unroll
                for (int k = 0; k < kChunks; ++k) {
                    if (nbytes[k] < 0) continue;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n"
                                 ::"r"(dst + 512u * k), "l"(src + goff[k]), "r"(row_ok ? nbytes[k] : 0) : "memory");
                }
            }
        } else {
            for (int r = warp; r < kFirRows; r += nwarps) {
                const bool row_ok = r < nrow;
                const float *src = in + (row0 + (row_ok ? r : 0)) * (int64_t)T;
                float *dst = xs + r * sh.SX;
                for (int pcol = lane * V; pcol < WX; pcol += 32 * V) {
                    const int gt = g0 + pcol;
                    const bool ok = row_ok && gt >= 0 && gt < T;
                    cp_async<4 * V>(dst + pcol, ok ? src + gt : in, ok);
                }
            }
        }
        cp_async_commit();
    };

    const int groups = K >> 2;          // full groups of 4 taps
    const int tail = K & 3;
    constexpr unsigned step = DIR < 0 ? 0u - 16u : 16u;   // bytes the window moves per group (mod 2^32)
    const unsigned fs_addr = (unsigned)__cvta_generic_to_shared(fs);
    const unsigned xbuf_addr = (unsigned)__cvta_generic_to_shared(xbuf);

    int64_t tile = blockIdx.x;
    if (tile < ntiles) fill(0, tile);
    for (int it = 0; tile < ntiles; tile += gridDim.x, ++it) {
        cp_async_wait<0>();
        __syncthreads();                 // this tile has landed; the other buffer is free again
        const int64_t next = tile + gridDim.x;
        if (next < ntiles) fill((it + 1) & 1, next);

        const int64_t rb = tile / sh.ttiles;
        const int t0 = (int)(tile - rb * sh.ttiles) * Tt;
        const int64_t row = rb * kFirRows + lane;
        // byte address of tile position 0 of this lane's row
        const unsigned xrow = xbuf_addr + 4u * (unsigned)((it & 1) * tile_words + lane * sh.SX + (DIR < 0 ? sh.halo : 0));

        for (int seg = warp; seg < sh.nseg; seg += nwarps) {
            const int tb = seg * kFirSeg;
            if (t0 + tb >= T) break;    // whole segment beyond the row end (warp-uniform)
            float acc[kFirSeg];
#pragma unroll
            for (int m = 0; m < kFirSeg; ++m) acc[m] = 0.0f;

            // initial window (phase 0): conv x[tb-4 .. tb+16), corr x[tb .. tb+20)
            float w[kFirRing];
            const unsigned x0 = xrow + 4u * (unsigned)tb - (DIR < 0 ? 16u : 0u);
#pragma unroll
            for (int q = 0; q < kFirWin / 4; ++q) put4(w, 4 * q, ld4(x0 + 16 * q));
            unsigned xp = DIR < 0 ? x0 - 16 : x0 + 4 * kFirWin;    // next sample quad to fetch
            unsigned fp = fs_addr;
            float4 f[2];
            f[0] = ld4(fp);
            int g = 0;
            for (; g + kFirPhases <= groups; g += kFirPhases) {
                fir_step<DIR, 0>(acc, w, f, fp, xp);
                fir_step<DIR, 1>(acc, w, f, fp, xp);
                fir_step<DIR, 2>(acc, w, f, fp, xp);
                fir_step<DIR, 3>(acc, w, f, fp, xp);
                fir_step<DIR, 4>(acc, w, f, fp, xp);
                fir_step<DIR, 5>(acc, w, f, fp, xp);
                xp += kFirPhases * step;
                fp += 16 * kFirPhases;
            }
            fir_rest<DIR, 0>(acc, w, f, fp, xp, groups - g, tail);

            if (row < rows) {
                float *dst = out + row * (int64_t)T + t0 + tb;
                const int left = T - (t0 + tb);          // > 0, multiple of V
                if (V == 4) {
#pragma unroll
                    for (int q = 0; q < kFirSeg / 4; ++q)
                        if (4 * q < left)
                            *reinterpret_cast<float4 *>(dst + 4 * q) = make_float4(
                                acc[4 * q] * Ts, acc[4 * q + 1] * Ts, acc[4 * q + 2] * Ts, acc[4 * q + 3] * Ts);
                } else if (V == 2) {
#pragma unroll
                    for (int q = 0; q < kFirSeg / 2; ++q)
                        if (2 * q < left)
                            *reinterpret_cast<float2 *>(dst + 2 * q) = make_float2(acc[2 * q] * Ts, acc[2 * q + 1] * Ts);
                } else {
#pragma unroll
                    for (int q = 0; q < kFirSeg; ++q)
                        if (q < left) dst[q] = acc[q] * Ts;
                }
            }
        }
    }
    cp_async_wait<0>();
}


typedef unsigned long long f2;      // two packed fp32 values

// ---------------------------------------------------------------------------------------
// Packed variant: two rows per lane, two fp32 FMAs per instruction.
//
// fma.rn.ftz.f32x2 performs two independent single-precision fused multiply-adds on the halves
// of 64-bit registers; each half rounds exactly like the scalar instruction, so results keep
// their bits.  The FMA pipe does the same number of lane-operations per clock either way, but
// the packed form needs half the issue slots, which leaves room for the shared-memory loads and
// the address arithmetic that otherwise compete with the FMAs for issue.  Every operand has to
// be a register pair, and a pair that has to be put together from two registers costs moves
// that eat the gain, so the data is arranged to make the pairs natural:
//   - a lane owns TWO rows (2l and 2l+1 of a 64-row tile); the tile the arithmetic reads
//     interleaves the two rows sample by sample (A0 B0 A1 B1 ...), so one 128-bit load yields
//     two ready (A_t, B_t) pairs and the sliding window is a ring of pairs;
//   - taps sit in shared memory duplicated (f0 f0 f1 f1 ...), one 128-bit broadcast load
//     yields two (f, f) pairs;
//   - accumulators are pairs (outA[m], outB[m]).
// Global memory cannot be copied into the interleaved form efficiently (it would take 4-byte
// copies), so a tile takes two steps: 16-byte cp.async copies land the next tile in a staging
// buffer with plain rows while the current tile is being computed, and a short pass of all
// warps re-packs staging -> interleaved (two 128-bit loads, two 128-bit stores per 8 samples)
// between two barriers.  The same pass notes which sample positions hold a non-zero in any of
// the 64 rows (see the zero-skipping segment below).  A bit-packed input is staged as words
// and expanded by the re-pack pass.
// One CTA per SM (staging + interleaved tile of up to 64 rows x 428 samples), warps take
// 16-sample segments.
// ---------------------------------------------------------------------------------------
constexpr int kFir2Rows = 64;
constexpr int kFir2MaxSamples = 428;     // staged samples per row: staging + tile of 64 rows x 428 words fit one SM
constexpr int kFir2HalfSamples = 212;    // ... and of 64 rows x 212 words fit twice
constexpr int kFir2MaskWords = 20;       // one bit per staged sample position (14 words for 428 samples) plus the
                                         // words a segment's 128-bit window may read past them
constexpr int kFir2StageWords = 16;      // packed input: staged words per row (covers 428 samples at any bit offset)
constexpr int kFir2ScanEvery = 8;        // dense mode: look at every 8th tile for zeros
constexpr int kFir2SparsePercent = 45;   // a tile runs the zero-skipping path below this share of live positions

// 64-bit load of one (row A, row B) sample pair
__device__ __forceinline__ f2 ld1p(unsigned saddr)
{
    f2 v;
    asm volatile("ld.shared.b64 %0, [%1];" : "=l"(v) : "r"(saddr));
    return v;
}

__device__ __forceinline__ void st4(unsigned saddr, float a, float b, float c, float d)
{
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ void ld2p(unsigned saddr, f2 &a, f2 &b)
{
    asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "r"(saddr));
}

__device__ __forceinline__ void fma2_acc(f2 &acc, f2 a, f2 b)
{
    asm("fma.rn.ftz.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}

__device__ __forceinline__ void unpack2(f2 v, float &lo, float &hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

template <int DIR, int PH, int NT>
__device__ __forceinline__ void fir2_group(f2 (&acc)[kFirSeg], const f2 (&w)[kFirRing], const f2 (&f)[4])
{
#pragma unroll
    for (int ii = 0; ii < NT; ++ii) {
#pragma unroll
        for (int m = 0; m < kFirSeg; ++m)
            fma2_acc(acc[m], w[win_reg<DIR, PH>(DIR < 0 ? m + 4 - ii : m + ii)], f[ii]);
    }
}

template <int DIR, int PH>
__device__ __forceinline__ void fir2_group_n(f2 (&acc)[kFirSeg], const f2 (&w)[kFirRing], const f2 (&f)[4], int ntaps)
{
    switch (ntaps) {
        case 1: fir2_group<DIR, PH, 1>(acc, w, f); break;
        case 2: fir2_group<DIR, PH, 2>(acc, w, f); break;
        case 3: fir2_group<DIR, PH, 3>(acc, w, f); break;
        default: fir2_group<DIR, PH, 4>(acc, w, f); break;
    }
}

// One group of four taps in phase PH; before its arithmetic it starts the loads of the next
// group: four sample pairs into the free ring quad, four tap pairs into the idle tap quad.
template <int DIR, int PH>
__device__ __forceinline__ void fir2_step(f2 (&acc)[kFirSeg], f2 (&w)[kFirRing], f2 (&f)[2][4],
                                          unsigned fp_next, unsigned xp)
{
    constexpr int base = win_reg<DIR, PH>(DIR < 0 ? -4 + kFirRing : kFirWin);
    ld2p(xp, w[base], w[base + 1]);
    ld2p(xp + 16, w[base + 2], w[base + 3]);
    ld2p(fp_next, f[(PH + 1) & 1][0], f[(PH + 1) & 1][1]);
    ld2p(fp_next + 16, f[(PH + 1) & 1][2], f[(PH + 1) & 1][3]);
    fir2_group<DIR, PH, 4>(acc, w, f[PH & 1]);
}

template <int DIR, int PH>
__device__ __forceinline__ void fir2_rest(f2 (&acc)[kFirSeg], f2 (&w)[kFirRing], f2 (&f)[2][4],
                                          unsigned fp_next, unsigned xp, int left, int tail)
{
    if (left == 0) {
        if (tail) fir2_group_n<DIR, PH>(acc, w, f[PH & 1], tail);
        return;
    }
    fir2_step<DIR, PH>(acc, w, f, fp_next, xp);
    if constexpr (PH + 1 < kFirPhases)
        fir2_rest<DIR, PH + 1>(acc, w, f, fp_next + 32, xp + (DIR < 0 ? 0u - 32u : 32u), left - 1, tail);
}


// Zero-skipping form of one 16-output segment.  Spike tensors are mostly zeros, and a zero
// sample leaves every accumulator it is multiplied into unchanged, so only the sample positions
// where at least one of the warp's 64 rows is non-zero need any arithmetic.  `colmask` holds one
// bit per staged sample position of the tile (bit set = some row is non-zero there).  The live
// positions of the segment's window are visited in the order that keeps every output's chain in
// ascending tap order (conv: newest sample first; corr: oldest first); each costs 16 packed FMAs
// with the 16 consecutive taps that connect it to the segment's outputs, read from a copy of the
// taps with 16 zeros in front and behind: a tap outside [0, K) multiplies the sample by zero,
// which changes nothing for finite samples (tiles that hold an Inf or NaN take the dense form).
// pos0 = tile position of the window's first sample.
constexpr int kFir2WinWords = 4;         // the zero-skipping segment holds its window's mask in 4 registers
constexpr int kFir2SparseMaxTaps = 32 * kFir2WinWords - kFirSeg + 1;      // 113: K + 15 positions fit 128 bits

template <int DIR>
__device__ __forceinline__ void fir2_sparse_segment(f2 (&acc)[kFirSeg], const unsigned *colmask, unsigned xrow_tile0,
                                                    unsigned fsA_addr, unsigned fsB_addr, int pos0, int K)
{
    // window: positions pos0 .. pos0 + K + 14 (K - 1 past samples + 16 outputs); its mask, bit j of
    // the 128-bit value = position pos0 + j, is cut out of the tile's mask once
    const int npos = K + kFirSeg - 1;
    const int w0 = pos0 >> 5, sh = pos0 & 31;
    unsigned m[kFir2WinWords];
#pragma unroll
    for (int k = 0; k < kFir2WinWords; ++k) {
        const unsigned lo = colmask[w0 + k], hi = colmask[w0 + k + 1];       // the mask array is padded
        m[k] = __funnelshift_r(lo, hi, sh);
        const int left = npos - 32 * k;                                        // window bits in this word
        if (left < 32) m[k] &= left > 0 ? (1u << left) - 1u : 0u;
    }
    // conv walks the live positions downwards from the last one, corr upwards from the first one
#pragma unroll
    for (int kk = 0; kk < kFir2WinWords; ++kk) {
        const int k = DIR < 0 ? kFir2WinWords - 1 - kk : kk;
        unsigned mk = m[k];
        while (mk) {
            const int b = DIR < 0 ? 31 - __clz(mk) : __ffs(mk) - 1;
            mk &= ~(1u << b);
            const int j = 32 * k + b;                                          // position pos0 + j
            const f2 x = ld1p(xrow_tile0 + 8u * (unsigned)(pos0 + j));
            // conv: output mm takes tap (K - 1 + mm) - j;  corr: tap j - mm
            const int a = DIR < 0 ? K - 1 - j : j - (kFirSeg - 1);             // lowest tap index of the 16
            const int n0 = a + kFirSeg;                                        // index into the padded table (>= 1)
            const unsigned tp = ((n0 & 1) ? fsB_addr + 8u * (unsigned)(n0 - 1) : fsA_addr + 8u * (unsigned)n0);
            f2 f[kFirSeg];
#pragma unroll
            for (int q = 0; q < kFirSeg / 2; ++q) ld2p(tp + 16 * q, f[2 * q], f[2 * q + 1]);
#pragma unroll
            for (int mm = 0; mm < kFirSeg; ++mm) fma2_acc(acc[mm], x, f[DIR < 0 ? mm : kFirSeg - 1 - mm]);
        }
    }
}

// V: width of the global accesses in floats (4, 2 or 1; T % V == 0 and both `in` (unless PK) and
// `out` aligned to 4*V bytes).
// PK: the input is a bit-packed spike tensor (`in` points to 32-bit words, ceil(T / 32) per row,
// bit i of word w = sample 32 w + i is `spike_value`, else 0); the words are staged and the
// re-pack pass expands them.
template <int DIR, int V, bool PK = false>
__global__ void __launch_bounds__(kFirMaxWarps * 32, 1)
fir2_kernel(float *__restrict__ out, const float *__restrict__ in, const float *__restrict__ filt,
            int64_t rows, int T, int K, float Ts, FirShape sh, int64_t ntiles, bool sparse_ok, float spike_value,
            const int *skip_flag)
{
    if (skip_flag != nullptr && *skip_flag != 0) return;      // the event-driven kernel has this call
    extern __shared__ __align__(16) float smem[];
    const int Tt = sh.nseg * kFirSeg;
    const int WX = Tt + sh.halo;
    const int KP = ((K + 3) & ~3) + 4;       // taps, zero padded; one spare quad for the look-ahead load
    const int KS = ((K + 3) & ~3) + 2 * kFirSeg;   // taps with 16 zeros in front and at least 16 behind (sparse path)
    const int SXs = PK ? kFir2StageWords : ((WX + 3) & ~3);     // staging: words per row
    float *fs = smem;                        // 2 * KP words: every tap twice
    float *fsA = fs + 2 * KP;                // 2 * KS words: padded taps, every tap twice
    float *fsB = fsA + 2 * KS;               // the same, one tap further on (16-byte alignment for odd starts)
    unsigned *colmask = reinterpret_cast<unsigned *>(fsB + 2 * KS);     // 2 x kFir2MaskWords words, then 2 flags (+2 pad)
    unsigned *nonfinite = colmask + 2 * kFir2MaskWords;
    float *stage = reinterpret_cast<float *>(nonfinite + 4);            // [64 rows x SXs]
    float *xbuf = stage + kFir2Rows * SXs;                              // [32 row pairs x SX], interleaved

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;

    for (int i = threadIdx.x; i < KP; i += blockDim.x) {
        const float v = i < K ? filt[i] : 0.0f;
        fs[2 * i] = v;
        fs[2 * i + 1] = v;
    }
    for (int n = threadIdx.x; n < KS; n += blockDim.x) {       // padded tap n = tap n - 16
        const float a = (n >= kFirSeg && n - kFirSeg < K) ? filt[n - kFirSeg] : 0.0f;
        const float b = (n + 1 >= kFirSeg && n + 1 - kFirSeg < K) ? filt[n + 1 - kFirSeg] : 0.0f;
        fsA[2 * n] = a;
        fsA[2 * n + 1] = a;
        fsB[2 * n] = b;
        fsB[2 * n + 1] = b;
    }
    for (int i = threadIdx.x; i < 2 * kFir2MaskWords + 4; i += blockDim.x) colmask[i] = 0u;

    // asynchronous copy of one input tile into the staging buffer: warp w fills rows w,
    // w+nwarps, ... from contiguous global segments; samples outside the row (or rows outside
    // the array) become zeros.  With 16-byte accesses a lane copies at most four chunks per row,
    // and which of them lie inside [0, T) is the same for every row of the tile.
    const unsigned stage_saddr = (unsigned)__cvta_generic_to_shared(stage);
    const unsigned xbuf_saddr = (unsigned)__cvta_generic_to_shared(xbuf);
    auto tile_origin = [&](int64_t tile, int64_t &row0, int &t0) {
        const int64_t rb = tile / sh.ttiles;
        t0 = (int)(tile - rb * sh.ttiles) * Tt;
        row0 = rb * kFir2Rows;
    };
    auto fill = [&](int64_t tile) {
        int64_t row0;
        int t0;
        tile_origin(tile, row0, t0);
        const int64_t nrow = rows - row0;
        const int g0 = DIR < 0 ? t0 - sh.halo : t0;      // global time of tile position 0
        if constexpr (PK) {
            // the words that hold samples g0 .. g0 + WX - 1 of each row, word index w_lo + lane
            const unsigned *words_in = reinterpret_cast<const unsigned *>(in);
            const int words = (T + 31) >> 5;
            const int wi = (g0 >> 5) + lane;             // arithmetic shift: floor for negative g0
            const bool word_ok = lane < kFir2StageWords && wi >= 0 && wi < words;
            if (lane < kFir2StageWords) {
                for (int r = warp; r < kFir2Rows; r += nwarps) {
                    const bool ok = word_ok && r < nrow;
                    cp_async<4>(stage + r * kFir2StageWords + lane, ok ? words_in + (row0 + r) * (int64_t)words + wi : words_in, ok);
                }
            }
        } else if constexpr (V == 4) {
            constexpr int kChunks = (kFir2MaxSamples + 127) / 128;     // 4
            int goff[kChunks], nbytes[kChunks];          // source offset in the row; 16, 0 (zero fill) or -1 (no chunk)
#pragma unroll
            for (int k = 0; k < kChunks; ++k) {
                const int pcol = lane * 4 + 128 * k;
                const int gt = g0 + pcol;
                const bool ok = gt >= 0 && gt < T;
                goff[k] = ok ? gt : 0;
                nbytes[k] = pcol < WX ? (ok ? 16 : 0) : -1;
            }
            for (int r = warp; r < kFir2Rows; r += nwarps) {
                const bool row_ok = r < nrow;
                const float *src = in + (row0 + (row_ok ? r : 0)) * (int64_t)T;
                const unsigned dst = stage_saddr + 4u * (unsigned)(r * SXs + lane * 4);
#pragma unroll
                for (int k = 0; k < kChunks; ++k) {
                    if (nbytes[k] < 0) continue;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n"
                                 ::"r"(dst + 512u * k), "l"(src + goff[k]), "r"(row_ok ? nbytes[k] : 0) : "memory");
                }
            }
        } else {
            for (int r = warp; r < kFir2Rows; r += nwarps) {
                const bool row_ok = r < nrow;
                const float *src = in + (row0 + (row_ok ? r : 0)) * (int64_t)T;
                float *dst = stage + r * SXs;
                for (int pcol = lane * V; pcol < WX; pcol += 32 * V) {
                    const int gt = g0 + pcol;
                    const bool ok = row_ok && gt >= 0 && gt < T;
                    cp_async<4 * V>(dst + pcol, ok ? src + gt : in, ok);
                }
            }
        }
        cp_async_commit();
    };

    // Re-pack the staged tile into the interleaved tile: pair p = rows 2p and 2p+1.  With `note`
    // the pass also records, in mask[] (one bit per sample position, set by atomic OR), where any
    // row is non-zero, and in *flag whether any sample is Inf or NaN.
    auto repack = [&](int64_t tile, bool note, unsigned *mask, unsigned *flag) {
        if constexpr (PK) {
            int64_t row0;
            int t0;
            tile_origin(tile, row0, t0);
            const int g0 = DIR < 0 ? t0 - sh.halo : t0;
            const int w_lo = g0 >> 5;
            const unsigned *sw = reinterpret_cast<const unsigned *>(stage);
            for (int p = warp; p < kFir2Rows / 2; p += nwarps) {
                const unsigned *wa = sw + (2 * p) * kFir2StageWords, *wb = wa + kFir2StageWords;
                float *dst = xbuf + p * sh.SX;
                for (int pos = lane; pos < ((WX + 31) & ~31); pos += 32) {
                    const int gt = g0 + pos;
                    const int wi = (gt >> 5) - w_lo;                 // 0 .. kFir2StageWords - 1
                    const unsigned inside = gt < T ? 1u : 0u;           // bits past the row end are ignored
                    const unsigned ba = (wa[wi] >> (gt & 31)) & inside, bb = (wb[wi] >> (gt & 31)) & inside;
                    if (pos < WX)
                        *reinterpret_cast<float2 *>(dst + 2 * pos) = make_float2(ba ? spike_value : 0.0f, bb ? spike_value : 0.0f);
                    const unsigned live = __ballot_sync(0xffffffffu, pos < WX && (ba | bb));
                    if (note && lane == 0 && live) atomicOr(mask + (pos >> 5), live);
                }
            }
        } else {
            const int chunks = SXs >> 2;                 // 16-byte chunks per staged row
            for (int p = warp; p < kFir2Rows / 2; p += nwarps) {
                const unsigned sa = stage_saddr + 4u * (unsigned)((2 * p) * SXs), sb = sa + 4u * (unsigned)SXs;
                const unsigned dst = xbuf_saddr + 4u * (unsigned)(p * sh.SX);
                for (int c = lane; c < chunks; c += 32) {
                    const float4 a = ld4(sa + 16u * c), b = ld4(sb + 16u * c);
                    st4(dst + 32u * c, a.x, b.x, a.y, b.y);
                    st4(dst + 32u * c + 16u, a.z, b.z, a.w, b.w);
                    if (note) {
                        const unsigned m0 = __float_as_uint(a.x) | __float_as_uint(b.x), m1 = __float_as_uint(a.y) | __float_as_uint(b.y);
                        const unsigned m2 = __float_as_uint(a.z) | __float_as_uint(b.z), m3 = __float_as_uint(a.w) | __float_as_uint(b.w);
                        const unsigned nib = ((m0 & 0x7fffffffu) ? 1u : 0u) | ((m1 & 0x7fffffffu) ? 2u : 0u) |
                                             ((m2 & 0x7fffffffu) ? 4u : 0u) | ((m3 & 0x7fffffffu) ? 8u : 0u);
                        if (nib) atomicOr(mask + (c >> 3), nib << ((c & 7) * 4));
                        // 0 * v is NaN exactly when v is Inf or NaN, and NaN survives the sum
                        float z = a.x * 0.0f;
                        z = fmaf(a.y, 0.0f, z); z = fmaf(a.z, 0.0f, z); z = fmaf(a.w, 0.0f, z);
                        z = fmaf(b.x, 0.0f, z); z = fmaf(b.y, 0.0f, z); z = fmaf(b.z, 0.0f, z); z = fmaf(b.w, 0.0f, z);
                        if (z != z) *flag = 1u;
                    }
                }
            }
        }
    };

    const int groups = K >> 2;          // full groups of 4 taps
    const int tail = K & 3;
    constexpr unsigned step = DIR < 0 ? 0u - 32u : 32u;   // bytes the window moves per group (mod 2^32)
    const unsigned fs_addr = (unsigned)__cvta_generic_to_shared(fs);
    const unsigned fsA_addr = (unsigned)__cvta_generic_to_shared(fsA);
    const unsigned fsB_addr = (unsigned)__cvta_generic_to_shared(fsB);
    const int mask_words = (WX + 31) >> 5;
    const bool may_skip = sparse_ok && K >= 8 && K <= kFir2SparseMaxTaps && (!PK || (__float_as_uint(spike_value) & 0x7f800000u) != 0x7f800000u);
    bool sparse = false;                 // the last tile looked at was mostly zeros (same value in every thread)

    int64_t tile = blockIdx.x;
    if (tile < ntiles) fill(tile);
    for (int it = 0; tile < ntiles; tile += gridDim.x, ++it) {
        cp_async_wait<0>();
        __syncthreads();                 // the staged tile has landed; nobody reads the interleaved tile any more
        // zeros are looked for in every tile while tiles are sparse (and always for packed input,
        // where it costs one ballot), else in one tile out of kFir2ScanEvery
        const bool note = may_skip && (PK || sparse || (it % kFir2ScanEvery) == 0);
        unsigned *mask = colmask + (it & 1) * kFir2MaskWords;
        repack(tile, note, mask, nonfinite + (it & 1));
        __syncthreads();                 // the interleaved tile is complete; the staging buffer is free again
        const int64_t next = tile + gridDim.x;
        if (next < ntiles) fill(next);
        if (note) {
            int live = 0;
            for (int wd = 0; wd < mask_words; ++wd) live += __popc(mask[wd]);
            sparse = nonfinite[it & 1] == 0u && live * 100 < kFir2SparsePercent * WX;
        } else {
            sparse = false;
        }
        // clear the other mask for the next tile (its last readers passed the first barrier)
        if (threadIdx.x < kFir2MaskWords) colmask[((it + 1) & 1) * kFir2MaskWords + threadIdx.x] = 0u;
        if (threadIdx.x == kFir2MaskWords) nonfinite[(it + 1) & 1] = 0u;

        int64_t row0;
        int t0;
        tile_origin(tile, row0, t0);
        const int64_t rowA = row0 + 2 * lane;
        // byte address of tile position 0 of this lane's row pair
        const unsigned xtile0 = xbuf_saddr + 4u * (unsigned)(lane * sh.SX);
        const unsigned xrow = xtile0 + 8u * (unsigned)(DIR < 0 ? sh.halo : 0);

        for (int seg = warp; seg < sh.nseg; seg += nwarps) {
            const int tb = seg * kFirSeg;
            if (t0 + tb >= T) break;    // whole segment beyond the row end (warp-uniform)
            f2 acc[kFirSeg];
#pragma unroll
            for (int m = 0; m < kFirSeg; ++m) acc[m] = 0ull;

            if (sparse) {
                // window of the segment in tile positions: conv starts K - 1 samples before the
                // first output (tile position halo + tb), corr at the first output
                fir2_sparse_segment<DIR>(acc, mask, xtile0, fsA_addr, fsB_addr, DIR < 0 ? sh.halo + tb - (K - 1) : tb, K);
            } else {
                // initial window (phase 0): conv x[tb-4 .. tb+16), corr x[tb .. tb+20)
                f2 w[kFirRing];
                const unsigned x0 = xrow + 8u * (unsigned)tb - (DIR < 0 ? 32u : 0u);
#pragma unroll
                for (int q = 0; q < kFirWin / 2; ++q) ld2p(x0 + 16 * q, w[2 * q], w[2 * q + 1]);
                unsigned xp = DIR < 0 ? x0 - 32 : x0 + 8 * kFirWin;    // next four sample pairs to fetch
                unsigned fp = fs_addr;
                f2 f[2][4];
                ld2p(fp, f[0][0], f[0][1]);
                ld2p(fp + 16, f[0][2], f[0][3]);
                int g = 0;
                for (; g + kFirPhases <= groups; g += kFirPhases) {
                    fir2_step<DIR, 0>(acc, w, f, fp + 32, xp);
                    fir2_step<DIR, 1>(acc, w, f, fp + 64, xp + step);
                    fir2_step<DIR, 2>(acc, w, f, fp + 96, xp + 2 * step);
                    fir2_step<DIR, 3>(acc, w, f, fp + 128, xp + 3 * step);
                    fir2_step<DIR, 4>(acc, w, f, fp + 160, xp + 4 * step);
                    fir2_step<DIR, 5>(acc, w, f, fp + 192, xp + 5 * step);
                    xp += kFirPhases * step;
                    fp += 32 * kFirPhases;
                }
                fir2_rest<DIR, 0>(acc, w, f, fp + 32, xp, groups - g, tail);
            }

            float oa[kFirSeg], ob[kFirSeg];
#pragma unroll
            for (int m = 0; m < kFirSeg; ++m) {
                unpack2(acc[m], oa[m], ob[m]);
                oa[m] *= Ts;
                ob[m] *= Ts;
            }
            const int left = T - (t0 + tb);          // > 0, multiple of V
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int64_t row = rowA + h;
                if (row >= rows) continue;
                const float *o = h ? ob : oa;
                float *dst = out + row * (int64_t)T + t0 + tb;
                if (V == 4) {
#pragma unroll
                    for (int q = 0; q < kFirSeg / 4; ++q)
                        if (4 * q < left)
                            *reinterpret_cast<float4 *>(dst + 4 * q) = make_float4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
                } else if (V == 2) {
#pragma unroll
                    for (int q = 0; q < kFirSeg / 2; ++q)
                        if (2 * q < left) *reinterpret_cast<float2 *>(dst + 2 * q) = make_float2(o[2 * q], o[2 * q + 1]);
                } else {
#pragma unroll
                    for (int q = 0; q < kFirSeg; ++q)
                        if (q < left) dst[q] = o[q];
                }
            }
        }
    }
    cp_async_wait<0>();
}


// ---------------------------------------------------------------------------------------
// The scalar kernel without a CTA-wide barrier per tile ("flow" form, the default).
//
// fir_kernel above synchronises its warps at every tile; with 19 segments over 8 warps three
// warps carry 3 segments and five carry 2, so about a fifth of the warp-time of a tile is spent
// waiting at the barrier (barrier stalls are the largest stall reason in its profile).  Here
// the 16-sample segments of all tiles of a CTA form one sequence that is dealt out to the warps
// round robin, across tile boundaries, so every warp gets the same number of segments in the
// long run, and the two hand-overs of a double-buffered tile are split-phase barriers in shared
// memory (mbarrier) that nobody has to reach at the same time:
//   landed[b]  every thread attaches its cp.async copies of a tile to it
//              (cp.async.mbarrier.arrive.noinc); a warp waits for it before its first segment
//              of that tile;
//   free[b]    a warp arrives when it has finished its segments of the tile in buffer b; a warp
//              waits for it before it copies the tile after next into that buffer, which it
//              does after its first segment of the tile in between - so a fast warp always has
//              a segment to work on while the slow ones finish.
// Arithmetic, tile layout and results are those of fir_kernel.  Every wait is bounded: a warp
// that gives up records kStatusFirWaitTimeout in the device status word and leaves.
// ---------------------------------------------------------------------------------------
constexpr int kStatusFirWaitTimeout = 0x5102;
constexpr int kFirPollLimit = 1 << 22;

__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// the barrier's pending count was initialised to include this arrival, which happens when the
// cp.async copies this thread has issued so far have completed
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t *bar)
{
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// MINB = 2 caps the registers at 64 per thread (two CTAs of up to 16 warps per SM); MINB = 1 lets
// the compiler take about 110, which two CTAs of 8 warps still fit.
// Poll a barrier at most `limit` times.  Returns false if the phase did not complete; the result
// is the same in every lane of the warp.  (Backing off between polls with nanosleep, and issuing
// the next tile's copy before the first segment when the buffer is already free, were both
// measured and both cost 4-6 %.)
__device__ __forceinline__ bool fir_wait(uint64_t *bar, unsigned parity, int limit)
{
    return !__any_sync(0xffffffffu, !mbar_wait_bounded(bar, parity, limit));
}

// PK: `in` points to bit-packed spikes (32-bit words, ceil(T / 32) per row, bit b of word w =
// "sample 32 w + b is spike_value"); the words a tile needs are copied into a small staging slot
// two tiles ahead and the warps expand their rows into the same fp32 tile the copies would have
// filled, so the arithmetic and the results are those of the fp32 input.  V then is the access
// width of `out`.
// RHO: every output is multiplied by the surrogate gradient of the spike function at the
// potential `rho.u` of the same row and step, out = (Ts * sum) * (c * exp(-|u - theta| / tau)):
// the filtered value rounded to fp32 exactly as it would have been stored, then the expression
// of the separate surrogate-gradient pass - the backward of "spike, then psp" in one launch.
struct FirRho {
    const float *u;
    float theta, tau, c;
    float tau_inv;          // 1 / tau, correctly rounded (computed once on the host)
};

// a / b rounded to nearest for a divisor that is the same for the whole launch, from its
// correctly rounded reciprocal y: q0 = a y, then two residual corrections with fused
// multiply-adds (r = a - b q exactly; q + r y rounds to the quotient - Markstein's theorem; the
// second step is a safety margin).  The hardware division costs one pass through the
// special-function unit per element, which this epilogue cannot hide behind memory time as the
// separate surrogate-gradient pass does.  Infinite or NaN a, and quotients that overflow, return
// q0, which then already is the quotient's value.
__device__ __forceinline__ float div_by_launch_constant(float a, float b, float y)
{
    const float q0 = a * y;
    const float r0 = fmaf(-b, q0, a);
    const float q1 = fmaf(r0, y, q0);
    const float r1 = fmaf(-b, q1, a);
    const float q2 = fmaf(r1, y, q1);
    return fabsf(q0) <= FLT_MAX ? q2 : q0;
}

// rho_times (common.cuh) with the division above: g * (c * exp(-|u - theta| / tau))
__device__ __forceinline__ float rho_times_fir(float g, float u, const FirRho &rho)
{
    const float e = expf(div_by_launch_constant(-fabsf(u - rho.theta), rho.tau, rho.tau_inv));
    return g * (rho.c * e);
}

// SH (with V = 4): rows that do not start on 16-byte boundaries although the arrays do (T % 4 != 0).
// Row R starts s = (R T) mod 4 samples past a boundary; its shared-memory row is filled from that
// boundary on, so position p holds sample g0 + p - s, every copy is a 16-byte copy again, and the
// lane of the row produces the outputs of the samples s earlier than its neighbours' - which puts
// its 16-byte stores on boundaries too.  Only the quads that contain a row's first or last
// sample are handled element by element.
// RX: how the groups of four taps that do not fill a run of six are handled.  false: behind the
// loop over whole runs (up to five more group bodies); true: the loop is left where the groups
// end, so that no group body exists twice - the code a segment walks through then fits the
// instruction cache whatever K is (110 taps, 4 runs + 3 groups: 1.02 -> 0.83 ms per 131072 x
// 1448), at the price of a compare and branch per group (77 taps, 3 runs + 1: 3 % slower).
template <int DIR, int V, int MINB, bool PK = false, bool RHO = false, bool SH = false, bool RX = false>
__global__ void __launch_bounds__(kFirMaxWarps * 32, MINB)
fir_flow_kernel(float *__restrict__ out, const float *__restrict__ in, const float *__restrict__ filt,
                int64_t rows, int T, int K, float Ts, FirShape sh, int64_t ntiles, int *status, const int *skip_flag,
                float spike_value, FirRho rho)
{
    if (skip_flag != nullptr && *skip_flag != 0) return;      // the event-driven kernel has this call
    extern __shared__ __align__(16) float smem[];
    const int Tt = sh.nseg * kFirSeg;
    const int WX = Tt + sh.halo;
    const int KP = ((K + 3) & ~3) + 4;       // taps, zero padded; one spare quad for the look-ahead load
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);      // landed[0], landed[1], free[0], free[1]
    float *fs = smem + 8;
    float *xbuf = fs + KP;                   // 2 x [kFirRows x SX]
    const int tile_words = kFirRows * sh.SX;

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;

    for (int i = threadIdx.x; i < KP; i += blockDim.x) fs[i] = i < K ? filt[i] : 0.0f;
    if (threadIdx.x == 0) {
        mbar_init(bars + 0, blockDim.x);
        mbar_init(bars + 1, blockDim.x);
        mbar_init(bars + 2, nwarps);
        mbar_init(bars + 3, nwarps);
        mbar_init_fence();
    }
    __syncthreads();

    // PK: two staging slots of [32 rows x kFirStageWords] words behind the tiles.  A warp copies
    // (and later expands) the words of its own rows only, so its own cp.async groups order them.
    unsigned *stage = reinterpret_cast<unsigned *>(xbuf + 2 * tile_words);
    auto stage_words = [&](int slot, int64_t tile) {
        if (tile < ntiles) {
            const int64_t rb = tile / sh.ttiles;
            const int t0 = (int)(tile - rb * sh.ttiles) * Tt;
            const int64_t row0 = rb * kFirRows;
            const int64_t nrow = rows - row0;
            const int w0 = (DIR < 0 ? t0 - sh.halo : t0) >> 5;
            const unsigned *words = reinterpret_cast<const unsigned *>(in);
            const int nwords = (T + 31) >> 5;
            if (lane < kFirStageWords) {
                for (int r = warp; r < kFirRows; r += nwarps) {
                    const bool ok = r < nrow && w0 + lane >= 0 && w0 + lane < nwords;
                    cp_async<4>(stage + (slot * kFirRows + r) * kFirStageWords + lane,
                                ok ? words + (row0 + r) * (int64_t)nwords + (w0 + lane) : words, ok);
                }
            }
        }
        cp_async_commit();
    };
    const unsigned xbuf_saddr = (unsigned)__cvta_generic_to_shared(xbuf);
    auto fill = [&](int buf, int64_t tile) {
        float *xs = xbuf + buf * tile_words;
        const int64_t rb = tile / sh.ttiles;
        const int t0 = (int)(tile - rb * sh.ttiles) * Tt;
        const int64_t row0 = rb * kFirRows;
        const int64_t nrow = rows - row0;
        const int g0 = DIR < 0 ? t0 - sh.halo : t0;      // global time of tile position 0
        if constexpr (PK) {
            // The words of this tile were copied into staging slot `buf` two fills ago (see
            // stage_words below): expand them.  Tile position 4 * lane + 128 k holds samples
            // g0 + that .. + 3; g0 is a multiple of four, so the four bits lie in one word.
            constexpr int kChunks = (kFirTileWordsPerRow + 127) / 128;     // 4
            cp_async_wait<1>();              // all but the copies for the tile after this one
            __syncwarp();
            const unsigned *st = stage + buf * (kFirRows * kFirStageWords);
            const int w0 = g0 >> 5;          // (arithmetic shift: g0 may be negative)
            for (int r = warp; r < kFirRows; r += nwarps) {
#pragma unroll
                for (int k = 0; k < kChunks; ++k) {
                    const int pcol = lane * 4 + 128 * k;
                    if (pcol >= WX) continue;
                    const int gt = g0 + pcol;
                    unsigned m = st[r * kFirStageWords + ((gt >> 5) - w0)] >> (gt & 31);
                    const int left = T - gt;                 // bits past the row end do not count
                    if (left < 4) m &= left > 0 ? (1u << left) - 1u : 0u;
                    *reinterpret_cast<float4 *>(xs + r * sh.SX + pcol) =
                        make_float4((m & 1u) ? spike_value : 0.0f, (m & 2u) ? spike_value : 0.0f,
                                    (m & 4u) ? spike_value : 0.0f, (m & 8u) ? spike_value : 0.0f);
                }
            }
            __syncwarp();                    // the slot has been read: it takes the words of the tile two further on
            stage_words(buf, tile + 2 * (int64_t)gridDim.x);
            mbar_arrive(bars + buf);         // (release) this thread's part of the tile is in place
            return;
        }
        if constexpr (SH) {
            constexpr int kChunks = (kFirTileWordsPerRow + 127) / 128;     // 4
            for (int r = warp; r < kFirRows; r += nwarps) {
                const bool row_ok = r < nrow;
                const int64_t R = row0 + (row_ok ? r : 0);
                const int srow = (int)((R * (int64_t)T) & 3);       // samples the row starts past a 16-byte boundary
                const float *src = in + R * (int64_t)T;
                float *drow = xs + r * sh.SX;
#pragma unroll
                for (int k = 0; k < kChunks; ++k) {
                    const int pcol = lane * 4 + 128 * k;
                    if (pcol >= WX) continue;
                    const int gt = g0 + pcol - srow;                // sample of the chunk's first element
                    const unsigned dst = xbuf_saddr + 4u * (unsigned)(buf * tile_words + r * sh.SX + pcol);
                    if (!row_ok || gt >= T || gt + 4 <= 0) {
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, 0;\n" ::"r"(dst), "l"(in) : "memory");
                    } else if (gt >= 0) {
                        // whole chunk, or the row's last samples and zeros behind them
                        const int bytes = gt + 4 <= T ? 16 : 4 * (T - gt);
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src + gt), "r"(bytes) : "memory");
                    } else {
                        // the row's first samples with zeros in front: element by element
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const bool ok = gt + j >= 0 && gt + j < T;
                            cp_async<4>(drow + pcol + j, ok ? src + gt + j : in, ok);
                        }
                    }
                }
            }
        } else if constexpr (V == 4) {
            constexpr int kChunks = (kFirTileWordsPerRow + 127) / 128;     // 4
            int goff[kChunks], nbytes[kChunks];          // source offset in the row; 16, 0 (zero fill) or -1 (no chunk)
#pragma unroll
            for (int k = 0; k < kChunks; ++k) {
                const int pcol = lane * 4 + 128 * k;
                const int gt = g0 + pcol;
                const bool ok = gt >= 0 && gt < T;
                goff[k] = ok ? gt : 0;
                nbytes[k] = pcol < WX ? (ok ? 16 : 0) : -1;
            }
            for (int r = warp; r < kFirRows; r += nwarps) {
                const bool row_ok = r < nrow;
                const float *src = in + (row0 + (row_ok ? r : 0)) * (int64_t)T;
                const unsigned dst = xbuf_saddr + 4u * (unsigned)(buf * tile_words + r * sh.SX + lane * 4);
#pragma unroll
                for (int k = 0; k < kChunks; ++k) {
                    if (nbytes[k] < 0) continue;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n"
                                 ::"r"(dst + 512u * k), "l"(src + goff[k]), "r"(row_ok ? nbytes[k] : 0) : "memory");
                }
            }
        } else {
            for (int r = warp; r < kFirRows; r += nwarps) {
                const bool row_ok = r < nrow;
                const float *src = in + (row0 + (row_ok ? r : 0)) * (int64_t)T;
                float *dst = xs + r * sh.SX;
                for (int pcol = lane * V; pcol < WX; pcol += 32 * V) {
                    const int gt = g0 + pcol;
                    const bool ok = row_ok && gt >= 0 && gt < T;
                    cp_async<4 * V>(dst + pcol, ok ? src + gt : in, ok);
                }
            }
        }
        cp_async_arrive_noinc(bars + buf);
    };

    const int groups = K >> 2;          // full groups of 4 taps
    const int tail = K & 3;
    constexpr unsigned step = DIR < 0 ? 0u - 16u : 16u;   // bytes the window moves per group (mod 2^32)
    const unsigned fs_addr = (unsigned)__cvta_generic_to_shared(fs);

    // this CTA's tiles: blockIdx.x, blockIdx.x + gridDim.x, ...
    const int64_t first = blockIdx.x;
    const int n = first < ntiles ? (int)((ntiles - first + gridDim.x - 1) / gridDim.x) : 0;
    if constexpr (PK) {
        stage_words(0, first);
        stage_words(1, first + gridDim.x);
    }
    if (n > 0) fill(0, first);
    if (n > 1) fill(1, first + gridDim.x);
    bool gave_up = false;
    int unit0 = warp;                   // this warp's next segment in the CTA-wide sequence, minus it * nseg
    for (int it = 0; it < n && !gave_up; ++it) {
        const int b = it & 1;
        const int64_t tile = first + (int64_t)it * gridDim.x;
        if (!fir_wait(bars + b, (unsigned)(it >> 1) & 1u, kFirPollLimit)) {
            gave_up = true;
            break;
        }
        const int64_t rb = tile / sh.ttiles;
        const int t0 = (int)(tile - rb * sh.ttiles) * Tt;
        const int64_t row = rb * kFirRows + lane;
        // byte address of tile position 0 of this lane's row
        const unsigned xrow = xbuf_saddr + 4u * (unsigned)(b * tile_words + lane * sh.SX + (DIR < 0 ? sh.halo : 0));

        // the tile after this one goes into the other buffer once every warp is done with the tile
        // that is in it now; this warp sees to its rows after its first segment of this tile
        bool next_pending = it >= 1 && it + 1 < n;
        const unsigned free_parity = (unsigned)((it - 1) >> 1) & 1u;
        auto fill_next = [&]() {
            if (!fir_wait(bars + 2 + (b ^ 1), free_parity, kFirPollLimit)) {
                gave_up = true;
                return;
            }
            fill(b ^ 1, tile + gridDim.x);
        };

        int seg = unit0;
        for (; seg < sh.nseg && !gave_up; seg += nwarps) {
            const int tb = seg * kFirSeg;
            if (t0 + tb < T + (SH ? 3 : 0)) {          // else: whole segment beyond the row end (warp-uniform)
                // SH: this lane's outputs are those of the samples srow earlier
                const int srow = SH ? (int)(((row < rows ? row : 0) * (int64_t)T) & 3) : 0;
                float acc[kFirSeg];
#pragma unroll
                for (int m = 0; m < kFirSeg; ++m) acc[m] = 0.0f;

                // RHO: the potentials of this thread's 16 outputs are requested now and used after
                // the arithmetic, a few microseconds later
                float uv[RHO ? kFirSeg : 1];
                if constexpr (RHO) {
                    const int left = T - (t0 + tb);
                    const float *up = rho.u + (row < rows ? row : 0) * (int64_t)T + t0 + tb - srow;
                    if (SH) {
                        const int tf = t0 + tb - srow;              // sample of this lane's first output
#pragma unroll
                        for (int q = 0; q < kFirSeg / 4; ++q) {
                            float4 t4 = make_float4(0.f, 0.f, 0.f, 0.f);
                            const int tq = tf + 4 * q;
                            if (tq >= 0 && tq + 4 <= T) {
                                asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];"
                                             : "=f"(t4.x), "=f"(t4.y), "=f"(t4.z), "=f"(t4.w) : "l"(up + 4 * q));
                            } else {
                                if (tq >= 0 && tq < T) t4.x = __ldg(up + 4 * q);
                                if (tq + 1 >= 0 && tq + 1 < T) t4.y = __ldg(up + 4 * q + 1);
                                if (tq + 2 >= 0 && tq + 2 < T) t4.z = __ldg(up + 4 * q + 2);
                                if (tq + 3 >= 0 && tq + 3 < T) t4.w = __ldg(up + 4 * q + 3);
                            }
                            uv[4 * q] = t4.x; uv[4 * q + 1] = t4.y; uv[4 * q + 2] = t4.z; uv[4 * q + 3] = t4.w;
                        }
                    } else if (V == 4) {
#pragma unroll
                        for (int q = 0; q < kFirSeg / 4; ++q) {
                            float4 t4 = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (4 * q < left)
                                asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];"
                                             : "=f"(t4.x), "=f"(t4.y), "=f"(t4.z), "=f"(t4.w) : "l"(up + 4 * q));
                            uv[4 * q] = t4.x; uv[4 * q + 1] = t4.y; uv[4 * q + 2] = t4.z; uv[4 * q + 3] = t4.w;
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < kFirSeg; ++q) {
                            uv[q] = 0.0f;
                            if (q < left) asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(uv[q]) : "l"(up + q));
                        }
                    }
                }

                // initial window (phase 0): conv x[tb-4 .. tb+16), corr x[tb .. tb+20)
                float w[kFirRing];
                const unsigned x0 = xrow + 4u * (unsigned)tb - (DIR < 0 ? 16u : 0u);
#pragma unroll
                for (int q = 0; q < kFirWin / 4; ++q) put4(w, 4 * q, ld4(x0 + 16 * q));
                unsigned xp = DIR < 0 ? x0 - 16 : x0 + 4 * kFirWin;    // next sample quad to fetch
                unsigned fp = fs_addr;
                float4 f[2];
                f[0] = ld4(fp);
                if constexpr (!RX) {
                    int g = 0;
                    for (; g + kFirPhases <= groups; g += kFirPhases) {
                        fir_step<DIR, 0>(acc, w, f, fp, xp);
                        fir_step<DIR, 1>(acc, w, f, fp, xp);
                        fir_step<DIR, 2>(acc, w, f, fp, xp);
                        fir_step<DIR, 3>(acc, w, f, fp, xp);
                        fir_step<DIR, 4>(acc, w, f, fp, xp);
                        fir_step<DIR, 5>(acc, w, f, fp, xp);
                        xp += kFirPhases * step;
                        fp += 16 * kFirPhases;
                    }
                    fir_rest<DIR, 0>(acc, w, f, fp, xp, groups - g, tail);
                } else {
                    // Several groups left over after the runs of six: leave the run where the
                    // groups end instead of repeating up to five group bodies behind the loop -
                    // the code a segment walks through stays small enough for the instruction
                    // cache (110 taps: 27 groups = 4 runs + 3).
                    int n = groups;
                    for (;;) {
                        if (n == 0) { fir_tail<DIR, 0>(acc, w, f, tail); break; }
                        fir_step<DIR, 0>(acc, w, f, fp, xp);
                        if (n == 1) { fir_tail<DIR, 1>(acc, w, f, tail); break; }
                        fir_step<DIR, 1>(acc, w, f, fp, xp);
                        if (n == 2) { fir_tail<DIR, 2>(acc, w, f, tail); break; }
                        fir_step<DIR, 2>(acc, w, f, fp, xp);
                        if (n == 3) { fir_tail<DIR, 3>(acc, w, f, tail); break; }
                        fir_step<DIR, 3>(acc, w, f, fp, xp);
                        if (n == 4) { fir_tail<DIR, 4>(acc, w, f, tail); break; }
                        fir_step<DIR, 4>(acc, w, f, fp, xp);
                        if (n == 5) { fir_tail<DIR, 5>(acc, w, f, tail); break; }
                        fir_step<DIR, 5>(acc, w, f, fp, xp);
                        n -= kFirPhases;
                        xp += kFirPhases * step;
                        fp += 16 * kFirPhases;
                    }
                }

                if (row < rows) {
                    float *dst = out + row * (int64_t)T + t0 + tb;
                    const int left = T - (t0 + tb);          // > 0, multiple of V
                    if constexpr (RHO) {
#pragma unroll
                        for (int q = 0; q < kFirSeg; ++q) acc[q] = rho_times_fir(acc[q] * Ts, uv[q], rho);
                    } else {
#pragma unroll
                        for (int q = 0; q < kFirSeg; ++q) acc[q] *= Ts;
                    }
                    if (SH) {
                        const int tf = t0 + tb - srow;              // sample of this lane's first output
                        float *d = dst - srow;
#pragma unroll
                        for (int q = 0; q < kFirSeg / 4; ++q) {
                            const int tq = tf + 4 * q;
                            if (tq >= 0 && tq + 4 <= T) {
                                *reinterpret_cast<float4 *>(d + 4 * q) = make_float4(
                                    acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
                            } else {
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                    if (tq + j >= 0 && tq + j < T) d[4 * q + j] = acc[4 * q + j];
                            }
                        }
                    } else if (V == 4) {
#pragma unroll
                        for (int q = 0; q < kFirSeg / 4; ++q)
                            if (4 * q < left)
                                *reinterpret_cast<float4 *>(dst + 4 * q) = make_float4(
                                    acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
                    } else if (V == 2) {
#pragma unroll
                        for (int q = 0; q < kFirSeg / 2; ++q)
                            if (2 * q < left)
                                *reinterpret_cast<float2 *>(dst + 2 * q) = make_float2(acc[2 * q], acc[2 * q + 1]);
                    } else {
#pragma unroll
                        for (int q = 0; q < kFirSeg; ++q)
                            if (q < left) dst[q] = acc[q];
                    }
                }
            }
            if (next_pending) {
                next_pending = false;
                fill_next();
            }
        }
        if (next_pending && !gave_up) fill_next();      // this warp had no segment in this tile
        unit0 = seg - sh.nseg;                          // position of its next segment in the next tile
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + 2 + b);       // done with this tile's buffer
    }
    if (gave_up && lane == 0) atomicExch(status, kStatusFirWaitTimeout);
    cp_async_wait<0>();
}

// Thread-per-output restatement for filters too long for the shared-memory tile.
template <int DIR>
__global__ void __launch_bounds__(256)
fir_long_kernel(float *__restrict__ out, const float *__restrict__ in, const float *__restrict__ filt,
                int64_t rows, int64_t T, int64_t K, float Ts, const int *skip_flag)
{
    if (skip_flag != nullptr && *skip_flag != 0) return;      // the event-driven kernel has this call
    const int64_t n = rows * T;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
        const int64_t r = e / T, t = e - r * T;
        const float *x = in + r * T;
        float acc = 0.0f;
        if (DIR < 0) {
            const int64_t km = K < t + 1 ? K : t + 1;
            for (int64_t i = 0; i < km; ++i) acc = fmaf(x[t - i], filt[i], acc);
        } else {
            const int64_t km = K < T - t ? K : T - t;
            for (int64_t i = 0; i < km; ++i) acc = fmaf(x[t + i], filt[i], acc);
        }
        out[e] = acc * Ts;
    }
}

static inline int pad_stride(int w)       // smallest s >= w with s = 4 (mod 8)
{
    int s = (w + 3) & ~3;
    if ((s & 7) == 0) s += 4;
    return s;
}

// Tile shape for rows of length T and K taps; returns false if the filter is too long to tile.
static bool fir_shape(int64_t rows, int64_t T, int64_t K, FirShape &sh, int max_words = kFirTileWordsPerRow)
{
    sh.halo = (int)(((K + 3) & ~3LL) + 8);     // taps rounded up plus two quads of look-ahead
    const int room = max_words - 4 - sh.halo;                 // words left for outputs (4 = stride padding)
    const int nseg_max = room / kFirSeg;
    if (nseg_max < 1) return false;
    const int64_t segs = ceil_div(T, kFirSeg);
    sh.ttiles = (int)ceil_div(segs, nseg_max);
    // few rows: cut time finer so that every SM gets a tile (the halo is re-read from L2)
    const int64_t row_blocks = ceil_div(rows, kFirRows);
    const int64_t want = 2 * (int64_t)sm_count();
    if (row_blocks * sh.ttiles < want) {
        int64_t tt = ceil_div(want, row_blocks);
        if (tt > segs) tt = segs;
        if (tt > sh.ttiles) sh.ttiles = (int)tt;
    }
    sh.nseg = (int)ceil_div(segs, sh.ttiles);
    sh.ttiles = (int)ceil_div(segs, sh.nseg);
    sh.SX = pad_stride(sh.nseg * kFirSeg + sh.halo);
    // Warps per CTA.  Warp w runs on scheduler w % 4 and takes segments w, w+nw, ...; pick the
    // multiple of four whose busiest scheduler has the least work, preferring 8 warps.
    if (sh.nseg <= 8) {             // one segment per warp
        sh.nwarps = sh.nseg;
        return true;
    }
    int best_load = 1 << 30;
    sh.nwarps = 8;
    const int candidates[4] = {8, 12, 16, 4};
    for (int nw : candidates) {
        int load[4] = {0, 0, 0, 0};
        for (int w = 0; w < nw; ++w) load[w & 3] += (sh.nseg - w + nw - 1) / nw;   // segments of warp w
        int worst = load[0];
        for (int k = 1; k < 4; ++k) worst = load[k] > worst ? load[k] : worst;
        if (worst < best_load) { best_load = worst; sh.nwarps = nw; }
    }
    return true;
}

// Tile shape of the packed kernel (64-row tiles, one CTA per SM); false if the filter is too long.
static bool fir2_shape(int64_t rows, int64_t T, int64_t K, FirShape &sh, int max_samples)
{
    sh.halo = (int)(((K + 3) & ~3LL) + 8);     // taps rounded up plus two quads of look-ahead
    const int room = max_samples - 4 - sh.halo;               // samples left for outputs (4 = stride padding)
    const int nseg_max = room / kFirSeg;
    if (nseg_max < 1) return false;
    const int64_t segs = ceil_div(T, kFirSeg);
    sh.ttiles = (int)ceil_div(segs, nseg_max);
    // few rows: cut time finer so that every SM gets a tile (the halo is re-read from L2)
    const int64_t row_blocks = ceil_div(rows, kFir2Rows);
    const int64_t want = (int64_t)sm_count();
    if (row_blocks * sh.ttiles < want) {
        int64_t tt = ceil_div(want, row_blocks);
        if (tt > segs) tt = segs;
        if (tt > sh.ttiles) sh.ttiles = (int)tt;
    }
    sh.nseg = (int)ceil_div(segs, sh.ttiles);
    sh.ttiles = (int)ceil_div(segs, sh.nseg);
    // words per row pair of the interleaved tile: = 4 (mod 8), so that the 128-bit loads of a
    // quarter warp fall into distinct bank groups
    sh.SX = pad_stride(2 * (sh.nseg * kFirSeg + sh.halo));
    // Warps per CTA: warp w runs on scheduler w % 4 and takes segments w, w+nw, ...; pick the
    // multiple of four whose busiest scheduler has the least work, preferring fewer warps.
    if (sh.nseg <= 8) {
        sh.nwarps = sh.nseg;
        return true;
    }
    int best_load = 1 << 30;
    sh.nwarps = 8;
    const int candidates[3] = {8, 12, 16};
    for (int nw : candidates) {
        int load[4] = {0, 0, 0, 0};
        for (int w = 0; w < nw; ++w) load[w & 3] += (sh.nseg - w + nw - 1) / nw;
        int worst = load[0];
        for (int k = 1; k < 4; ++k) worst = load[k] > worst ? load[k] : worst;
        if (worst < best_load) { best_load = worst; sh.nwarps = nw; }
    }
    return true;
}

static std::atomic<int> g_fir_packed{0};
static std::atomic<int> g_fir_flow{2};
static std::atomic<int> g_fir_skip_zeros{1};
// Below this many input samples the dense kernel takes less than about 0.1 ms and the probe and
// the second launch (about 10 microseconds together) are not worth it.
constexpr int64_t kFirProbeMinElements = 1 << 25;

template <int DIR, bool PK = false>
static int launch_fir2(float *out, const float *in, const float *filt,
                       int64_t rows, int64_t T, int64_t Keff, float Ts, cudaStream_t stream, bool &taken,
                       float spike_value = 0.0f, const int *skip_flag = nullptr)
{
    // Two CTAs per SM with half-size tiles (more warps to keep the FMA pipe busy across barriers,
    // and one CTA's tile copy overlaps the other's arithmetic) where a half-size tile still has
    // room for five segments next to the filter's halo; else one CTA per SM with full-size tiles.
    FirShape sh;
    const int halo = (int)(((Keff + 3) & ~3LL) + 8);
    const int mode = g_fir_packed.load();
    const bool half = mode == 2 ? true : (mode == 3 ? false : (kFir2HalfSamples - 4 - halo) / kFirSeg >= 5);
    taken = (half && fir2_shape(rows, T, Keff, sh, kFir2HalfSamples)) || fir2_shape(rows, T, Keff, sh, kFir2MaxSamples);
    if (!taken) return SLAYER_B200_OK;
    const int64_t ntiles = ceil_div(rows, kFir2Rows) * sh.ttiles;
    const size_t kp = (size_t)((Keff + 3) & ~3LL);
    const size_t wx = (size_t)sh.nseg * kFirSeg + sh.halo;
    const size_t stage_words = (size_t)kFir2Rows * (PK ? (size_t)kFir2StageWords : ((wx + 3) & ~(size_t)3));
    const size_t smem = sizeof(float) * (2 * (kp + 4) + 4 * (kp + 2 * kFirSeg) + 2 * kFir2MaskWords + 4 + stage_words +
                                         (size_t)(kFir2Rows / 2) * sh.SX);
    const int vw = PK ? tile_vec_width(T, {out}) : tile_vec_width(T, {out, in});
    auto kern = vw == 4 ? fir2_kernel<DIR, 4, PK> : (vw == 2 ? fir2_kernel<DIR, 2, PK> : fir2_kernel<DIR, 1, PK>);
    int rc = reserve_dynamic_smem((const void *)kern, smem);
    if (rc) return rc;
    // CTAs per SM: bounded by shared memory and by registers (128 per thread at most)
    int64_t by_smem = (int64_t)(226 * 1024 / (smem + 1024));
    int64_t by_regs = 65536 / (128 * 32 * (int64_t)sh.nwarps);
    int64_t ctas_per_sm = by_smem < by_regs ? by_smem : by_regs;
    if (ctas_per_sm > 8) ctas_per_sm = 8;
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    int64_t grid = ctas_per_sm * (int64_t)sm_count();
    if (grid > ntiles) grid = ntiles;
    kern<<<(unsigned)grid, sh.nwarps * 32, smem, stream>>>(out, in, filt, rows, (int)T, (int)Keff, Ts, sh, ntiles,
                                                           g_fir_skip_zeros.load() != 0, spike_value, skip_flag);
    return check_launch("fir (packed) kernel launch");
}

// The scalar tiled kernels (and, for filters too long to tile, the thread-per-output kernel).
// PK: `in` points to bit-packed spikes; only the flow kernel expands them, so `taken` comes back
// false when the shape or the missing status word rules that kernel out.
template <int DIR, bool PK, bool RHO = false>
static int launch_fir_tiled(float *out, const float *in, const float *filt, int64_t rows, int64_t T, int64_t Keff,
                            float Ts, cudaStream_t stream, const int *skip_flag, float spike_value, bool &taken,
                            FirRho rho = FirRho{nullptr, 0.0f, 1.0f, 0.0f, 1.0f})
{
    constexpr bool kFlowOnly = PK || RHO;           // forms that only the flow kernel has
    taken = true;
    FirShape sh;
    // (packed input: the tiles give up 16 words per row to the two staging slots, so that two
    // CTAs still fit an SM)
    const bool tiled = fir_shape(rows, T, Keff, sh, PK ? kFirTileWordsPerRow - kFirStageWords : kFirTileWordsPerRow);
    const int64_t ntiles = tiled ? ceil_div(rows, kFirRows) * sh.ttiles : 0;
    if (!tiled) {
        if (kFlowOnly) { taken = false; return SLAYER_B200_OK; }
        const int64_t n = rows * T;
        int64_t g = ceil_div(n, 256);
        const int64_t cap = (int64_t)sm_count() * 32;
        if (g > cap) g = cap;
        fir_long_kernel<DIR><<<(unsigned)g, 256, 0, stream>>>(out, in, filt, rows, T, Keff, Ts, skip_flag);
        return check_launch("fir (long filter) kernel launch");
    }
    const int vw = PK ? tile_vec_width(T, {out}) : (RHO ? tile_vec_width(T, {out, in, rho.u}) : tile_vec_width(T, {out, in}));
    // groups of four taps left over after the runs of six: two or more take the form of the
    // kernel that leaves the run where the groups end, and so do the forms with more code around
    // the arithmetic (packed input, surrogate epilogue), which measure 2-3 % faster that way
    // even with one group left over (mode 4 of slayer_b200_set_fir_flow: always)
    const bool rx = ((Keff >> 2) % kFirPhases) >= 2 || kFlowOnly || g_fir_flow.load() == 4;
    // Rows off the 16-byte grid although the arrays are on it (T % 4 != 0): the flow kernel with a
    // per-row offset, so that copies and stores are 16 bytes wide instead of 8 or 4.  Its tiles
    // have to cover up to three samples more, and it always takes the form of the tap loop with the
    // smaller instruction footprint (its fill and store code is the longest).  Measured, 110 taps
    // on 131072 rows: T = 1449 0.93 ms (4-byte accesses: 1.37 ms), against T = 1450 with 8-byte
    // accesses 0.97 ms and T = 1448 0.84 ms; 77 taps on 917504 x 301: 1.09 against 1.82 ms.
    if constexpr (!PK) {
        const int fmode = g_fir_flow.load();
        if (vw < 4 && T >= 8 && (fmode == 2 || fmode == 4 || (kFlowOnly && fmode != 3)) && aligned16(out) && aligned16(in) &&
            (!RHO || aligned16(rho.u))) {
            FirShape sh2;
            int *status2 = device_status_word();
            if (status2 && fir_shape(rows, T + 3, Keff, sh2)) {
                const int64_t ntiles2 = ceil_div(rows, kFirRows) * sh2.ttiles;
                const size_t smem2 = sizeof(float) * (8 + (size_t)((Keff + 3) & ~3LL) + 4 + 2 * (size_t)kFirRows * sh2.SX);
                int64_t per_sm = (int64_t)(220 * 1024 / (smem2 + 1024));
                if (per_sm > 8) per_sm = 8;
                if (per_sm < 1) per_sm = 1;
                int64_t grid2 = per_sm * (int64_t)sm_count();
                if (grid2 > ntiles2) grid2 = ntiles2;
                auto kern2 = sh2.nwarps <= 8 ? fir_flow_kernel<DIR, 4, 1, false, RHO, true, true> : fir_flow_kernel<DIR, 4, 2, false, RHO, true, true>;
                int rc2 = reserve_dynamic_smem((const void *)kern2, smem2);
                if (rc2) return rc2;
                kern2<<<(unsigned)grid2, sh2.nwarps * 32, smem2, stream>>>(out, in, filt, rows, (int)T, (int)Keff, Ts, sh2, ntiles2,
                                                                           status2, skip_flag, spike_value, rho);
                return check_launch("fir (flow, row offsets) kernel launch");
            }
        }
    }
    const size_t smem = sizeof(float) * (8 + (size_t)((Keff + 3) & ~3LL) + 4 + 2 * (size_t)kFirRows * sh.SX +
                                         (PK ? 2 * (size_t)kFirRows * kFirStageWords : 0));
    int64_t ctas_per_sm = (int64_t)(220 * 1024 / (smem + 1024));      // 2 for full-size tiles
    if (ctas_per_sm > 8) ctas_per_sm = 8;
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    int64_t grid = ctas_per_sm * (int64_t)sm_count();
    if (grid > ntiles) grid = ntiles;
    int *status = (kFlowOnly || g_fir_flow.load() != 0) ? device_status_word() : nullptr;
    if (status) {
        const bool roomy = (kFlowOnly || g_fir_flow.load() >= 2) && sh.nwarps <= 8;
        auto pick = [&](auto rxc) {
            constexpr bool RXV = decltype(rxc)::value;
            return roomy ? (vw == 4 ? fir_flow_kernel<DIR, 4, 1, PK, RHO, false, RXV>
                                    : (vw == 2 ? fir_flow_kernel<DIR, 2, 1, PK, RHO, false, RXV> : fir_flow_kernel<DIR, 1, 1, PK, RHO, false, RXV>))
                         : (vw == 4 ? fir_flow_kernel<DIR, 4, 2, PK, RHO, false, RXV>
                                    : (vw == 2 ? fir_flow_kernel<DIR, 2, 2, PK, RHO, false, RXV> : fir_flow_kernel<DIR, 1, 2, PK, RHO, false, RXV>));
        };
        auto kern = rx ? pick(std::true_type{}) : pick(std::false_type{});
        int rc = reserve_dynamic_smem((const void *)kern, smem);
        if (rc) return rc;
        kern<<<(unsigned)grid, sh.nwarps * 32, smem, stream>>>(out, in, filt, rows, (int)T, (int)Keff, Ts, sh, ntiles, status, skip_flag,
                                                               spike_value, rho);
        return check_launch("fir (flow) kernel launch");
    }
    if constexpr (kFlowOnly) {
        taken = false;
        return SLAYER_B200_OK;
    } else {
        auto kern = vw == 4 ? fir_kernel<DIR, 4> : (vw == 2 ? fir_kernel<DIR, 2> : fir_kernel<DIR, 1>);
        int rc = reserve_dynamic_smem((const void *)kern, smem);
        if (rc) return rc;
        kern<<<(unsigned)grid, sh.nwarps * 32, smem, stream>>>(out, in, filt, rows, (int)T, (int)Keff, Ts, sh, ntiles, skip_flag);
        return check_launch("fir kernel launch");
    }
}

template <int DIR>
static int launch_fir(float *out, const float *in, const float *filt,
                      int64_t rows, int64_t T, int64_t K, float Ts, cudaStream_t stream)
{
    if (rows == 0 || T == 0) return SLAYER_B200_OK;
    if (K == 0) {
        cudaError_t e = cudaMemsetAsync(out, 0, (size_t)rows * T * sizeof(float), stream);
        if (e != cudaSuccess) { set_error("fir: memset failed: %s", cudaGetErrorString(e)); return SLAYER_B200_ECUDA; }
        return SLAYER_B200_OK;
    }
    const int64_t Keff = K < T ? K : T;              // taps beyond the row length never contribute
    // Mostly-zero inputs (spike tensors) of some size: the event-driven kernel.  Mode 2 takes it
    // unconditionally; mode 1 lets a probe on the device decide between it and the dense kernel
    // (both are enqueued; the one ruled out returns at once).
    const int *skip_flag = nullptr;
    const int zmode = g_fir_skip_zeros.load();
    if (zmode != 0 && fir_sparse_eligible(rows, T, Keff)) {
        if (zmode == 2) return fir_sparse_launch(DIR, false, out, in, filt, rows, T, Keff, Ts, 0.0f, nullptr, stream);
        // (corr runs in the backward pass, on gradients, which are dense: it is not probed)
        if (DIR < 0 && rows * T >= kFirProbeMinElements) {
            int rc = fir_sparse_probe(in, rows, T, false, filt, Keff, stream, &skip_flag);
            if (rc) return rc;
            if (skip_flag) {
                rc = fir_sparse_launch(DIR, false, out, in, filt, rows, T, Keff, Ts, 0.0f, skip_flag, stream);
                if (rc) return rc;
            }
        }
    }
    if (g_fir_packed.load() != 0) {
        bool taken = false;
        const int rc = launch_fir2<DIR>(out, in, filt, rows, T, Keff, Ts, stream, taken, 0.0f, skip_flag);
        if (taken) return rc;
    }
    bool taken = false;
    return launch_fir_tiled<DIR, false>(out, in, filt, rows, T, Keff, Ts, stream, skip_flag, 0.0f, taken);
}

static int check_fir_args(const char *name, float *out, const float *in, const float *filt,
                          int64_t rows, int64_t T, int64_t K)
{
    SB200_REQUIRE(rows >= 0 && T >= 0 && K >= 0, "%s: negative size", name);
    SB200_REQUIRE(T < (1LL << 31) - 4096, "%s: T=%lld too large", name, (long long)T);
    SB200_REQUIRE(rows == 0 || T == 0 || (out && in && (filt || K == 0)), "%s: null pointer", name);
    SB200_REQUIRE(out != in || rows == 0 || T == 0, "%s: out must not alias in", name);
    return SLAYER_B200_OK;
}

}  // namespace sb200

extern "C" int slayer_b200_set_fir_packed(int enable)
{
    return sb200::g_fir_packed.exchange(enable < 0 ? 0 : (enable > 3 ? 1 : enable));
}

extern "C" int slayer_b200_set_fir_flow(int mode)
{
    return sb200::g_fir_flow.exchange(mode < 0 || mode > 4 ? 1 : mode);
}

extern "C" int slayer_b200_set_fir_skip_zeros(int mode)
{
    return sb200::g_fir_skip_zeros.exchange(mode < 0 || mode > 2 ? 1 : mode);
}

extern "C" int slayer_b200_conv(float *out, const float *in, const float *filter,
                                int64_t rows, int64_t T, int64_t K, float Ts, void *stream)
{
    using namespace sb200;
    clear_error();
    int rc = check_fir_args("conv", out, in, filter, rows, T, K);
    if (rc) return rc;
    return launch_fir<-1>(out, in, filter, rows, T, K, Ts, (cudaStream_t)stream);
}

extern "C" int slayer_b200_conv_packed(float *out, const uint32_t *bits, const float *filter,
                                       int64_t rows, int64_t T, int64_t K, float spike_value, float Ts, void *stream)
{
    using namespace sb200;
    clear_error();
    int rc = check_fir_args("conv_packed", out, reinterpret_cast<const float *>(bits), filter, rows, T, K);
    if (rc) return rc;
    SB200_REQUIRE((reinterpret_cast<uintptr_t>(bits) & 3u) == 0, "conv_packed: bits must be 4-byte aligned");
    if (rows == 0 || T == 0) return SLAYER_B200_OK;
    if (K == 0) {
        cudaError_t e = cudaMemsetAsync(out, 0, (size_t)rows * T * sizeof(float), (cudaStream_t)stream);
        if (e != cudaSuccess) { set_error("conv_packed: memset failed: %s", cudaGetErrorString(e)); return SLAYER_B200_ECUDA; }
        return SLAYER_B200_OK;
    }
    const int64_t Keff = K < T ? K : T;
    const int *skip_flag = nullptr;
    const int zmode = g_fir_skip_zeros.load();
    FirShape probe_shape;
    const bool dense_ok = fir_shape(rows, T, Keff, probe_shape, kFirTileWordsPerRow - kFirStageWords) ||
                          fir2_shape(rows, T, Keff, probe_shape, kFir2MaxSamples);
    if (zmode != 0 && fir_sparse_eligible(rows, T, Keff) && fabsf(spike_value) <= FLT_MAX) {
        // (filters too long for the tiled kernel: the event-driven one, whatever the density)
        if (zmode == 2 || !dense_ok) return fir_sparse_launch(-1, true, out, bits, filter, rows, T, Keff, Ts, spike_value, nullptr, (cudaStream_t)stream);
        if (rows * T >= kFirProbeMinElements) {
            rc = fir_sparse_probe(bits, rows, T, true, filter, Keff, (cudaStream_t)stream, &skip_flag);
            if (rc) return rc;
            if (skip_flag) {
                rc = fir_sparse_launch(-1, true, out, bits, filter, rows, T, Keff, Ts, spike_value, skip_flag, (cudaStream_t)stream);
                if (rc) return rc;
            }
        }
    }
    // dense input: the scalar kernel expanding the bits as it fills its tiles; the packed two-row
    // kernel only where slayer_b200_set_fir_packed asks for it or the scalar one cannot take the shape
    bool taken = false;
    if (g_fir_packed.load() == 0) {
        rc = launch_fir_tiled<-1, true>(out, reinterpret_cast<const float *>(bits), filter, rows, T, Keff, Ts,
                                        (cudaStream_t)stream, skip_flag, spike_value, taken);
        if (taken) return rc;
    }
    rc = launch_fir2<-1, true>(out, reinterpret_cast<const float *>(bits), filter, rows, T, Keff, Ts,
                               (cudaStream_t)stream, taken, spike_value, skip_flag);
    if (!taken) {
        set_error("conv_packed: a filter of %lld taps is too long for the tiled kernel; unpack the spikes and call "
                  "slayer_b200_conv", (long long)K);
        return SLAYER_B200_EUNSUPPORTED;
    }
    return rc;
}

extern "C" int slayer_b200_corr(float *out, const float *in, const float *filter,
                                int64_t rows, int64_t T, int64_t K, float Ts, void *stream)
{
    using namespace sb200;
    clear_error();
    int rc = check_fir_args("corr", out, in, filter, rows, T, K);
    if (rc) return rc;
    return launch_fir<1>(out, in, filter, rows, T, K, Ts, (cudaStream_t)stream);
}

extern "C" int slayer_b200_corr_spike_grad(float *out, const float *in, const float *filter, const float *u,
                                           int64_t rows, int64_t T, int64_t K, float Ts,
                                           float theta, float tau, float scale, void *stream)
{
    using namespace sb200;
    clear_error();
    int rc = check_fir_args("corr_spike_grad", out, in, filter, rows, T, K);
    if (rc) return rc;
    SB200_REQUIRE(rows == 0 || T == 0 || u != nullptr, "corr_spike_grad: null pointer");
    SB200_REQUIRE(out != u || rows == 0 || T == 0, "corr_spike_grad: out must not alias u");
    if (rows == 0 || T == 0) return SLAYER_B200_OK;
    // (the epilogue divides by tau through its reciprocal, which wants a tau well inside the
    // normal range; any other tau takes the two passes)
    if (K > 0 && tau >= 0x1p-60f && tau <= 0x1p60f) {
        bool taken = false;
        rc = launch_fir_tiled<1, false, true>(out, in, filter, rows, T, K < T ? K : T, Ts, (cudaStream_t)stream, nullptr, 0.0f,
                                              taken, FirRho{u, theta, tau, scale / tau, 1.0f / tau});
        if (taken) return rc;
    }
    // shapes the tiled kernel does not take (and the empty filter): the two passes, the second in place
    rc = launch_fir<1>(out, in, filter, rows, T, K, Ts, (cudaStream_t)stream);
    if (rc) return rc;
    return slayer_b200_spike_grad(out, out, u, rows * T, theta, tau, scale, stream);
}
