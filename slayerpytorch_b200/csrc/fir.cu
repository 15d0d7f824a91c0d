// Temporal FIR filter along the last axis and its adjoint:
//   conv: out[r,t] = Ts * sum_{i<K, t-i>=0} in[r,t-i] * f[i]      (psp, forward)
//   corr: out[r,t] = Ts * sum_{i<K, t+i<T}  in[r,t+i] * f[i]      (psp, backward)
// Each output is one fp32 fused-multiply-add chain over the taps in ascending order starting
// from +0, scaled by Ts once at the end — the same sequence of roundings as a thread-per-
// output loop, so results are reproducible bit for bit whatever the tiling.  Samples outside
// the row enter the chain as +0, which leaves the accumulator unchanged for finite taps.
//
// Cost: 8 algorithmic bytes and 2K flops per element.  For K above ~47 taps the fp32 FMA
// pipes, not HBM, bound the kernel, so the design goal is one FMA per issue slot:
//   - a CTA stages a [32 rows x (Tt + halo)] input tile in shared memory once;
//   - lane l of every warp owns row l, a warp owns 8-sample time segments, and a thread
//     keeps 8 accumulators plus a 12-sample sliding input window in registers;
//   - per group of 4 taps a thread issues 32 FMAs, one 128-bit load of new window samples and
//     one 128-bit broadcast load of taps; the window rotates through three register banks by
//     unrolling, so no moves are spent on it.
// The row stride of the tile is = 4 (mod 8) words, which makes the per-row 128-bit loads of a
// warp conflict free.  Results leave through a second tile so that global stores are
// contiguous row segments.
#include "common.cuh"
#include "tile.cuh"

namespace sb200 {

constexpr int kFirRows = 32;        // rows per CTA (= lanes)
constexpr int kFirWarps = 8;
constexpr int kFirSeg = 8;          // outputs per thread per pass
constexpr int kFirPassLen = kFirWarps * kFirSeg;   // 64 outputs of a row per pass

__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }

// acc[m] += sum_{ii<4} win[m + base(ii)] * f[ii], ascending ii.  win = lo|mid|hi (12 samples).
// DIR < 0 (conv): sample for (m, ii) is win[m + 4 - ii];  DIR > 0 (corr): win[m + ii].
template <int DIR, int NT>
__device__ __forceinline__ void fir_group(float (&acc)[kFirSeg], const float4 &lo, const float4 &mid,
                                          const float4 &hi, const float4 &f)
{
    const float win[12] = {lo.x, lo.y, lo.z, lo.w, mid.x, mid.y, mid.z, mid.w, hi.x, hi.y, hi.z, hi.w};
    const float fv[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
    for (int ii = 0; ii < NT; ++ii) {
#pragma unroll
        for (int m = 0; m < kFirSeg; ++m)
            acc[m] = fmaf(win[DIR < 0 ? m + 4 - ii : m + ii], fv[ii], acc[m]);
    }
}

template <int DIR>
__device__ __forceinline__ void fir_group_n(float (&acc)[kFirSeg], const float4 &lo, const float4 &mid,
                                            const float4 &hi, const float4 &f, int ntaps)
{
    switch (ntaps) {
        case 1: fir_group<DIR, 1>(acc, lo, mid, hi, f); break;
        case 2: fir_group<DIR, 2>(acc, lo, mid, hi, f); break;
        case 3: fir_group<DIR, 3>(acc, lo, mid, hi, f); break;
        default: fir_group<DIR, 4>(acc, lo, mid, hi, f); break;
    }
}

// DIR = -1: conv, DIR = +1: corr.  V: global access width in floats (4, 2 or 1; T % V == 0
// and bases aligned to 4*V bytes).
template <int DIR, int V>
__global__ void __launch_bounds__(kFirWarps * 32)
fir_kernel(float *__restrict__ out, const float *__restrict__ in, const float *__restrict__ filt,
           int64_t rows, int T, int K, float Ts, int passes, int halo, int SX, int SY, int ttiles)
{
    extern __shared__ __align__(16) float smem[];
    const int Tt = passes * kFirPassLen;
    const int WX = Tt + halo;
    const int KP = (K + 3) & ~3;
    float *fs = smem;                        // KP taps
    float *xs = fs + KP;                     // kFirRows x SX
    float *ys = xs + kFirRows * SX;          // kFirRows x SY

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t rb = blockIdx.x / ttiles;
    const int tt = blockIdx.x - (int)(rb * ttiles);
    const int64_t row0 = rb * kFirRows;
    const int t0 = tt * Tt;
    const int64_t nrow = rows - row0;
    // global time of tile-local input position 0
    const int g0 = DIR < 0 ? t0 - halo : t0;

    for (int i = threadIdx.x; i < KP; i += blockDim.x) fs[i] = i < K ? filt[i] : 0.0f;

    // stage the input tile with asynchronous copies (all in flight together): warp w fills rows
    // w, w+8, w+16, w+24 from contiguous global segments; samples outside the row become zeros
#pragma unroll
    for (int rr = 0; rr < kFirRows / kFirWarps; ++rr) {
        const int r = warp + rr * kFirWarps;
        const bool row_ok = r < nrow;
        const float *src = in + (row0 + (row_ok ? r : 0)) * (int64_t)T;
        float *dst = xs + r * SX;
        for (int p = lane * V; p < WX; p += 32 * V) {
            const int gt = g0 + p;
            const bool ok = row_ok && gt >= 0 && gt < T;
            cp_async<4 * V>(dst + p, ok ? src + gt : in, ok);
        }
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    const float *xrow = xs + lane * SX + (DIR < 0 ? halo : 0);   // tile-local position 0
    float *yrow = ys + lane * SY;
    const int groups = K >> 2;          // full groups of 4 taps
    const int tail = K & 3;

    for (int pass = 0; pass < passes; ++pass) {
        const int tb = (pass * kFirWarps + warp) * kFirSeg;
        if (t0 + tb >= T) break;        // whole segment beyond the row end (warp-uniform)
        float acc[kFirSeg];
#pragma unroll
        for (int m = 0; m < kFirSeg; ++m) acc[m] = 0.0f;

        // window banks; conv slides toward lower positions, corr toward higher ones
        float4 A, B, C;
        const float *xp;                // next sample quad to fetch
        if (DIR < 0) {
            A = ld4(xrow + tb - 4); B = ld4(xrow + tb); C = ld4(xrow + tb + 4);
            xp = xrow + tb - 8;
        } else {
            A = ld4(xrow + tb); B = ld4(xrow + tb + 4); C = ld4(xrow + tb + 8);
            xp = xrow + tb + 12;
        }
        const float *fp = fs;
        int g = 0;
        if (DIR < 0) {
            for (; g + 3 <= groups; g += 3) {
                fir_group<DIR, 4>(acc, A, B, C, ld4(fp));     C = ld4(xp);
                fir_group<DIR, 4>(acc, C, A, B, ld4(fp + 4)); B = ld4(xp - 4);
                fir_group<DIR, 4>(acc, B, C, A, ld4(fp + 8)); A = ld4(xp - 8);
                xp -= 12; fp += 12;
            }
            for (; g < groups; ++g) {
                fir_group<DIR, 4>(acc, A, B, C, ld4(fp));
                C = B; B = A; A = ld4(xp);
                xp -= 4; fp += 4;
            }
            if (tail) fir_group_n<DIR>(acc, A, B, C, ld4(fp), tail);
        } else {
            for (; g + 3 <= groups; g += 3) {
                fir_group<DIR, 4>(acc, A, B, C, ld4(fp));     A = ld4(xp);
                fir_group<DIR, 4>(acc, B, C, A, ld4(fp + 4)); B = ld4(xp + 4);
                fir_group<DIR, 4>(acc, C, A, B, ld4(fp + 8)); C = ld4(xp + 8);
                xp += 12; fp += 12;
            }
            for (; g < groups; ++g) {
                fir_group<DIR, 4>(acc, A, B, C, ld4(fp));
                A = B; B = C; C = ld4(xp);
                xp += 4; fp += 4;
            }
            if (tail) fir_group_n<DIR>(acc, A, B, C, ld4(fp), tail);
        }
        *reinterpret_cast<float4 *>(yrow + tb) =
            make_float4(acc[0] * Ts, acc[1] * Ts, acc[2] * Ts, acc[3] * Ts);
        *reinterpret_cast<float4 *>(yrow + tb + 4) =
            make_float4(acc[4] * Ts, acc[5] * Ts, acc[6] * Ts, acc[7] * Ts);
    }
    __syncthreads();

    // drain the result tile: contiguous row segments
    const int tvalid = min(Tt, T - t0);
#pragma unroll
    for (int rr = 0; rr < kFirRows / kFirWarps; ++rr) {
        const int r = warp + rr * kFirWarps;
        if (r >= nrow) continue;
        float *dst = out + (row0 + r) * (int64_t)T + t0;
        const float *src = ys + r * SY;
        typedef typename vec_t<V>::type vec;
        for (int p = lane * V; p < tvalid; p += 32 * V)
            *reinterpret_cast<vec *>(dst + p) = *reinterpret_cast<const vec *>(src + p);
    }
}

// Thread-per-output restatement for filters too long for the shared-memory tile.
template <int DIR>
__global__ void __launch_bounds__(256)
fir_long_kernel(float *__restrict__ out, const float *__restrict__ in, const float *__restrict__ filt,
                int64_t rows, int64_t T, int64_t K, float Ts)
{
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
    const int halo = (int)(((Keff + 3) & ~3LL) + 4);
    // choose the number of 64-sample passes per tile: least padding, then fewest tiles
    int best_p = 0;
    int64_t best_cover = 0;
    const size_t smem_cap = 100 * 1024;              // two CTAs per SM
    for (int p = 8; p >= 1; --p) {
        const int Tt = p * kFirPassLen;
        const size_t bytes = sizeof(float) * ((size_t)((Keff + 3) & ~3LL) +
                             (size_t)kFirRows * (pad_stride(Tt + halo) + pad_stride(Tt)));
        if (bytes > smem_cap && p > 1) continue;
        const int64_t cover = ceil_div(T, Tt) * Tt;
        if (best_p == 0 || cover < best_cover) { best_p = p; best_cover = cover; }
    }
    const int Tt = best_p * kFirPassLen;
    const int SX = pad_stride(Tt + halo), SY = pad_stride(Tt);
    const size_t smem = sizeof(float) * ((size_t)((Keff + 3) & ~3LL) + (size_t)kFirRows * (SX + SY));
    const int64_t ttiles = ceil_div(T, Tt);
    const int64_t blocks = ceil_div(rows, kFirRows) * ttiles;
    if (smem > 220 * 1024 || blocks > 0x7fffffffLL) {
        const int64_t n = rows * T;
        int64_t g = ceil_div(n, 256);
        const int64_t cap = (int64_t)sm_count() * 32;
        if (g > cap) g = cap;
        fir_long_kernel<DIR><<<(unsigned)g, 256, 0, stream>>>(out, in, filt, rows, T, Keff, Ts);
        return check_launch("fir (long filter) kernel launch");
    }
    const int vw = tile_vec_width(T, {out, in});
    auto kern = vw == 4 ? fir_kernel<DIR, 4> : (vw == 2 ? fir_kernel<DIR, 2> : fir_kernel<DIR, 1>);
    int rc = reserve_dynamic_smem((const void *)kern, smem);
    if (rc) return rc;
    kern<<<(unsigned)blocks, kFirWarps * 32, smem, stream>>>(
        out, in, filt, rows, (int)T, (int)Keff, Ts, best_p, halo, SX, SY, (int)ttiles);
    return check_launch("fir kernel launch");
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

extern "C" int slayer_b200_conv(float *out, const float *in, const float *filter,
                                int64_t rows, int64_t T, int64_t K, float Ts, void *stream)
{
    using namespace sb200;
    clear_error();
    int rc = check_fir_args("conv", out, in, filter, rows, T, K);
    if (rc) return rc;
    return launch_fir<-1>(out, in, filter, rows, T, K, Ts, (cudaStream_t)stream);
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
