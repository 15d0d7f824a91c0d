// Axonal-delay time shift: out[r,t] = in[r,t-d_r], zero filled, d_r = trunc(shift_r / Ts).
//
// Pure data movement, bound by HBM bandwidth (8 algorithmic bytes per element).  One launch
// covers every row of the batch; the per-neuron table is indexed by row % nNeurons.
//
// Work split: a group of LPR lanes (a power of two, up to a full warp) owns one row and
// strides along time, so every global access of a group is contiguous.  When both buffers are
// 16-byte aligned the row is walked in aligned 16-byte quads: a quad is one aligned 128-bit
// store assembled from the two aligned source quads that straddle its source.  With T % 4 == 0
// a quad is either wholly inside its row or wholly outside, so zero fill stays exact; for any
// other row length the few quads at the ends of a row (or whose source crosses an end) go
// sample by sample and no neighbouring row is touched.
//
// The same kernels also serve the fused backward step of "spike then delay": with RHO they
// multiply every shifted gradient sample by the surrogate gradient of the spike function at
// the membrane potential of the output position, out = shift(g) * rho(u), in the one pass
// (12 bytes per element instead of 8 + 12 for the two separate passes).
#include "common.cuh"

namespace sb200 {

struct RhoArgs {
    const float *u;             // membrane potential, same shape as the output
    float theta, tau, c;        // c = scale / tau
};

template <bool RHO>
__device__ __forceinline__ float4 rho4(float4 r, const RhoArgs &ra, int64_t quad)
{
    if (RHO) {
        const float4 uv = __ldg(reinterpret_cast<const float4 *>(ra.u) + quad);
        r.x = rho_times(r.x, uv.x, ra.theta, ra.tau, ra.c);
        r.y = rho_times(r.y, uv.y, ra.theta, ra.tau, ra.c);
        r.z = rho_times(r.z, uv.z, ra.theta, ra.tau, ra.c);
        r.w = rho_times(r.w, uv.w, ra.theta, ra.tau, ra.c);
    }
    return r;
}

template <bool RHO>
__device__ __forceinline__ float rho1(float r, const RhoArgs &ra, int64_t e)
{
    return RHO ? rho_times(r, __ldg(ra.u + e), ra.theta, ra.tau, ra.c) : r;
}

// Row length a multiple of four: every aligned quad of the flat array lies inside one row.
template <bool LUT, bool RHO>
__global__ void __launch_bounds__(256)
shift_vec4_kernel(float4 *__restrict__ out, const float4 *__restrict__ in,
                  const float *__restrict__ lut, float shift, float Ts,
                  int64_t rows, int T4, int64_t nNeurons, int lpr_log2, RhoArgs ra)
{
    const int lpr = 1 << lpr_log2;
    const int lane_in_row = threadIdx.x & (lpr - 1);
    const int64_t groups_per_block = blockDim.x >> lpr_log2;
    const int64_t group0 = (int64_t)blockIdx.x * groups_per_block + (threadIdx.x >> lpr_log2);
    const int64_t group_stride = (int64_t)gridDim.x * groups_per_block;
    const int T = T4 * 4;

    for (int64_t row = group0; row < rows; row += group_stride) {
        const float sv = LUT ? __ldg(lut + (row % nNeurons)) : shift;
        const int d = shift_steps(sv, Ts);
        const float4 *src = in + row * T4;
        float4 *dst = out + row * T4;
        if (d >= T || d <= -T) {
            for (int q = lane_in_row; q < T4; q += lpr)
                dst[q] = rho4<RHO>(make_float4(0.f, 0.f, 0.f, 0.f), ra, row * T4 + q);
            continue;
        }
        // source element index of output element 4q is 4q - d = 4*(q + a) + o, o in [0,3]
        const int a = (-d) >> 2;          // arithmetic shift = floor division
        const int o = (-d) & 3;
#pragma unroll 2
        for (int q = lane_in_row; q < T4; q += lpr) {
            const int q0 = q + a;
            float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
            if (q0 >= 0 && q0 < T4) v0 = __ldg(src + q0);
            if (o != 0 && q0 + 1 >= 0 && q0 + 1 < T4) v1 = __ldg(src + q0 + 1);
            float4 r;
            switch (o) {
                case 0:  r = v0; break;
                case 1:  r = make_float4(v0.y, v0.z, v0.w, v1.x); break;
                case 2:  r = make_float4(v0.z, v0.w, v1.x, v1.y); break;
                default: r = make_float4(v0.w, v1.x, v1.y, v1.z); break;
            }
            dst[q] = rho4<RHO>(r, ra, row * T4 + q);
        }
    }
}

// Fused shift + surrogate gradient for T % 4 == 0 (16-byte aligned buffers).  Unlike the plain
// shift, this pass spends real arithmetic per sample (an exponential), so lanes must not idle
// at row ends: a CTA takes a block of consecutive rows and its threads stride over all quads
// of the block, (row, quad) advanced incrementally; the rows' shifts are worked out once per
// CTA in shared memory.
constexpr int kRhoRowsMax = 64;

template <bool LUT, bool RHO>
__global__ void __launch_bounds__(256)
spike_grad_shift_rows_kernel(float4 *__restrict__ out, const float4 *__restrict__ in, const float4 *__restrict__ u,
                             const float *__restrict__ lut, float shift, float Ts,
                             int64_t rows, int T4, int64_t nNeurons, int rows_per_block,
                             float theta, float tau, float c)
{
    __shared__ int sd[kRhoRowsMax];
    const int T = T4 * 4;
    const int step_r = (int)blockDim.x / T4, step_q = (int)blockDim.x % T4;
    for (int64_t r0 = (int64_t)blockIdx.x * rows_per_block; r0 < rows; r0 += (int64_t)gridDim.x * rows_per_block) {
        const int nr = (int)(rows - r0 < rows_per_block ? rows - r0 : rows_per_block);
        __syncthreads();                       // the previous block of rows is done with sd
        if ((int)threadIdx.x < nr)
            sd[threadIdx.x] = shift_steps(LUT ? __ldg(lut + ((r0 + threadIdx.x) % nNeurons)) : shift, Ts);
        __syncthreads();
        int r = (int)threadIdx.x / T4, q = (int)threadIdx.x % T4;
        while (r < nr) {
            const int d = sd[r];
            const int64_t base = (r0 + r) * (int64_t)T4;
            float4 uv = make_float4(0.f, 0.f, 0.f, 0.f);
            if (RHO) uv = __ldg(u + base + q);
            float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
            if (d < T && d > -T) {
                // source element index of output element 4q is 4q - d = 4*(q + a) + o, o in [0,3]
                const int a = (-d) >> 2, o = (-d) & 3;
                const int q0 = q + a;
                float4 v0 = g, v1 = g;
                if (q0 >= 0 && q0 < T4) v0 = __ldg(in + base + q0);
                if (o != 0 && q0 + 1 >= 0 && q0 + 1 < T4) v1 = __ldg(in + base + q0 + 1);
                switch (o) {
                    case 0:  g = v0; break;
                    case 1:  g = make_float4(v0.y, v0.z, v0.w, v1.x); break;
                    case 2:  g = make_float4(v0.z, v0.w, v1.x, v1.y); break;
                    default: g = make_float4(v0.w, v1.x, v1.y, v1.z); break;
                }
            }
            if (RHO)
                g = make_float4(rho_times(g.x, uv.x, theta, tau, c), rho_times(g.y, uv.y, theta, tau, c),
                                rho_times(g.z, uv.z, theta, tau, c), rho_times(g.w, uv.w, theta, tau, c));
            out[base + q] = g;
            r += step_r;
            q += step_q;
            if (q >= T4) { q -= T4; ++r; }
        }
    }
}

// The same fused pass for rows of any length (16-byte aligned buffers, T % 4 != 0): rows start
// anywhere in a 16-byte quad, so a CTA takes a block of rows whose first element is quad aligned
// (rows_per_block is a multiple of 4 / gcd(T, 4)) and its threads stride over the aligned quads
// of that contiguous range, (row, time) advanced incrementally.  A quad inside one row whose
// source samples lie inside the same row is assembled from two aligned source quads; the few
// quads that straddle a row end, or whose source does, go sample by sample.
template <bool LUT>
__global__ void __launch_bounds__(256)
spike_grad_shift_flat_rows_kernel(float *__restrict__ out, const float *__restrict__ in, const float *__restrict__ u,
                                  const float *__restrict__ lut, float shift, float Ts,
                                  int64_t rows, int T, int64_t nNeurons, int rows_per_block,
                                  float theta, float tau, float c)
{
    __shared__ int sd[kRhoRowsMax];
    const int64_t total = rows * (int64_t)T;
    const int step_e = 4 * (int)blockDim.x;                 // elements a thread advances per iteration
    const int step_r = step_e / T, step_t = step_e % T;
    for (int64_t r0 = (int64_t)blockIdx.x * rows_per_block; r0 < rows; r0 += (int64_t)gridDim.x * rows_per_block) {
        const int nr = (int)(rows - r0 < rows_per_block ? rows - r0 : rows_per_block);
        __syncthreads();                       // the previous block of rows is done with sd
        if ((int)threadIdx.x < nr)
            sd[threadIdx.x] = shift_steps(LUT ? __ldg(lut + ((r0 + threadIdx.x) % nNeurons)) : shift, Ts);
        __syncthreads();
        const int64_t base = r0 * (int64_t)T;               // multiple of 4: the block starts on a quad
        const int n_el = nr * T;                            // elements of the block (the last block may end inside a quad)
        int e = 4 * (int)threadIdx.x;                       // element offset of this thread's quad inside the block
        int r = e / T, t = e - r * T;
        for (; e < n_el; e += step_e) {
            const int d = sd[r < nr ? r : nr - 1];
            const int64_t src = base + e - d;               // flat index of the first source sample
            const bool whole = e + 4 <= n_el;               // false only for the ragged end of the array
            // u and out are element for element the same quad, whatever the rows do
            float4 uv = make_float4(0.f, 0.f, 0.f, 0.f);
            if (whole) uv = __ldg(reinterpret_cast<const float4 *>(u + base + e));
            float4 g;
            if (t + 4 <= T && t - d >= 0 && t - d + 4 <= T && (src & ~3LL) + 8 <= total) {
                // whole quad inside row r, fed from inside row r: two aligned source quads
                const float4 *in4 = reinterpret_cast<const float4 *>(in);
                const int64_t a = src >> 2;
                const int o = (int)(src & 3);
                const float4 v0 = __ldg(in4 + a);
                g = v0;
                if (o != 0) {
                    const float4 v1 = __ldg(in4 + a + 1);
                    if (o == 1) g = make_float4(v0.y, v0.z, v0.w, v1.x);
                    else if (o == 2) g = make_float4(v0.z, v0.w, v1.x, v1.y);
                    else g = make_float4(v0.w, v1.x, v1.y, v1.z);
                }
            } else {
                // a quad that straddles a row end, or whose source does: four independent loads
                float ge[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    int rk = r, tk = t + k;
                    while (tk >= T) { tk -= T; ++rk; }
                    const bool in_block = e + k < n_el;
                    const int ts = tk - sd[in_block ? rk : 0];
                    ge[k] = (in_block && ts >= 0 && ts < T) ? __ldg(in + base + (int64_t)rk * T + ts) : 0.0f;
                }
                g = make_float4(ge[0], ge[1], ge[2], ge[3]);
            }
            if (whole) {
                *reinterpret_cast<float4 *>(out + base + e) =
                    make_float4(rho_times(g.x, uv.x, theta, tau, c), rho_times(g.y, uv.y, theta, tau, c),
                                rho_times(g.z, uv.z, theta, tau, c), rho_times(g.w, uv.w, theta, tau, c));
            } else {
                const float ge[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (e + k < n_el) out[base + e + k] = rho_times(ge[k], __ldg(u + base + e + k), theta, tau, c);
            }
            r += step_r;
            t += step_t;
            if (t >= T) { t -= T; ++r; }
        }
    }
}

// Any row length (16-byte aligned buffers): rows start anywhere in a quad.
template <bool LUT, bool RHO>
__global__ void __launch_bounds__(256)
shift_flat4_kernel(float *__restrict__ out, const float *__restrict__ in,
                  const float *__restrict__ lut, float shift, float Ts,
                  int64_t rows, int T, int64_t nNeurons, int lpr_log2, RhoArgs ra)
{
    const int lpr = 1 << lpr_log2;
    const int lane_in_row = threadIdx.x & (lpr - 1);
    const int64_t groups_per_block = blockDim.x >> lpr_log2;
    const int64_t group0 = (int64_t)blockIdx.x * groups_per_block + (threadIdx.x >> lpr_log2);
    const int64_t group_stride = (int64_t)gridDim.x * groups_per_block;
    const int64_t total = rows * (int64_t)T;
    const float4 *in4 = reinterpret_cast<const float4 *>(in);
    float4 *out4 = reinterpret_cast<float4 *>(out);

    for (int64_t row = group0; row < rows; row += group_stride) {
        const float sv = LUT ? __ldg(lut + (row % nNeurons)) : shift;
        const int d = shift_steps(sv, Ts);
        const int64_t S = row * (int64_t)T, E = S + T;        // the row as a range of the flat array
        const bool all_zero = d >= T || d <= -T;
        // aligned 16-byte quads of the flat array that touch the row
        for (int64_t q = (S >> 2) + lane_in_row; q < ((E + 3) >> 2); q += lpr) {
            const int64_t F = q << 2;
            const int64_t src = F - d;                            // flat index of the first source sample
            if (F >= S && F + 4 <= E && all_zero) {
                out4[q] = rho4<RHO>(make_float4(0.f, 0.f, 0.f, 0.f), ra, q);
            } else if (F >= S && F + 4 <= E && src >= S && src + 4 <= E && (src & ~3LL) + 8 <= total) {
                // whole quad inside the row and fed from inside the row: two aligned source quads
                const int64_t a = src >> 2;
                const int o = (int)(src & 3);
                const float4 v0 = __ldg(in4 + a);
                float4 r = v0;
                if (o != 0) {
                    const float4 v1 = __ldg(in4 + a + 1);
                    if (o == 1) r = make_float4(v0.y, v0.z, v0.w, v1.x);
                    else if (o == 2) r = make_float4(v0.z, v0.w, v1.x, v1.y);
                    else r = make_float4(v0.w, v1.x, v1.y, v1.z);
                }
                out4[q] = rho4<RHO>(r, ra, q);
            } else {
                // a quad at an end of the row, or one whose source crosses an end: sample by sample
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int64_t e = F + k;
                    if (e < S || e >= E) continue;
                    const int64_t ts = e - S - d;
                    out[e] = rho1<RHO>((ts >= 0 && ts < T) ? __ldg(in + S + ts) : 0.0f, ra, e);
                }
            }
        }
    }
}

template <bool LUT, bool RHO>
__global__ void __launch_bounds__(256)
shift_scalar_kernel(float *__restrict__ out, const float *__restrict__ in,
                    const float *__restrict__ lut, float shift, float Ts,
                    int64_t rows, int T, int64_t nNeurons, int lpr_log2, RhoArgs ra)
{
    const int lpr = 1 << lpr_log2;
    const int lane_in_row = threadIdx.x & (lpr - 1);
    const int64_t groups_per_block = blockDim.x >> lpr_log2;
    const int64_t group0 = (int64_t)blockIdx.x * groups_per_block + (threadIdx.x >> lpr_log2);
    const int64_t group_stride = (int64_t)gridDim.x * groups_per_block;

    for (int64_t row = group0; row < rows; row += group_stride) {
        const float sv = LUT ? __ldg(lut + (row % nNeurons)) : shift;
        const int d = shift_steps(sv, Ts);
        const float *src = in + row * T;
        float *dst = out + row * T;
#pragma unroll 4
        for (int t = lane_in_row; t < T; t += lpr) {
            const int64_t id = (int64_t)t - d;
            dst[t] = rho1<RHO>((id >= 0 && id < T) ? __ldg(src + id) : 0.0f, ra, row * (int64_t)T + t);
        }
    }
}

template <bool RHO>
static int launch_shift(float *out, const float *in, const float *lut, float shift, float Ts,
                        int64_t rows, int64_t T, int64_t nNeurons, cudaStream_t stream, RhoArgs ra)
{
    if (rows == 0 || T == 0) return SLAYER_B200_OK;
    const bool aligned = aligned16(out) && aligned16(in) && (!RHO || aligned16(ra.u));
    const bool vec = aligned && (T % 4 == 0);
    const bool flat = aligned && !vec && T >= 8;
    const int64_t units = vec ? T / 4 : (flat ? T / 4 + 1 : T);   // accesses per row
    int lpr_log2 = 0;
    while ((1 << lpr_log2) < units && lpr_log2 < 5) ++lpr_log2;
    const int threads = 256;
    const int64_t groups_per_block = threads >> lpr_log2;
    int64_t blocks = ceil_div(rows, groups_per_block);
    const int64_t cap = (int64_t)sm_count() * 8 * 4;   // a few waves of resident CTAs
    if (blocks > cap) blocks = cap;
    const unsigned g = (unsigned)blocks;
    const float *l = lut;
    const int64_t nn = lut ? nNeurons : 1;
    if (vec && RHO) {
        const int T4 = (int)(T / 4);
        int rpb = (1024 + T4 - 1) / T4;                 // about four quads per thread and block of rows
        if (rpb > kRhoRowsMax) rpb = kRhoRowsMax;
        int64_t nb = ceil_div(rows, rpb);
        if (nb > cap) nb = cap;
        if (lut) spike_grad_shift_rows_kernel<true, RHO><<<(unsigned)nb, threads, 0, stream>>>(
            (float4 *)out, (const float4 *)in, (const float4 *)ra.u, l, 0.f, Ts, rows, T4, nn, rpb, ra.theta, ra.tau, ra.c);
        else spike_grad_shift_rows_kernel<false, RHO><<<(unsigned)nb, threads, 0, stream>>>(
            (float4 *)out, (const float4 *)in, (const float4 *)ra.u, nullptr, shift, Ts, rows, T4, nn, rpb, ra.theta, ra.tau, ra.c);
    } else if (vec) {
        if (lut) shift_vec4_kernel<true, RHO><<<g, threads, 0, stream>>>((float4 *)out, (const float4 *)in, l, 0.f, Ts, rows, (int)(T / 4), nn, lpr_log2, ra);
        else shift_vec4_kernel<false, RHO><<<g, threads, 0, stream>>>((float4 *)out, (const float4 *)in, nullptr, shift, Ts, rows, (int)(T / 4), nn, lpr_log2, ra);
    } else if (flat && RHO && T < (1 << 20)) {
        const int unit = (T & 1) ? 4 : 2;               // rows per quad-aligned unit (T % 4 != 0 here)
        int rpb = (int)((16384 + T - 1) / T);           // about sixteen quads per thread and block of rows: few barriers
        rpb = ((rpb + unit - 1) / unit) * unit;
        if (rpb > kRhoRowsMax) rpb = kRhoRowsMax;       // kRhoRowsMax is a multiple of 4
        int64_t nb = ceil_div(rows, rpb);
        if (nb > cap) nb = cap;
        if (lut) spike_grad_shift_flat_rows_kernel<true><<<(unsigned)nb, threads, 0, stream>>>(
            out, in, ra.u, l, 0.f, Ts, rows, (int)T, nn, rpb, ra.theta, ra.tau, ra.c);
        else spike_grad_shift_flat_rows_kernel<false><<<(unsigned)nb, threads, 0, stream>>>(
            out, in, ra.u, nullptr, shift, Ts, rows, (int)T, nn, rpb, ra.theta, ra.tau, ra.c);
    } else if (flat) {
        if (lut) shift_flat4_kernel<true, RHO><<<g, threads, 0, stream>>>(out, in, l, 0.f, Ts, rows, (int)T, nn, lpr_log2, ra);
        else shift_flat4_kernel<false, RHO><<<g, threads, 0, stream>>>(out, in, nullptr, shift, Ts, rows, (int)T, nn, lpr_log2, ra);
    } else {
        if (lut) shift_scalar_kernel<true, RHO><<<g, threads, 0, stream>>>(out, in, l, 0.f, Ts, rows, (int)T, nn, lpr_log2, ra);
        else shift_scalar_kernel<false, RHO><<<g, threads, 0, stream>>>(out, in, nullptr, shift, Ts, rows, (int)T, nn, lpr_log2, ra);
    }
    return check_launch(RHO ? "shift + surrogate gradient kernel launch" : "shift kernel launch");
}

}  // namespace sb200

extern "C" int slayer_b200_shift_scalar(float *out, const float *in, float shift,
                                        int64_t rows, int64_t T, float Ts, void *stream)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(rows >= 0 && T >= 0, "shift: negative size (rows=%lld, T=%lld)", (long long)rows, (long long)T);
    SB200_REQUIRE(T < (1LL << 31) - 8, "shift: T=%lld too large", (long long)T);
    SB200_REQUIRE(rows == 0 || T == 0 || (out && in), "shift: null pointer");
    SB200_REQUIRE(out != in || rows == 0 || T == 0, "shift: out must not alias in");
    return launch_shift<false>(out, in, nullptr, shift, Ts, rows, T, 1, (cudaStream_t)stream, RhoArgs{nullptr, 0.f, 1.f, 0.f});
}

extern "C" int slayer_b200_shift_lut(float *out, const float *in, const float *lut,
                                     int64_t nBatch, int64_t nNeurons, int64_t T, float Ts, void *stream)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(nBatch >= 0 && nNeurons >= 0 && T >= 0, "shift: negative size");
    SB200_REQUIRE(T < (1LL << 31) - 8, "shift: T=%lld too large", (long long)T);
    const int64_t rows = nBatch * nNeurons;
    SB200_REQUIRE(rows == 0 || T == 0 || (out && in && lut), "shift: null pointer");
    SB200_REQUIRE(out != in || rows == 0 || T == 0, "shift: out must not alias in");
    if (rows == 0) return SLAYER_B200_OK;
    return launch_shift<false>(out, in, lut, 0.f, Ts, rows, T, nNeurons, (cudaStream_t)stream, RhoArgs{nullptr, 0.f, 1.f, 0.f});
}

extern "C" int slayer_b200_spike_grad_shift(float *out, const float *grad_output, const float *u, const float *shift_lut,
                                            float shift, int64_t nBatch, int64_t nNeurons, int64_t T, float Ts,
                                            float theta, float tau, float scale, void *stream)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(nBatch >= 0 && nNeurons >= 0 && T >= 0, "spike_grad_shift: negative size");
    SB200_REQUIRE(T < (1LL << 31) - 8, "spike_grad_shift: T=%lld too large", (long long)T);
    const int64_t rows = nBatch * nNeurons;
    if (rows == 0 || T == 0) return SLAYER_B200_OK;
    SB200_REQUIRE(out && grad_output && u, "spike_grad_shift: null pointer");
    SB200_REQUIRE(out != grad_output, "spike_grad_shift: out must not alias grad_output");
    const RhoArgs ra = {u, theta, tau, scale / tau};
    return launch_shift<true>(out, grad_output, shift_lut, shift, Ts, rows, T, nNeurons, (cudaStream_t)stream, ra);
}
