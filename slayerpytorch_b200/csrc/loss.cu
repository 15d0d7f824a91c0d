// Spike-count loss (forward value and gradient) in one pass.
//
// For output spikes s[row, t] (rows = batch x classes) with a target region [lo, hi) and a
// desired number of spikes per row:
//   count      = Ts * sum_{t in region} s[t]
//   c          = float( (double(count) - desired) / (stop - start) * scale )        (one rounding)
//   e[t]       = psp(s outside the region)[t] + (t in region ? c : 0)               (psp = causal FIR, x Ts)
//   loss       = Ts / 2 * sum_{rows, t} e[t]^2
//   dloss/ds   = psp_adjoint(Ts * e)                                                (corr, x Ts)
// which is spikeLoss.numSpikes of the reference with its backward pass (the part of the output
// inside the region enters as a constant).  The reference builds the terms on the host with
// NumPy; a tensor-expression version costs about twenty small launches.  Here one warp walks one
// row: the row, its error signal and the taps sit in shared memory, lanes take time steps.
// psp and its adjoint are the same fp32 fused-multiply-add chains as the conv / corr operators
// (ascending taps, x Ts last).  The kernel leaves sum_t e^2 per row (double); the caller adds the
// rows up.
#include "common.cuh"

namespace sb200 {

constexpr int kLossWarps = 4;

__global__ void __launch_bounds__(kLossWarps * 32)
num_spikes_loss_kernel(float *__restrict__ grad, double *__restrict__ row_sq, const float *__restrict__ s,
                       const float *__restrict__ desired_count, const float *__restrict__ filt,
                       int64_t rows, int T, int K, int lo, int hi, int span, float Ts, float scale)
{
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    float *fs = smem;                                    // K taps
    float *x = fs + K + warp * 2 * T;                    // the row outside the region, then Ts * e
    float *e = x + T;
    for (int i = threadIdx.x; i < K; i += blockDim.x) fs[i] = filt[i];
    __syncthreads();

    for (int64_t row = (int64_t)blockIdx.x * kLossWarps + warp; row < rows; row += (int64_t)gridDim.x * kLossWarps) {
        const float *sr = s + row * (int64_t)T;
        float cnt = 0.0f;
        for (int t = lane; t < T; t += 32) {
            const float v = sr[t];
            const bool in = t >= lo && t < hi;
            x[t] = in ? 0.0f : v;
            if (in) cnt += v;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
        const float actual = cnt * Ts;
        const float c = (float)(((double)actual - (double)desired_count[row]) / (double)span * (double)scale);
        __syncwarp();
        double sq = 0.0;
        for (int t = lane; t < T; t += 32) {
            float acc = 0.0f;
            const int km = K < t + 1 ? K : t + 1;
            for (int i = 0; i < km; ++i) acc = fmaf(x[t - i], fs[i], acc);
            const float err = acc * Ts + ((t >= lo && t < hi) ? c : 0.0f);
            e[t] = err * Ts;
            sq += (double)err * (double)err;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) row_sq[row] = sq;
        __syncwarp();
        float *gr = grad + row * (int64_t)T;
        for (int t = lane; t < T; t += 32) {
            float acc = 0.0f;
            const int km = K < T - t ? K : T - t;
            for (int i = 0; i < km; ++i) acc = fmaf(e[t + i], fs[i], acc);
            gr[t] = acc * Ts;
        }
        __syncwarp();
    }
}

}  // namespace sb200

extern "C" int slayer_b200_num_spikes_loss(float *grad, double *row_sq, const float *s, const float *desired_count,
                                           const float *filter, int64_t rows, int64_t T, int64_t K,
                                           int64_t start, int64_t stop, float Ts, float scale, void *stream)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(rows >= 0 && T >= 0 && K >= 0, "num_spikes_loss: negative size");
    SB200_REQUIRE(stop != start, "num_spikes_loss: empty target region");
    if (rows == 0 || T == 0) return SLAYER_B200_OK;
    SB200_REQUIRE(grad && row_sq && s && desired_count && (filter || K == 0), "num_spikes_loss: null pointer");
    SB200_REQUIRE(grad != s, "num_spikes_loss: grad must not alias s");
    const int64_t Keff = K < T ? K : T;
    const size_t smem = sizeof(float) * ((size_t)Keff + (size_t)kLossWarps * 2 * T);
    if (T >= (1 << 24) || smem > 200 * 1024) {
        set_error("num_spikes_loss: rows of %lld steps do not fit the kernel's shared memory", (long long)T);
        return SLAYER_B200_EUNSUPPORTED;
    }
    // the slice [start:stop] of a row of T samples, as Python slicing resolves it
    int64_t lo = start < 0 ? start + T : start, hi = stop < 0 ? stop + T : stop;
    lo = lo < 0 ? 0 : (lo > T ? T : lo);
    hi = hi < 0 ? 0 : (hi > T ? T : hi);
    int rc = reserve_dynamic_smem((const void *)num_spikes_loss_kernel, smem);
    if (rc) return rc;
    int64_t blocks = ceil_div(rows, kLossWarps);
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    num_spikes_loss_kernel<<<(unsigned)blocks, kLossWarps * 32, smem, (cudaStream_t)stream>>>(
        grad, row_sq, s, desired_count, filter, rows, (int)T, (int)Keff, (int)lo, (int)hi, (int)(stop - start), Ts, scale);
    return check_launch("num_spikes_loss kernel launch");
}
