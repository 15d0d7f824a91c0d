// Gradient of the loss with respect to the per-neuron axonal delays, one fused pass:
//   gradDelay[n] = Ts * sum_{b,t} g[b,n,t] * diff[b,n,t],
//   diff[b,n,t]  = out[b,n,t] * (-1/Ts) + out[b,n,t-1] * (1/Ts)      (out[.., -1] = 0)
// where `out` is the delayed signal the forward pass produced and g the gradient arriving at
// it.  The reference composes this from a two-tap conv, an elementwise product and a tensor
// reduction, writing two full-size temporaries; here g and out are read once (8 algorithmic
// bytes per element, bound by HBM) and nothing but the [nNeurons] result is written.
//
// One CTA per neuron: warp w takes batch samples w, w+8, ..., lanes stride over time with
// 128-bit loads when rows are 16-byte aligned; partial sums are combined by warp shuffles and
// a fixed-order pass over the eight warp sums, so the result does not depend on scheduling.
#include "common.cuh"

namespace sb200 {

constexpr int kDelayGradWarps = 8;

template <bool VEC>
__global__ void __launch_bounds__(kDelayGradWarps * 32)
delay_grad_kernel(float *__restrict__ grad_delay, const float *__restrict__ g, const float *__restrict__ out,
                  int64_t nBatch, int64_t nNeurons, int T, float Ts)
{
    __shared__ float warp_sum[kDelayGradWarps];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const float f0 = -1.0f / Ts, f1 = 1.0f / Ts;

    for (int64_t n = blockIdx.x; n < nNeurons; n += gridDim.x) {
        float acc = 0.0f;
        // two batch samples per pass, so that each lane keeps four 128-bit loads in flight
        for (int64_t b = warp; b < nBatch; b += 2 * kDelayGradWarps) {
            const int64_t b2 = b + kDelayGradWarps;
            const bool two = b2 < nBatch;
            const float *g0 = g + (b * nNeurons + n) * (int64_t)T;
            const float *o0 = out + (b * nNeurons + n) * (int64_t)T;
            const float *g1 = two ? g + (b2 * nNeurons + n) * (int64_t)T : g0;
            const float *o1 = two ? out + (b2 * nNeurons + n) * (int64_t)T : o0;
            float acc1 = 0.0f;
            if (VEC) {
                for (int t = lane * 4; t < T; t += 128) {
                    const float4 ga = __ldg(reinterpret_cast<const float4 *>(g0 + t));
                    const float4 oa = __ldg(reinterpret_cast<const float4 *>(o0 + t));
                    const float4 gb = __ldg(reinterpret_cast<const float4 *>(g1 + t));
                    const float4 ob = __ldg(reinterpret_cast<const float4 *>(o1 + t));
                    const float pa = t > 0 ? __ldg(o0 + t - 1) : 0.0f;
                    const float pb = t > 0 ? __ldg(o1 + t - 1) : 0.0f;
                    acc = fmaf(ga.x, fmaf(pa, f1, oa.x * f0), acc);
                    acc = fmaf(ga.y, fmaf(oa.x, f1, oa.y * f0), acc);
                    acc = fmaf(ga.z, fmaf(oa.y, f1, oa.z * f0), acc);
                    acc = fmaf(ga.w, fmaf(oa.z, f1, oa.w * f0), acc);
                    acc1 = fmaf(gb.x, fmaf(pb, f1, ob.x * f0), acc1);
                    acc1 = fmaf(gb.y, fmaf(ob.x, f1, ob.y * f0), acc1);
                    acc1 = fmaf(gb.z, fmaf(ob.y, f1, ob.z * f0), acc1);
                    acc1 = fmaf(gb.w, fmaf(ob.z, f1, ob.w * f0), acc1);
                }
            } else {
                for (int t = lane; t < T; t += 32) {
                    const float pa = t > 0 ? __ldg(o0 + t - 1) : 0.0f;
                    const float pb = t > 0 ? __ldg(o1 + t - 1) : 0.0f;
                    acc = fmaf(__ldg(g0 + t), fmaf(pa, f1, __ldg(o0 + t) * f0), acc);
                    acc1 = fmaf(__ldg(g1 + t), fmaf(pb, f1, __ldg(o1 + t) * f0), acc1);
                }
            }
            if (two) acc += acc1;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (lane == 0) warp_sum[warp] = acc;
        __syncthreads();
        if (threadIdx.x == 0) {
            float total = 0.0f;
#pragma unroll
            for (int w = 0; w < kDelayGradWarps; ++w) total += warp_sum[w];
            grad_delay[n] = total * Ts;
        }
        __syncthreads();
    }
}

}  // namespace sb200

extern "C" int slayer_b200_delay_grad(float *grad_delay, const float *grad_output, const float *output,
                                      int64_t nBatch, int64_t nNeurons, int64_t T, float Ts, void *stream)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(nBatch >= 0 && nNeurons >= 0 && T >= 0, "delay_grad: negative size");
    SB200_REQUIRE(T < (1LL << 31) - 256, "delay_grad: T=%lld too large", (long long)T);
    if (nNeurons == 0) return SLAYER_B200_OK;
    SB200_REQUIRE(grad_delay != nullptr, "delay_grad: null pointer");
    SB200_REQUIRE(nBatch == 0 || T == 0 || (grad_output && output), "delay_grad: null pointer");
    int64_t grid = nNeurons;
    const int64_t cap = (int64_t)sm_count() * 32;
    if (grid > cap) grid = cap;
    const bool vec = (T % 4 == 0) && aligned16(grad_output) && aligned16(output);
    if (vec)
        delay_grad_kernel<true><<<(unsigned)grid, kDelayGradWarps * 32, 0, (cudaStream_t)stream>>>(
            grad_delay, grad_output, output, nBatch, nNeurons, (int)T, Ts);
    else
        delay_grad_kernel<false><<<(unsigned)grid, kDelayGradWarps * 32, 0, (cudaStream_t)stream>>>(
            grad_delay, grad_output, output, nBatch, nNeurons, (int)T, Ts);
    return check_launch("delay_grad kernel launch");
}
