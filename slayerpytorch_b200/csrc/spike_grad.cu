// Surrogate gradient of the spike function, one fused streaming pass:
//   out = g * ( scale / tau * exp(-|u - theta| / tau) )
// 12 algorithmic bytes per element (read u, read g, write out); bound by HBM bandwidth.
// Operation order and IEEE division follow the tensor expression it replaces, so the result
// differs from it only by the last-bit behaviour of exp.
#include "common.cuh"

namespace sb200 {

__global__ void __launch_bounds__(256)
spike_grad_vec4_kernel(float4 *out, const float4 *g,
                       const float4 *__restrict__ u, int64_t n4,
                       float theta, float tau, float c)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 gv = g[i];
        const float4 uv = __ldg(u + i);
        float4 r;
        r.x = rho_times(gv.x, uv.x, theta, tau, c);
        r.y = rho_times(gv.y, uv.y, theta, tau, c);
        r.z = rho_times(gv.z, uv.z, theta, tau, c);
        r.w = rho_times(gv.w, uv.w, theta, tau, c);
        out[i] = r;
    }
}

__global__ void __launch_bounds__(256)
spike_grad_scalar_kernel(float *out, const float *g,
                         const float *__restrict__ u, int64_t first, int64_t n,
                         float theta, float tau, float c)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = first + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = rho_times(g[i], u[i], theta, tau, c);
}

}  // namespace sb200

extern "C" int slayer_b200_spike_grad(float *out, const float *g, const float *u, int64_t n,
                                      float theta, float tau, float scale, void *stream_)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(n >= 0, "spike_grad: negative size");
    if (n == 0) return SLAYER_B200_OK;
    SB200_REQUIRE(out && g && u, "spike_grad: null pointer");
    cudaStream_t stream = (cudaStream_t)stream_;
    const float c = scale / tau;
    const int threads = 256;
    const int64_t cap = (int64_t)sm_count() * 8 * 4;
    int64_t done = 0;
    if (aligned16(out) && aligned16(g) && aligned16(u) && n >= 4) {
        const int64_t n4 = n / 4;
        int64_t blocks = ceil_div(n4, threads);
        if (blocks > cap) blocks = cap;
        spike_grad_vec4_kernel<<<(unsigned)blocks, threads, 0, stream>>>(
            (float4 *)out, (const float4 *)g, (const float4 *)u, n4, theta, tau, c);
        done = n4 * 4;
    }
    if (done < n) {
        int64_t blocks = ceil_div(n - done, threads);
        if (blocks > cap) blocks = cap;
        spike_grad_scalar_kernel<<<(unsigned)blocks, threads, 0, stream>>>(out, g, u, done, n, theta, tau, c);
    }
    return check_launch("spike_grad kernel launch");
}
