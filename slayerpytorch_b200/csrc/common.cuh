// Shared host/device helpers of the slayer_b200 kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "slayer_b200.h"

namespace sb200 {

// Thread-local error message behind slayer_b200_last_error().
void set_error(const char *fmt, ...);
void clear_error();

// Number of SMs of the current device (cached per device).
int sm_count();

// Make sure `func` may be launched with `bytes` of dynamic shared memory on the current
// device (raises the per-function limit above 48 KB when needed; remembered per device).
int reserve_dynamic_smem(const void *func, size_t bytes);

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Checks the launch that was just enqueued.
inline int check_launch(const char *what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(e));
        return SLAYER_B200_ECUDA;
    }
    return SLAYER_B200_OK;
}

#define SB200_REQUIRE(cond, ...)                      \
    do {                                              \
        if (!(cond)) {                                \
            ::sb200::set_error(__VA_ARGS__);          \
            return SLAYER_B200_EINVAL;                \
        }                                             \
    } while (0)

// trunc(shift / Ts) with IEEE division, saturating like the hardware float->int conversion.
__host__ __device__ inline int shift_steps(float shift, float Ts)
{
#ifdef __CUDA_ARCH__
    return __float2int_rz(__fdiv_rn(shift, Ts));
#else
    float q = shift / Ts;
    if (!(q == q)) return 0;
    if (q >= 2147483648.0f) return 2147483647;
    if (q <= -2147483648.0f) return -2147483647 - 1;
    return static_cast<int>(q);
#endif
}

#ifdef __CUDACC__
// g * (c * exp(-|u - theta| / tau)): the surrogate gradient of the spike function applied to
// an incoming gradient sample; c = scale / tau.  IEEE division, as the tensor expression.
__device__ __forceinline__ float rho_times(float g, float u, float theta, float tau, float c)
{
    const float e = expf(__fdiv_rn(-fabsf(u - theta), tau));
    return g * (c * e);
}
#endif

}  // namespace sb200
