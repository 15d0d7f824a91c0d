// Bit-packed spike tensors: conversion to and from the fp32 form of the operator interface.
//
// A spike tensor holds two values, 0 and 1/Ts.  Packed, a row of T samples is ceil(T / 32)
// 32-bit words, bit i of word w = "sample 32 w + i is a spike" (bits past T are zero) - 1/32 of
// the bytes.  The spike kernels can write this form directly (slayer_b200_srm_get_spikes_packed)
// and the psp filter can read it (slayer_b200_conv_packed); the two kernels here are the fp32
// views at the edge: 4 + 1/8 algorithmic bytes per element each, bound by HBM.
#include "common.cuh"

namespace sb200 {

// one warp per (row, word): 32 consecutive samples of a row, one ballot
__global__ void __launch_bounds__(256)
pack_spikes_kernel(unsigned *__restrict__ bits, const float *__restrict__ s, int64_t rows, int T, int words)
{
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const int64_t items = rows * words;
    for (int64_t it = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); it < items; it += nwarps) {
        const int64_t row = it / words;
        const int w = (int)(it - row * words);
        const int t = 32 * w + lane;
        const float v = t < T ? s[row * (int64_t)T + t] : 0.0f;
        const unsigned m = __ballot_sync(0xffffffffu, v != 0.0f);
        if (lane == 0) bits[it] = m;
    }
}

__global__ void __launch_bounds__(256)
unpack_spikes_kernel(float *__restrict__ s, const unsigned *__restrict__ bits, int64_t rows, int T, int words, float value)
{
    const int64_t n = rows * (int64_t)T;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
        const int64_t row = e / T;
        const int t = (int)(e - row * T);
        s[e] = ((__ldg(bits + row * words + (t >> 5)) >> (t & 31)) & 1u) ? value : 0.0f;
    }
}

}  // namespace sb200

extern "C" int slayer_b200_pack_spikes(uint32_t *bits, const float *s, int64_t rows, int64_t T, void *stream)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(rows >= 0 && T >= 0, "pack_spikes: negative size");
    SB200_REQUIRE(T < (1LL << 31) - 64, "pack_spikes: T=%lld too large", (long long)T);
    if (rows == 0 || T == 0) return SLAYER_B200_OK;
    SB200_REQUIRE(bits && s, "pack_spikes: null pointer");
    const int words = (int)((T + 31) >> 5);
    int64_t blocks = ceil_div(rows * words, 8);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    pack_spikes_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(bits, s, rows, (int)T, words);
    return check_launch("pack_spikes kernel launch");
}

extern "C" int slayer_b200_unpack_spikes(float *s, const uint32_t *bits, int64_t rows, int64_t T, float value, void *stream)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(rows >= 0 && T >= 0, "unpack_spikes: negative size");
    SB200_REQUIRE(T < (1LL << 31) - 64, "unpack_spikes: T=%lld too large", (long long)T);
    if (rows == 0 || T == 0) return SLAYER_B200_OK;
    SB200_REQUIRE(bits && s, "unpack_spikes: null pointer");
    const int words = (int)((T + 31) >> 5);
    int64_t blocks = ceil_div(rows * T, 256);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    unpack_spikes_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(s, bits, rows, (int)T, words, value);
    return check_launch("unpack_spikes kernel launch");
}
