// SRM spike generation with refractory response (in place on the membrane potential).
//
// Sequential definition, per row:  for t = 0..T-1:  if u[t] >= theta { s[t] = 1/Ts;
// u[t+j] += nu[j] for j < nuSize, t+j < T } else s[t] = 0.
//
// Formulation used here ("gather"): the value tested at time t is the ORIGINAL u[t] plus the
// refractory taps of the spikes of the last nuSize-1 steps, added oldest spike first.  Each
// tap is its own fp32 add and the adds reach a sample in spike order, exactly as in the
// sequential definition, so spikes and the updated potential are bit-identical to it.  What
// changes is the data flow: a lane keeps its row's recent spike history as a bit window in
// registers and never writes ahead of itself, so the recurrence reads memory strictly forward
// and time can be tiled with no state in memory between tiles.
//
// Memory: 12 algorithmic bytes per element (read u, write u, write s), bound by HBM.  A warp
// owns 32 rows and walks them in tiles of 32 time steps through the swizzled shared-memory
// tile of tile.cuh, so every global access is a contiguous 128-byte row segment.
#include "common.cuh"
#include "tile.cuh"

namespace sb200 {

constexpr int kMaxHistWords = 8;     // register history covers refractory kernels up to 257 taps

template <int W>
__global__ void __launch_bounds__(256)
srm_get_spikes_kernel(float *s, float *u, const float *__restrict__ nu,
                      int64_t rows, int nuEff, int T, float theta, float spikeVal)
{
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps_per_block = blockDim.x >> 5;
    const int nuPad = (nuEff + 3) & ~3;
    float *nu_s = smem;
    float *tile = smem + nuPad + warp * kTileWords;

    for (int i = threadIdx.x; i < nuEff; i += blockDim.x) nu_s[i] = nu[i];
    __syncthreads();

    const bool has_nu0 = nuEff >= 1;
    const float nu0 = has_nu0 ? nu_s[0] : 0.0f;

    // bit b of the history (word b/32, bit b%32) = "spiked b+1 steps ago"; keep b <= nuEff-2
    unsigned wmask[W];
#pragma unroll
    for (int w = 0; w < W; ++w) {
        const int nb = nuEff - 1 - 32 * w;
        wmask[w] = nb >= 32 ? 0xffffffffu : (nb <= 0 ? 0u : ((1u << nb) - 1u));
    }

    const int64_t nblocks = (rows + kTile - 1) / kTile;
    const int64_t wstride = (int64_t)gridDim.x * warps_per_block;
    for (int64_t rb = (int64_t)blockIdx.x * warps_per_block + warp; rb < nblocks; rb += wstride) {
        const int64_t row0 = rb * kTile;
        unsigned hist[W];
#pragma unroll
        for (int w = 0; w < W; ++w) hist[w] = 0u;

        for (int t0 = 0; t0 < T; t0 += kTile) {
            tile_load(tile, u, row0, rows, t0, T, lane);
            __syncwarp();

            unsigned smask = 0u;
#pragma unroll 1
            for (int c4 = 0; c4 < kTile / 4; ++c4) {
                float4 *chunk = reinterpret_cast<float4 *>(tile + tile_chunk(lane, c4));
                const float4 in4 = *chunk;
                float vv[4] = {in4.x, in4.y, in4.z, in4.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float v = vv[j];
                    // refractory taps of recent spikes, oldest spike first
#pragma unroll
                    for (int w = W - 1; w >= 0; --w) {
                        unsigned m = hist[w];
                        while (m) {
                            const int k = 31 - __clz(m);
                            v += nu_s[32 * w + k + 1];
                            m &= ~(1u << k);
                        }
                    }
                    const bool spk = v >= theta;
                    vv[j] = (spk && has_nu0) ? v + nu0 : v;
                    smask |= (spk ? 1u : 0u) << (c4 * 4 + j);
#pragma unroll
                    for (int w = W - 1; w > 0; --w)
                        hist[w] = ((hist[w] << 1) | (hist[w - 1] >> 31)) & wmask[w];
                    hist[0] = ((hist[0] << 1) | (spk ? 1u : 0u)) & wmask[0];
                }
                *chunk = make_float4(vv[0], vv[1], vv[2], vv[3]);
            }
            __syncwarp();

            tile_store(tile, u, row0, rows, t0, T, lane);
            mask_store(smask, spikeVal, s, row0, rows, t0, T, lane);
            __syncwarp();
        }
    }
}

// Direct restatement for refractory kernels too long for the register history: one thread per
// row on global memory.  Correct for any size; only reached for nuSize > 257.
__global__ void __launch_bounds__(128)
srm_get_spikes_long_kernel(float *s, float *u, const float *__restrict__ nu,
                           int64_t rows, int64_t nuSize, int64_t T, float theta, float spikeVal)
{
    const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    float *ur = u + row * T;
    float *sr = s + row * T;
    for (int64_t t = 0; t < T; ++t) {
        if (ur[t] >= theta) {
            sr[t] = spikeVal;
            const int64_t n = nuSize < T - t ? nuSize : T - t;
            for (int64_t j = 0; j < n; ++j) ur[t + j] += nu[j];
        } else {
            sr[t] = 0.0f;
        }
    }
}

template <int W>
static int launch_srm(float *s, float *u, const float *nu, int64_t rows, int nuEff, int T,
                      float theta, float spikeVal, cudaStream_t stream)
{
    const int64_t nblocks = ceil_div(rows, kTile);
    const int sms = sm_count();
    int warps = 8;                                   // spread small problems over all SMs
    while (warps > 1 && ceil_div(nblocks, warps) < 2 * (int64_t)sms) warps >>= 1;
    int64_t grid = ceil_div(nblocks, warps);
    const int64_t cap = (int64_t)sms * 16;
    if (grid > cap) grid = cap;
    const size_t smem = (size_t)(((nuEff + 3) & ~3) + warps * kTileWords) * sizeof(float);
    srm_get_spikes_kernel<W><<<(unsigned)grid, warps * 32, smem, stream>>>(
        s, u, nu, rows, nuEff, T, theta, spikeVal);
    return check_launch("srm_get_spikes kernel launch");
}

}  // namespace sb200

extern "C" int slayer_b200_srm_get_spikes(float *s, float *u, const float *nu,
                                          int64_t rows, int64_t nuSize, int64_t T,
                                          float theta, float Ts, void *stream_)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(rows >= 0 && nuSize >= 0 && T >= 0, "srm_get_spikes: negative size");
    SB200_REQUIRE(T < (1LL << 31) - 64, "srm_get_spikes: T=%lld too large", (long long)T);
    if (rows == 0 || T == 0) return SLAYER_B200_OK;
    SB200_REQUIRE(s && u && (nu || nuSize == 0), "srm_get_spikes: null pointer");
    SB200_REQUIRE(s != u, "srm_get_spikes: s must not alias u");
    cudaStream_t stream = (cudaStream_t)stream_;
    const float spikeVal = 1.0f / Ts;
    const int64_t nuEff = nuSize < T ? nuSize : T;    // taps beyond the row end never land
    const int64_t words = ceil_div(nuEff > 1 ? nuEff - 1 : 1, 32);
    if (words <= 1) return launch_srm<1>(s, u, nu, rows, (int)nuEff, (int)T, theta, spikeVal, stream);
    if (words <= 2) return launch_srm<2>(s, u, nu, rows, (int)nuEff, (int)T, theta, spikeVal, stream);
    if (words <= 4) return launch_srm<4>(s, u, nu, rows, (int)nuEff, (int)T, theta, spikeVal, stream);
    if (words <= kMaxHistWords)
        return launch_srm<8>(s, u, nu, rows, (int)nuEff, (int)T, theta, spikeVal, stream);
    const int threads = 128;
    srm_get_spikes_long_kernel<<<(unsigned)ceil_div(rows, threads), threads, 0, stream>>>(
        s, u, nu, rows, nuSize, T, theta, spikeVal);
    return check_launch("srm_get_spikes (long refractory kernel) launch");
}
