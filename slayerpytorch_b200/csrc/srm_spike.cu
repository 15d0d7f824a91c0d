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
// Two variants of the inner step:
//   - window of up to 32 steps (NB > 0): the taps live in registers and the step is a fully
//     unrolled run of NB predicated adds, oldest first - no loop, no branch, no memory access;
//   - longer windows (up to 256 steps, W history words): a loop over the set history bits with
//     the taps in shared memory.
//
// Memory: 12 algorithmic bytes per element (read u, write u, write s), bound by HBM.  A warp
// owns 32 rows and walks them in tiles of 32 time steps through the swizzled shared-memory
// tiles of tile.cuh, prefetching the next tile with cp.async while it works on the current one.
#include "common.cuh"
#include "tile.cuh"

namespace sb200 {

constexpr int kMaxHistWords = 8;     // register history covers refractory kernels up to 257 taps

// V: global access width in floats.  NB > 0: unrolled window of NB history bits (W must be 1).
// NB == 0: looped window of W history words.
template <int V, int NB, int W>
__global__ void __launch_bounds__(256)
srm_get_spikes_kernel(float *s, float *u, const float *__restrict__ nu,
                      int64_t rows, int nuEff, int T, float theta, float spikeVal)
{
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps_per_block = blockDim.x >> 5;
    const int nuPad = NB > 0 ? 0 : ((nuEff + 3) & ~3);
    float *nu_s = smem;
    float *tiles = smem + nuPad + warp * (3 * kTileWords);   // two potential tiles (prefetch ring)
    float *tile_s = tiles + 2 * kTileWords;                  // spike tile

    if (NB == 0) {
        for (int i = threadIdx.x; i < nuEff; i += blockDim.x) nu_s[i] = nu[i];
        __syncthreads();
    }

    const bool has_nu0 = nuEff >= 1;
    const float nu0 = has_nu0 ? __ldg(nu) : 0.0f;
    float nu_r[NB > 0 ? NB : 1];     // nu_r[k] = tap of a spike k+1 steps ago
#pragma unroll
    for (int k = 0; k < NB; ++k) nu_r[k] = (k + 1 < nuEff) ? __ldg(nu + k + 1) : 0.0f;

    // bit b of the history (word b/32, bit b%32) = "spiked b+1 steps ago"; keep b <= nuEff-2
    unsigned wmask[W];
#pragma unroll
    for (int w = 0; w < W; ++w) {
        const int nb = nuEff - 1 - 32 * w;
        wmask[w] = nb >= 32 ? 0xffffffffu : (nb <= 0 ? 0u : ((1u << nb) - 1u));
    }

    const int ntiles = (T + kTile - 1) / kTile;
    const int64_t nblocks = (rows + kTile - 1) / kTile;
    const int64_t wstride = (int64_t)gridDim.x * warps_per_block;
    for (int64_t rb = (int64_t)blockIdx.x * warps_per_block + warp; rb < nblocks; rb += wstride) {
        const int64_t row0 = rb * kTile;
        unsigned hist[W];
#pragma unroll
        for (int w = 0; w < W; ++w) hist[w] = 0u;

        tile_prefetch<V>(tiles, u, row0, rows, 0, T, lane);
        cp_async_commit();
        for (int it = 0; it < ntiles; ++it) {
            const int t0 = it * kTile;
            float *tile = tiles + (it & 1) * kTileWords;
            if (it + 1 < ntiles)
                tile_prefetch<V>(tiles + ((it + 1) & 1) * kTileWords, u, row0, rows, t0 + kTile, T, lane);
            cp_async_commit();
            cp_async_wait<1>();
            __syncwarp();

            // walk the 32 steps; the next chunk is fetched before the current one is processed
            float4 cur = *reinterpret_cast<const float4 *>(tile + tile_chunk(lane, 0));
#pragma unroll 2
            for (int c4 = 0; c4 < kTile / 4; ++c4) {
                float4 nxt = cur;
                if (c4 + 1 < kTile / 4) nxt = *reinterpret_cast<const float4 *>(tile + tile_chunk(lane, c4 + 1));
                float vv[4] = {cur.x, cur.y, cur.z, cur.w};
                float sv[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float v = vv[j];
                    // refractory taps of recent spikes, oldest spike first
                    if (NB > 0) {
#pragma unroll
                        for (int k = NB - 1; k >= 0; --k)
                            if (hist[0] & (1u << k)) v += nu_r[k];
                    } else {
#pragma unroll
                        for (int w = W - 1; w >= 0; --w) {
                            unsigned m = hist[w];
                            while (m) {
                                const int k = 31 - __clz(m);
                                v += nu_s[32 * w + k + 1];
                                m &= ~(1u << k);
                            }
                        }
                    }
                    const bool spk = v >= theta;
                    vv[j] = (spk && has_nu0) ? v + nu0 : v;
                    sv[j] = spk ? spikeVal : 0.0f;
#pragma unroll
                    for (int w = W - 1; w > 0; --w)
                        hist[w] = ((hist[w] << 1) | (hist[w - 1] >> 31)) & wmask[w];
                    hist[0] = ((hist[0] << 1) | (spk ? 1u : 0u)) & wmask[0];
                }
                *reinterpret_cast<float4 *>(tile + tile_chunk(lane, c4)) = make_float4(vv[0], vv[1], vv[2], vv[3]);
                *reinterpret_cast<float4 *>(tile_s + tile_chunk(lane, c4)) = make_float4(sv[0], sv[1], sv[2], sv[3]);
                cur = nxt;
            }
            __syncwarp();

            tile_store<V>(tile, u, row0, rows, t0, T, lane);
            tile_store<V>(tile_s, s, row0, rows, t0, T, lane);
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

struct SrmArgs {
    float *s, *u;
    const float *nu;
    int64_t rows;
    int nuEff, T;
    float theta, spikeVal;
    cudaStream_t stream;
};

template <int V, int NB, int W>
static int launch_srm(const SrmArgs &a)
{
    const int64_t nblocks = ceil_div(a.rows, kTile);
    int warps, grid;
    spike_launch_shape(nblocks, 3 * kTileWords * sizeof(float), warps, grid);
    const size_t smem = (size_t)((NB > 0 ? 0 : ((a.nuEff + 3) & ~3)) + warps * 3 * kTileWords) * sizeof(float);
    auto kern = srm_get_spikes_kernel<V, NB, W>;
    int rc = reserve_dynamic_smem((const void *)kern, smem);
    if (rc) return rc;
    kern<<<(unsigned)grid, warps * 32, smem, a.stream>>>(a.s, a.u, a.nu, a.rows, a.nuEff, a.T, a.theta, a.spikeVal);
    return check_launch("srm_get_spikes kernel launch");
}

template <int V>
static int dispatch_srm(const SrmArgs &a)
{
    const int window = a.nuEff > 1 ? a.nuEff - 1 : 0;     // history bits needed
    if (window <= 2) return launch_srm<V, 2, 1>(a);
    if (window <= 4) return launch_srm<V, 4, 1>(a);
    if (window <= 6) return launch_srm<V, 6, 1>(a);
    if (window <= 8) return launch_srm<V, 8, 1>(a);
    if (window <= 10) return launch_srm<V, 10, 1>(a);
    if (window <= 12) return launch_srm<V, 12, 1>(a);
    if (window <= 16) return launch_srm<V, 16, 1>(a);
    if (window <= 24) return launch_srm<V, 24, 1>(a);
    if (window <= 32) return launch_srm<V, 32, 1>(a);
    if (window <= 64) return launch_srm<V, 0, 2>(a);
    if (window <= 128) return launch_srm<V, 0, 4>(a);
    return launch_srm<V, 0, 8>(a);
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
    if (nuEff - 1 > 32 * kMaxHistWords) {
        const int threads = 128;
        srm_get_spikes_long_kernel<<<(unsigned)ceil_div(rows, threads), threads, 0, stream>>>(
            s, u, nu, rows, nuSize, T, theta, spikeVal);
        return check_launch("srm_get_spikes (long refractory kernel) launch");
    }
    const SrmArgs a = {s, u, nu, rows, (int)nuEff, (int)T, theta, spikeVal, stream};
    switch (tile_vec_width(T, {s, u})) {
        case 4: return dispatch_srm<4>(a);
        case 2: return dispatch_srm<2>(a);
        default: return dispatch_srm<1>(a);
    }
}
