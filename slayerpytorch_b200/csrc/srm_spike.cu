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
// Three variants of the inner step, all producing the same bits:
//   - "ring" (refractory window shorter than the time tile and every tap negative or -0.0,
//     which is what refractory kernels look like): spikes are kept as 0.0 / 1.0 flags in a
//     register ring indexed at compile time (the time tile is fully unrolled), the potentials
//     of the tile sit in registers, and once the flag of a step is known its taps go to the
//     following samples as v = fma(flag, tap, v).  fma(1, tap, v) is the add the definition
//     asks for; fma(+0, tap, v) adds -0.0 and returns v unchanged, bit for bit.  A sample still
//     receives its taps oldest spike first, but the adds that follow one flag are independent,
//     so the dependency from step to step is one multiply-add, one compare and one select.
//     No predicates, no branches: the step runs on the FMA pipe;
//   - "bits" (window of up to 32 steps, any taps): history bits in a register, a fully
//     unrolled run of predicated adds, oldest first;
//   - "loop" (windows up to 256 steps): a loop over the set history bits, taps in shared memory.
//
// Memory: 12 algorithmic bytes per element (read u, write u, write s), bound by HBM.  A warp
// owns 32 rows and walks them in time tiles staged in swizzled shared memory, so that global
// memory only ever sees contiguous row segments; tiles are 64 steps wide (256 bytes per row)
// wherever the buffers are 16-byte aligned, because DRAM serves longer row segments faster.
// Three data-movement paths feed the same recurrence: bulk tensor copies (TMA) for the loads
// when rows start on 16-byte boundaries (T % 4 == 0), cp.async with row-skewed wide tiles for
// any other row length, and cp.async with 32-step tiles for unaligned buffers.
#include <atomic>
#include <mutex>

#include "common.cuh"
#include "tile.cuh"
#include "tma.cuh"

namespace sb200 {

constexpr int kMaxHistWords = 8;     // register history covers refractory kernels up to 257 taps

// Per-row state of the recurrence and one time step of it.
// NB > 0: unrolled window of NB history bits, taps in registers (W must be 1).
// NB == 0: looped window of W history words, taps in shared memory.
template <int NB, int W>
struct SrmRow {
    unsigned hist[W];        // bit b (word b/32, bit b%32) = "spiked b+1 steps ago"
    unsigned wmask[W];       // keeps only b <= nuEff-2
    float nu_r[NB > 0 ? NB : 1];   // nu_r[k] = tap of a spike k+1 steps ago
    float nu0, theta, spikeVal;
    bool has_nu0;
    bool taps_negative;      // every tap after the first is finite with its sign bit set (ring variant is exact)
    const float *nu_s;

    __device__ __forceinline__ void init(const float *__restrict__ nu, const float *nu_smem, int nuEff,
                                         float theta_, float spikeVal_)
    {
        theta = theta_;
        spikeVal = spikeVal_;
        nu_s = nu_smem;
        has_nu0 = nuEff >= 1;
        nu0 = has_nu0 ? __ldg(nu) : 0.0f;
        taps_negative = true;
#pragma unroll
        for (int k = 0; k < NB; ++k) {
            nu_r[k] = (k + 1 < nuEff) ? __ldg(nu + k + 1) : -0.0f;
            // sign bit set and not Inf / NaN: the ring variant multiplies every tap by a 0/1 flag,
            // and 0 * -inf is NaN where the definition adds nothing (a tap of -inf is a legitimate
            // way to write an absolute refractory period; it takes the bits variant)
            const unsigned bits = __float_as_uint(nu_r[k]);
            taps_negative = taps_negative && (bits >> 31) && ((bits & 0x7f800000u) != 0x7f800000u);
        }
#pragma unroll
        for (int w = 0; w < W; ++w) {
            const int nb = nuEff - 1 - 32 * w;
            wmask[w] = nb >= 32 ? 0xffffffffu : (nb <= 0 ? 0u : ((1u << nb) - 1u));
        }
    }

    __device__ __forceinline__ void reset()
    {
#pragma unroll
        for (int w = 0; w < W; ++w) hist[w] = 0u;
    }

    // v: original potential in, updated potential out; returns whether the row spiked
    __device__ __forceinline__ bool step(float &v)
    {
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
        if (spk && has_nu0) v += nu0;
#pragma unroll
        for (int w = W - 1; w > 0; --w) hist[w] = ((hist[w] << 1) | (hist[w - 1] >> 31)) & wmask[w];
        hist[0] = ((hist[0] << 1) | (spk ? 1u : 0u)) & wmask[0];
        return spk;
    }
};

// v = a * b + v with IEEE rounding and no flushing, so that a flag of +0 leaves v untouched
__device__ __forceinline__ void fma_keep(float &v, float a, float b)
{
    asm("fma.rn.f32 %0, %1, %2, %0;" : "+f"(v) : "f"(a), "f"(b));
}

// Word offset of 16-byte chunk c of row r in a time tile of R = 32 steps: the 128-byte swizzle
// of tile.cuh, which is also the layout a bulk tensor copy with that swizzle mode produces.
template <int R>
__device__ __forceinline__ int chunk_of(int r, int c)
{
    static_assert(R == kTile, "time tiles are 32 steps wide");
    return tile_chunk(r, c);
}

// Walk one time tile of R steps for this lane's row: potentials are updated in place in
// `tile`; the spikes are returned as a bit mask (bit i = spiked at step i) and, with FLOATS,
// also written as samples to `tile_s`.  RING selects the ring variant (needs NB < R).
//
// Ring variant.  ring[i] holds the 0/1 flag "spiked at step i" of the tile being walked (and,
// until step i overwrites it, of the previous tile).  The R potentials of the tile sit in
// registers; as soon as the flag of step i is known its refractory taps are added to the next
// NB potentials.  A potential thus receives its terms in the order the spikes occurred (oldest
// first, the order of a sequential walk), but the NB additions that follow one flag are
// independent of each other, so the loop-carried dependency per step is a single multiply-add,
// a compare and a select instead of a chain of NB multiply-adds.  Spikes of the previous tile
// reach the first NB steps through a triangular block of additions at the start of the tile.
template <int R, bool RING, int NB, int W, bool FLOATS = true>
__device__ __forceinline__ unsigned walk_tile(float *tile, float *tile_s, SrmRow<NB, W> &st, float (&ring)[R], int lane)
{
    unsigned mask = 0u;
    if constexpr (RING) {
        float a[R];
#pragma unroll
        for (int c4 = 0; c4 < R / 4; ++c4) {
            const float4 x = *reinterpret_cast<const float4 *>(tile + chunk_of<R>(lane, c4));
            a[4 * c4] = x.x; a[4 * c4 + 1] = x.y; a[4 * c4 + 2] = x.z; a[4 * c4 + 3] = x.w;
        }
        // spikes of the previous tile: step t < NB still lacks the taps k = NB .. t+1
#pragma unroll
        for (int t = 0; t < NB; ++t) {
#pragma unroll
            for (int k = NB; k > t; --k) fma_keep(a[t], ring[(t - k) & (R - 1)], st.nu_r[k - 1]);
        }
#pragma unroll
        for (int c4 = 0; c4 < R / 4; ++c4) {
            float sv[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = c4 * 4 + j;
                const bool spk = a[i] >= st.theta;
                const float f = spk ? 1.0f : 0.0f;
                ring[i] = f;
#pragma unroll
                for (int d = 1; d <= NB; ++d)
                    if (i + d < R) fma_keep(a[i + d], f, st.nu_r[d - 1]);
                if (spk && st.has_nu0) a[i] += st.nu0;
                if (FLOATS) sv[j] = spk ? st.spikeVal : 0.0f;
                else if (spk) mask |= 1u << i;
            }
            *reinterpret_cast<float4 *>(tile + chunk_of<R>(lane, c4)) =
                make_float4(a[4 * c4], a[4 * c4 + 1], a[4 * c4 + 2], a[4 * c4 + 3]);
            if (FLOATS)
                *reinterpret_cast<float4 *>(tile_s + chunk_of<R>(lane, c4)) = make_float4(sv[0], sv[1], sv[2], sv[3]);
        }
    } else {
        float4 cur = *reinterpret_cast<const float4 *>(tile + chunk_of<R>(lane, 0));
#pragma unroll
        for (int c4 = 0; c4 < R / 4; ++c4) {
            float4 nxt = cur;       // the next chunk is fetched before the current one is processed
            if (c4 + 1 < R / 4) nxt = *reinterpret_cast<const float4 *>(tile + chunk_of<R>(lane, c4 + 1));
            float vv[4] = {cur.x, cur.y, cur.z, cur.w};
            float sv[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const bool spk = st.step(vv[j]);
                if (FLOATS) sv[j] = spk ? st.spikeVal : 0.0f;
                else if (spk) mask |= 1u << (c4 * 4 + j);
            }
            *reinterpret_cast<float4 *>(tile + chunk_of<R>(lane, c4)) = make_float4(vv[0], vv[1], vv[2], vv[3]);
            if (FLOATS)
                *reinterpret_cast<float4 *>(tile_s + chunk_of<R>(lane, c4)) = make_float4(sv[0], sv[1], sv[2], sv[3]);
            cur = nxt;
        }
    }
    return mask;
}

template <int R>
__device__ __forceinline__ void ring_reset(float (&ring)[R])
{
#pragma unroll
    for (int i = 0; i < R; ++i) ring[i] = 0.0f;
}

// ---------------------------------------------------------------------------------------
// cp.async path for buffers that are not 16-byte aligned.  V: global access width in floats
// (2 or 1; T % V == 0 and bases aligned to 4*V bytes).
// ---------------------------------------------------------------------------------------
template <int V, int NB, int W>
__global__ void __launch_bounds__(256)
srm_get_spikes_kernel(float *s, float *u, const float *__restrict__ nu,
                      int64_t rows, int nuEff, int T, float theta, float spikeVal, int depth)
{
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps_per_block = blockDim.x >> 5;
    const int nuPad = NB > 0 ? 0 : ((nuEff + 3) & ~3);
    float *nu_s = smem;
    // per warp: `depth` potential tiles (prefetch ring, depth = 2 or 4) and one spike tile
    float *tiles = smem + nuPad + warp * ((depth + 1) * kTileWords);
    float *tile_s = tiles + depth * kTileWords;

    if (NB == 0) {
        for (int i = threadIdx.x; i < nuEff; i += blockDim.x) nu_s[i] = nu[i];
        __syncthreads();
    }
    SrmRow<NB, W> st;
    st.init(nu, nu_s, nuEff, theta, spikeVal);
    constexpr bool kRingOk = NB > 0 && NB < kTile;
    const bool use_ring = kRingOk && st.taps_negative;      // uniform over the grid
    float ring[kTile];

    // The warp's work is one stream of tiles: all time tiles of its first block of 32 rows, then
    // of its next block, ...  The depth-1 tiles after the current one - possibly the first tiles
    // of the next row block - are always in flight, so a change of row block costs no memory
    // latency.  Large launches hide latency with many resident warps and use depth 2; launches
    // with only a few warps per SM use depth 4 (more shared memory per warp, fewer stalls).
    static_assert(V == 1 || V == 2, "aligned buffers take the wide-tile or the bulk-tensor kernel");
    const int ntiles = (T + kTile - 1) / kTile;
    const int64_t nblocks = (rows + kTile - 1) / kTile;
    const int64_t wstride = (int64_t)gridDim.x * warps_per_block;
    int64_t rb = (int64_t)blockIdx.x * warps_per_block + warp;
    if (rb >= nblocks) return;
    int64_t rb_next = rb;           // (row block, tile) of the tile to prefetch next
    int it_next = 0;
    unsigned q = 0;                 // tiles walked so far: buffer = q & (depth - 1)
    const unsigned dmask = (unsigned)depth - 1u;

    auto prefetch = [&](float *dst) {
        tile_prefetch<V>(dst, u, rb_next * kTile, rows, it_next * kTile, T, lane);
        if (++it_next == ntiles) {
            it_next = 0;
            rb_next += wstride;
        }
    };
    for (int d = 0; d + 1 < depth; ++d) {
        if (rb_next < nblocks) prefetch(tiles + d * kTileWords);
        cp_async_commit();
    }

    for (int it = 0; rb < nblocks; ++q) {
        const int64_t row0 = rb * kTile;
        float *tile = tiles + (q & dmask) * kTileWords;
        if (it == 0) {
            st.reset();
            ring_reset(ring);
        }
        if (rb_next < nblocks) prefetch(tiles + ((q + dmask) & dmask) * kTileWords);
        cp_async_commit();
        if (depth == 2) cp_async_wait<1>();
        else cp_async_wait<3>();
        __syncwarp();

        if (use_ring) walk_tile<kTile, kRingOk, NB, W>(tile, tile_s, st, ring, lane);
        else walk_tile<kTile, false, NB, W>(tile, tile_s, st, ring, lane);
        __syncwarp();

        tile_store<V>(tile, u, row0, rows, it * kTile, T, lane);
        tile_store<V>(tile_s, s, row0, rows, it * kTile, T, lane);
        __syncwarp();
        if (++it == ntiles) {
            it = 0;
            rb += wstride;
        }
    }
}

// ---------------------------------------------------------------------------------------
// Wide-tile path (16-byte aligned bases, any T): row-skewed tiles of 64 steps, so that every
// global request covers 256 contiguous bytes of a row, which is what DRAM needs to run near
// its peak.  Per warp: `depth` potential tiles (8 KB each) and the spike bits of the tile being
// walked (256 bytes); spikes are expanded to samples on their way out.  Samples before a row's
// start are padded with -inf, which can neither spike nor be changed by a refractory tap, so
// the skewed lanes idle through them with their state untouched.
// ---------------------------------------------------------------------------------------
template <int NB, int W, bool SKEW>
__global__ void __launch_bounds__(256)
srm_get_spikes_wide_kernel(float *s, float *u, const float *__restrict__ nu,
                           int64_t rows, int nuEff, int T, float theta, float spikeVal, int depth)
{
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps_per_block = blockDim.x >> 5;
    const int nuPad = NB > 0 ? 0 : ((nuEff + 3) & ~3);
    float *nu_s = smem;
    float *tiles = smem + nuPad + warp * (depth * kWideWords + 2 * kTile);
    unsigned *masks = reinterpret_cast<unsigned *>(tiles + depth * kWideWords);

    if (NB == 0) {
        for (int i = threadIdx.x; i < nuEff; i += blockDim.x) nu_s[i] = nu[i];
        __syncthreads();
    }
    SrmRow<NB, W> st;
    st.init(nu, nu_s, nuEff, theta, spikeVal);
    constexpr bool kRingOk = NB > 0 && NB < kTile;
    const bool use_ring = kRingOk && st.taps_negative;      // uniform over the grid
    float ring[kTile];

    const int ntiles = SKEW ? skew_wide_tiles(T) : (T + kWide - 1) / kWide;
    const unsigned phase = (unsigned)(reinterpret_cast<uintptr_t>(u) >> 2) & 7u;
    const int64_t nblocks = (rows + kTile - 1) / kTile;
    const int64_t wstride = (int64_t)gridDim.x * warps_per_block;
    int64_t rb = (int64_t)blockIdx.x * warps_per_block + warp;
    if (rb >= nblocks) return;
    int64_t rb_next = rb;           // (row block, tile) of the tile to prefetch next
    int it_next = 0;
    int skew = block_skew(rb * kTile, T, phase);          // of the block being walked
    int skew_next = skew;                                  // of the block being prefetched
    unsigned q = 0;                 // tiles walked so far: buffer = q & (depth - 1)
    const unsigned dmask = (unsigned)depth - 1u;

    auto prefetch = [&](float *dst) {
        wide_prefetch_skew<SKEW>(dst, u, rb_next * kTile, rows, it_next, T, lane, skew_next, -INFINITY);
        if (++it_next == ntiles) {
            it_next = 0;
            rb_next += wstride;
            if (rb_next < nblocks) skew_next = block_skew(rb_next * kTile, T, phase);
        }
    };
    for (int d = 0; d + 1 < depth; ++d) {
        if (rb_next < nblocks) prefetch(tiles + d * kWideWords);
        cp_async_commit();
    }

    for (int it = 0; rb < nblocks; ++q) {
        const int64_t row0 = rb * kTile;
        float *tile = tiles + (q & dmask) * kWideWords;
        if (it == 0) {
            st.reset();
            ring_reset(ring);
        }
        if (rb_next < nblocks) prefetch(tiles + ((q + dmask) & dmask) * kWideWords);
        cp_async_commit();
        if (depth == 2) cp_async_wait<1>();
        else cp_async_wait<3>();
        __syncwarp();

        // the second half lies wholly past the end of every row when even the most skewed row
        // (7 steps behind) has run out of samples there
        const bool second = kWide * it + kTile - (SKEW ? 7 : 0) < T;
        unsigned m0 = 0u, m1 = 0u;
#pragma unroll 1
        for (int h = 0; h < (second ? 2 : 1); ++h) {
            const unsigned mh = use_ring
                ? walk_tile<kTile, kRingOk, NB, W, false>(tile + h * kTileWords, nullptr, st, ring, lane)
                : walk_tile<kTile, false, NB, W, false>(tile + h * kTileWords, nullptr, st, ring, lane);
            if (h == 0) m0 = mh;
            else m1 = mh;
        }
        masks[lane] = m0;
        masks[kTile + lane] = m1;
        __syncwarp();

        wide_store_skew<SKEW>(tile, u, row0, rows, it, T, lane, skew);
        wide_store_spikes_skew<SKEW>(masks, s, row0, rows, it, T, lane, skew, spikeVal);
        __syncwarp();
        if (++it == ntiles) {
            it = 0;
            rb += wstride;
            if (rb < nblocks) skew = block_skew(rb * kTile, T, phase);
        }
    }
}

// ---------------------------------------------------------------------------------------
// Bulk-tensor-copy path (T % 4 == 0, 16-byte aligned bases).  The potentials arrive as
// [32 rows x 32 steps] boxes requested by one lane per warp, so loading costs the warp no
// issue slots.  A stage is a wide tile: two boxes that are adjacent in time.  Boxes use the
// 128-byte swizzle, which is the layout of the 32-step tile (tile.cuh): a lane reading its own
// row's 16-byte chunks is bank-conflict free.  Results leave as ordinary 16-byte stores that
// cover 256 contiguous bytes of a row per 16 lanes (the updated potentials from the tile, the
// spikes expanded from bit masks): DRAM runs measurably closer to its peak on 256-byte row
// segments than on the 128-byte segments of a box, and writes are two thirds of the traffic.
// Per warp: `ustages` stages (one being walked, the others being loaded) and the spike bits
// of the tile being walked.
// Every wait on a load barrier is bounded: if it runs out the warp records a status code and
// stops, so a lost copy cannot hang the GPU.
// ---------------------------------------------------------------------------------------
constexpr int kBoxT = kTile;                    // time steps per box
constexpr int kBoxBytes = kTileWords * 4;       // 4 KB
constexpr int kStageBytes = 2 * kBoxBytes;      // one wide tile
constexpr int kUStages = 3;                     // stages per warp in large launches
constexpr int kMaxUStages = 8;
// stages per warp in large launches of the allocating entry points (2 or 3; a tuning switch)
static std::atomic<int> g_srm_stages{kUStages};
constexpr int kLoadPollLimit = 1 << 22;         // polls of a load barrier before giving up

// dynamic shared memory of a launch with `warps` warps per CTA and `ustages` stages per warp
// mask_tiles: wide tiles whose spike bits a warp keeps (1, or all tiles of a row for the
// delayed-output variant)
constexpr int kRowMaskStride = kTile + 1;       // words between consecutive mask words of the whole-row bits
static inline size_t srm_tma_smem(int warps, int ustages, int nuEff, bool taps_in_smem, int mask_tiles = 1)
{
    return 1024 + (size_t)warps * ((size_t)ustages * kStageBytes + (size_t)mask_tiles * 2 * kRowMaskStride * sizeof(unsigned)
                                   + ustages * sizeof(uint64_t))
         + (taps_in_smem ? (size_t)((nuEff + 3) & ~3) * sizeof(float) : 0);
}

// What the delayed-output variant needs to know about the delay that follows the spikes.
struct DelayArgs {
    float *out;                 // delayed spikes
    const float *lut;           // one delay per neuron, or NULL
    float shift;                // the delay of every row when lut is NULL
    float Ts;
    int64_t nNeurons;
};

// Shared-memory word offsets of a lane's 16-byte chunk in the rows it visits when it drains a
// wide tile, two rows per pass (row = 2 * pass + rsub): the swizzle term depends on the pass
// only through (2 * pass) & 7, so four offsets cover all sixteen passes and the row term is a
// compile-time constant per pass.
struct DrainLane {
    int c16, rsub;
    int sw[4];                  // word offset inside the half for pass & 3 = 0..3, without the row term
    __device__ __forceinline__ explicit DrainLane(int lane)
    {
        c16 = lane & 15;
        rsub = lane >> 4;
        const int cq = c16 & 7;
#pragma unroll
        for (int k = 0; k < 4; ++k) sw[k] = (c16 >> 3) * kTileWords + rsub * kTile + ((cq ^ ((2 * k + rsub) & 7)) << 2);
    }
    // word offset of the chunk in row 2 * pass + rsub (pass is a compile-time constant at the call)
    __device__ __forceinline__ int word(int pass) const { return 2 * pass * kTile + sw[pass & 3]; }
};

// Potentials of an unskewed wide tile starting at time t0 (T % 4 == 0).
// `changed`: bit r set = row r of the tile differs from what was loaded; the other rows are in
// global memory already (the potential is updated in place) and are not written again.
__device__ __forceinline__ void wide_store(const float *tile, float *g, int64_t row0, int64_t rows,
                                           int t0, int T, int lane, unsigned changed)
{
    const DrainLane dl(lane);
    const int t = t0 + dl.c16 * 4;
    if (t >= T) return;
    const int64_t nrow = rows - row0;
    if (nrow < kTile) changed &= (1u << (int)nrow) - 1u;         // rows past the end of the array
    changed >>= dl.rsub;
    float *dst = g + (row0 + dl.rsub) * (int64_t)T + t;
    const int64_t pitch = 2 * (int64_t)T;
#pragma unroll
    for (int i = 0; i < kTile / 2; ++i) {
        if ((changed >> (2 * i)) & 1u)
            *reinterpret_cast<float4 *>(dst) = *reinterpret_cast<const float4 *>(tile + dl.word(i));
        dst += pitch;
    }
}

// Spike samples of an unskewed wide tile starting at time t0 (T % 4 == 0), from bit masks.
__device__ __forceinline__ void wide_store_spikes(const unsigned *masks, float *g, int64_t row0, int64_t rows,
                                                  int t0, int T, int lane, float value)
{
    const int c16 = lane & 15;
    const int rsub = lane >> 4;
    const int t = t0 + c16 * 4;
    if (t >= T) return;
    const unsigned *half = masks + (c16 >> 3) * kTile + rsub;
    const int sh = (c16 & 7) * 4;
    const int64_t nrow = rows - row0;
    float *dst = g + (row0 + rsub) * (int64_t)T + t;
    const int64_t pitch = 2 * (int64_t)T;
    const bool full = nrow >= kTile;
#pragma unroll
    for (int i = 0; i < kTile / 2; ++i) {
        if (full || i * 2 + rsub < nrow) {
            const unsigned m = half[2 * i] >> sh;
            *reinterpret_cast<float4 *>(dst) =
                make_float4((m & 1u) ? value : 0.0f, (m & 2u) ? value : 0.0f,
                            (m & 4u) ? value : 0.0f, (m & 8u) ? value : 0.0f);
        }
        dst += pitch;
    }
}

// Delayed spike samples of a block of 32 rows from the spike bits of the whole rows:
// out[r, t] = value if row r spiked at t - d_r (0 <= t - d_r < T), else 0.  masks is word-major
// ([word][row] with kRowMaskStride words per mask word, nwords words per row, bits past T
// clear); lane l holds d of row l.
__device__ __forceinline__ void store_delayed_spikes(const unsigned *masks, int nwords, float *g, int64_t row0,
                                                     int64_t rows, int T, int lane, int d_lane, float value)
{
    const int c16 = lane & 15;
    const int rsub = lane >> 4;
    const int64_t nrow = rows - row0;
    const int T4 = T >> 2;
    for (int q0 = 0; q0 < T4; q0 += 16) {
        const int q = q0 + c16;
#pragma unroll 4
        for (int i = 0; i < kTile / 2; ++i) {
            const int r = i * 2 + rsub;
            const int d = __shfl_sync(0xffffffffu, d_lane, r);
            if (q >= T4 || r >= nrow) continue;
            const int64_t src = (int64_t)4 * q - d;              // time of the first source sample
            unsigned m = 0u;
            if (src > -4 && src < T) {
                const int w = (int)(src >> 5), off = (int)(src & 31);
                const unsigned lo = (w >= 0 && w < nwords) ? masks[w * kRowMaskStride + r] : 0u;
                const unsigned hi = (w + 1 >= 0 && w + 1 < nwords) ? masks[(w + 1) * kRowMaskStride + r] : 0u;
                m = __funnelshift_r(lo, hi, off);
            }
            *reinterpret_cast<float4 *>(g + (row0 + r) * (int64_t)T + 4 * q) =
                make_float4((m & 1u) ? value : 0.0f, (m & 2u) ? value : 0.0f,
                            (m & 4u) ? value : 0.0f, (m & 8u) ? value : 0.0f);
        }
    }
}

// PER_BLOCK selects where a wait that ran out is recorded: false = the single status word of
// the device (`status` points to one int); true = one int per block of 32 rows (`status` points
// to an array with an entry for every row block), which the warp clears when it starts the
// block and sets to the number of tiles walked when it finishes it.
//
// DELAYED: the spikes are not written where they occur but shifted by a per-row delay, which is
// what an axonal delay right after the spike function does (out[t] = s[t - d], zero filled).
// The warp keeps the spike bits of the whole row (T / 32 words per row) in shared memory and
// writes the shifted samples when it has walked the row, so any delay - positive, negative,
// beyond the row - costs the same and the undelayed spikes never reach global memory.
//
// PACKED: the spikes leave as bits, not as fp32 samples: `s` then points to 32-bit words,
// ceil(T / 32) per row, bit i of word w = "spiked at step 32 w + i" (bits past T are zero).  The
// warp already holds exactly these words after walking a tile, so each lane stores the two words
// of its row; the spike output shrinks from 4 bytes to 1/8 byte per element.
template <int NB, int W, bool PER_BLOCK = false, bool DELAYED = false, bool PACKED = false>
__global__ void __launch_bounds__(256)
srm_get_spikes_tma_kernel(const __grid_constant__ CUtensorMap map_u, float *__restrict__ s, float *u,
                          const float *__restrict__ nu, int64_t rows, int nuEff, int T,
                          float theta, float spikeVal, int *status, int ustages, DelayArgs da)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps_per_block = blockDim.x >> 5;
    // the swizzle pattern repeats every 1 KB: align the tiles to that
    unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    float *u_tiles = reinterpret_cast<float *>(base) + (size_t)warp * ustages * kWideWords;
    unsigned char *after_tiles = base + (size_t)warps_per_block * ustages * kStageBytes;
    const int ntiles = (T + kWide - 1) / kWide;
    // per warp; word-major [word][row], one word of padding per mask word so that a lane group
    // reading consecutive words of one row hits different banks
    const int mask_words = (DELAYED ? ntiles : 1) * 2 * kRowMaskStride;
    unsigned *masks = reinterpret_cast<unsigned *>(after_tiles) + warp * mask_words;
    uint64_t *bars = reinterpret_cast<uint64_t *>(after_tiles + warps_per_block * mask_words * sizeof(unsigned))
                     + warp * ustages;
    float *nu_s = reinterpret_cast<float *>(reinterpret_cast<uint64_t *>(
                      after_tiles + warps_per_block * mask_words * sizeof(unsigned)) + warps_per_block * ustages);

    if (NB == 0) {
        for (int i = threadIdx.x; i < nuEff; i += blockDim.x) nu_s[i] = nu[i];
    }
    if (lane == 0) {
        for (int i = 0; i < ustages; ++i) mbar_init(bars + i, 1);
        mbar_init_fence();
    }
    __syncthreads();

    SrmRow<NB, W> st;
    st.init(nu, nu_s, nuEff, theta, spikeVal);
    constexpr bool kRingOk = NB > 0 && NB < kTile;
    const bool use_ring = kRingOk && st.taps_negative;      // uniform over the grid
    float ring[kTile];

    // The warp's work is one stream of wide tiles: all of its first block of 32 rows, then of
    // its next block, ...  Loads run ustages - 1 tiles ahead of the walk across row-block
    // boundaries, so a change of row block costs no memory latency.
    const int64_t nblocks = (rows + kTile - 1) / kTile;
    const int64_t wstride = (int64_t)gridDim.x * warps_per_block;
    int64_t rb = (int64_t)blockIdx.x * warps_per_block + warp;
    int64_t rb_next = rb;           // (row block, tile) of the next tile to load
    int j_next = 0;
    int sg_next = 0;                // stage the next load goes to
    int inflight = 0;               // lane 0: loads issued and not yet waited for
    int delay_steps = 0;            // DELAYED: the delay of this lane's row, in steps
    unsigned long long prev_bits = 0ull;    // spike bits of the previous tile of this lane's row
    auto issue_load = [&]() {       // lane 0 only
        const bool two = kWide * j_next + kBoxT < T;           // the second box starts inside the rows
        float *dst = u_tiles + sg_next * kWideWords;
        mbar_expect_tx(bars + sg_next, two ? kStageBytes : kBoxBytes);
        tma_load_2d(dst, &map_u, kWide * j_next, (int)(rb_next * kTile), bars + sg_next);
        if (two) tma_load_2d(dst + kTileWords, &map_u, kWide * j_next + kBoxT, (int)(rb_next * kTile), bars + sg_next);
        if (++sg_next == ustages) sg_next = 0;
        if (++j_next == ntiles) { j_next = 0; rb_next += wstride; }
        ++inflight;
    };
    if (lane == 0) {
        for (int i = 0; i + 1 < ustages; ++i)
            if (rb_next < nblocks) issue_load();
    }
    int j = 0;
    int sg = 0;                     // stage of the tile being walked
    unsigned parity = 0u;           // barrier phase of that stage
    while (rb < nblocks) {
        float *tile = u_tiles + sg * kWideWords;
        if (j == 0) {
            st.reset();
            ring_reset(ring);
            if (PER_BLOCK && lane == 0) status[rb] = 0;
            if (DELAYED) {
                const int64_t row = rb * kTile + lane;
                delay_steps = shift_steps(da.lut ? __ldg(da.lut + (row % da.nNeurons)) : da.shift, da.Ts);
            }
        }
        // the stage walked before this one was drained (and fenced) at the end of its iteration
        if (lane == 0 && rb_next < nblocks) issue_load();
        const bool ok = mbar_wait_bounded(bars + sg, parity, kLoadPollLimit);
        if (__any_sync(0xffffffffu, !ok)) {
            if (lane == 0) {
                if (PER_BLOCK) status[rb] = -kStatusSrmLoadTimeout;
                else atomicExch(status, kStatusSrmLoadTimeout);
                // the loads issued after the lost one may still be writing into this warp's
                // stages: give each of them the same bounded wait before the warp leaves
                for (int i = 1; i < inflight; ++i) {
                    const int stage = sg + i < ustages ? sg + i : sg + i - ustages;
                    (void)mbar_wait_bounded(bars + stage, sg + i < ustages ? parity : parity ^ 1u, kLoadPollLimit);
                }
            }
            __syncwarp();
            break;
        }
        if (lane == 0) --inflight;

        const bool two = kWide * j + kBoxT < T;
        if (j == 0) prev_bits = 0ull;
        unsigned m[2] = {0u, 0u};
#pragma unroll 1
        for (int h = 0; h < (two ? 2 : 1); ++h) {
            const unsigned mh = use_ring
                ? walk_tile<kTile, kRingOk, NB, W, false>(tile + h * kTileWords, nullptr, st, ring, lane)
                : walk_tile<kTile, false, NB, W, false>(tile + h * kTileWords, nullptr, st, ring, lane);
            if (h == 0) m[0] = mh;
            else m[1] = mh;
        }
        if (DELAYED || PACKED) {
            // bits of steps past the row end must read as zero
            const int left = T - kWide * j;                  // > 0
            if (left < kTile) m[0] &= (1u << left) - 1u;
            if (left < kWide) m[1] &= left > kTile ? (1u << (left - kTile)) - 1u : 0u;
        }
        if (PACKED) {
            const int64_t row = rb * kTile + lane;
            const int words = (T + 31) >> 5;
            if (row < rows) {
                unsigned *dst = reinterpret_cast<unsigned *>(s) + row * words + 2 * j;
                dst[0] = m[0];
                if (2 * j + 1 < words) dst[1] = m[1];
            }
        } else if (DELAYED) {
            // keep the bits of the whole row
            masks[(2 * j) * kRowMaskStride + lane] = m[0];
            masks[(2 * j + 1) * kRowMaskStride + lane] = m[1];
        } else {
            masks[lane] = m[0];
            masks[kTile + lane] = m[1];
        }
        __syncwarp();
        // A row's potentials change in this tile only if it spikes here or a spike of the last
        // nuEff - 1 steps before the tile still reaches into it (spikes further back than the
        // previous tile: assume they do).
        const unsigned long long cur_bits = ((unsigned long long)m[1] << 32) | m[0];
        const int reach = nuEff - 1;
        const bool row_changed = cur_bits != 0ull || reach > kWide ||
                                 (reach > 0 && (prev_bits >> (kWide - reach)) != 0ull);
        prev_bits = cur_bits;
        wide_store(tile, u, rb * kTile, rows, kWide * j, T, lane, __ballot_sync(0xffffffffu, row_changed));
        if (!DELAYED && !PACKED) wide_store_spikes(masks, s, rb * kTile, rows, kWide * j, T, lane, spikeVal);
        if (DELAYED && j == ntiles - 1)
            store_delayed_spikes(masks, 2 * ntiles, da.out, rb * kTile, rows, T, lane, delay_steps, spikeVal);
        // the reads of this stage (and of the masks) precede the bulk load that refills it
        fence_proxy_async();
        __syncwarp();

        if (++sg == ustages) { sg = 0; parity ^= 1u; }
        if (++j == ntiles) {
            if (PER_BLOCK && lane == 0) status[rb] = ntiles;
            j = 0;
            rb += wstride;
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
    bool use_tma;
};

template <int V, int NB, int W>
static int launch_srm(const SrmArgs &a)
{
    const int64_t nblocks = ceil_div(a.rows, kTile);
    int warps, grid;
    // Rows on 16-byte boundaries (T % 4 == 0): bulk tensor copies move the potentials, which
    // leaves the warps' issue slots to the recurrence.  Any other row length: the wide-tile
    // kernel with row-skewed cp.async tiles.
    if (V == 4 && a.use_tma && (a.T & 3) == 0) {
        CUtensorMap map_u;
        int *status = device_status_word();
        if (status && a.rows * (int64_t)kTile < (1LL << 31) &&
            encode_rows_tensor_map(&map_u, a.u, a.rows, a.T, kBoxT, kTile, CU_TENSOR_MAP_SWIZZLE_128B)) {
            // stages per warp: as many (up to 8) as still let every warp of the launch be resident
            const int sms = sm_count();
            const int64_t warps_per_sm = ceil_div(nblocks, sms);
            int ustages = (int)((208 * 1024) / (warps_per_sm * kStageBytes));
            if (ustages > kMaxUStages) ustages = kMaxUStages;
            if (ustages < g_srm_stages.load()) ustages = g_srm_stages.load();
            spike_launch_shape(nblocks, (size_t)ustages * kStageBytes + 512, warps, grid);
            const size_t smem = srm_tma_smem(warps, ustages, a.nuEff, NB == 0);
            auto kern = srm_get_spikes_tma_kernel<NB, W>;
            int rc = reserve_dynamic_smem((const void *)kern, smem);
            if (rc) return rc;
            kern<<<(unsigned)grid, warps * 32, smem, a.stream>>>(map_u, a.s, a.u, a.nu, a.rows, a.nuEff, a.T, a.theta,
                                                                 a.spikeVal, status, ustages, DelayArgs{});
            return check_launch("srm_get_spikes (bulk tensor copy) kernel launch");
        }
    }
    const size_t nu_bytes = (size_t)(NB > 0 ? 0 : ((a.nuEff + 3) & ~3)) * sizeof(float);
    if constexpr (V == 4) {
        // prefetch depth 4 when every warp of the launch is resident at once even with the
        // larger footprint (then latency, not bandwidth, bounds the launch), depth 2 otherwise
        const size_t deep_bytes = (4 * kWideWords + 2 * kTile) * sizeof(float);
        const int depth = nblocks <= (int64_t)((216 * 1024) / deep_bytes) * sm_count() ? 4 : 2;
        const size_t warp_bytes = (size_t)(depth * kWideWords + 2 * kTile) * sizeof(float);
        spike_launch_shape(nblocks, warp_bytes, warps, grid);
        const size_t smem = nu_bytes + warps * warp_bytes;
        // rows that start on 32-byte boundaries need no skew
        const bool skew = (a.T & 7) != 0 || (reinterpret_cast<uintptr_t>(a.u) & 31u) != 0;
        auto kern = skew ? srm_get_spikes_wide_kernel<NB, W, true> : srm_get_spikes_wide_kernel<NB, W, false>;
        int rc = reserve_dynamic_smem((const void *)kern, smem);
        if (rc) return rc;
        kern<<<(unsigned)grid, warps * 32, smem, a.stream>>>(a.s, a.u, a.nu, a.rows, a.nuEff, a.T, a.theta, a.spikeVal, depth);
        return check_launch("srm_get_spikes (wide tile) kernel launch");
    } else {
        const int64_t deep_warps_per_sm = (216 * 1024) / (5 * kTileWords * (int64_t)sizeof(float));
        const int depth = nblocks <= deep_warps_per_sm * sm_count() ? 4 : 2;
        spike_launch_shape(nblocks, (depth + 1) * kTileWords * sizeof(float), warps, grid);
        const size_t smem = nu_bytes + (size_t)warps * (depth + 1) * kTileWords * sizeof(float);
        auto kern = srm_get_spikes_kernel<V, NB, W>;
        int rc = reserve_dynamic_smem((const void *)kern, smem);
        if (rc) return rc;
        kern<<<(unsigned)grid, warps * 32, smem, a.stream>>>(a.s, a.u, a.nu, a.rows, a.nuEff, a.T, a.theta, a.spikeVal, depth);
        return check_launch("srm_get_spikes kernel launch");
    }
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

// Spikes written already delayed (slayer_b200_srm_get_spikes_delayed): the bulk-tensor kernel
// with the spike bits of whole rows kept in shared memory.  Needs what that kernel needs
// (T % 4 == 0, 16-byte aligned buffers) and rows short enough for the bits to fit.
constexpr int kDelayedMaxTiles = 32;            // T <= 2048

template <int NB, int W>
static int launch_srm_delayed(const SrmArgs &a, const DelayArgs &da)
{
    const int64_t nblocks = ceil_div(a.rows, kTile);
    const int ntiles = (int)ceil_div((int64_t)a.T, (int64_t)kWide);
    CUtensorMap map_u;
    int *status = device_status_word();
    if (!status || a.rows * (int64_t)kTile >= (1LL << 31) ||
        !encode_rows_tensor_map(&map_u, a.u, a.rows, a.T, kBoxT, kTile, CU_TENSOR_MAP_SWIZZLE_128B)) {
        set_error("srm_get_spikes_delayed: cannot describe the buffers for bulk tensor copies");
        return SLAYER_B200_EUNSUPPORTED;
    }
    const int sms = sm_count();
    const size_t mask_bytes = (size_t)ntiles * 2 * kRowMaskStride * sizeof(unsigned);
    const int64_t warps_per_sm = ceil_div(nblocks, (int64_t)sms);
    int ustages = (int)(((208 * 1024) / warps_per_sm - (int64_t)mask_bytes) / kStageBytes);
    if (ustages > kMaxUStages) ustages = kMaxUStages;
    if (ustages < g_srm_stages.load()) ustages = g_srm_stages.load();
    int warps, grid;
    spike_launch_shape(nblocks, (size_t)ustages * kStageBytes + mask_bytes + 256, warps, grid);
    const size_t smem = srm_tma_smem(warps, ustages, a.nuEff, NB == 0, ntiles);
    auto kern = srm_get_spikes_tma_kernel<NB, W, false, true>;
    int rc = reserve_dynamic_smem((const void *)kern, smem);
    if (rc) return rc;
    kern<<<(unsigned)grid, warps * 32, smem, a.stream>>>(map_u, nullptr, a.u, a.nu, a.rows, a.nuEff, a.T, a.theta,
                                                         a.spikeVal, status, ustages, da);
    return check_launch("srm_get_spikes_delayed kernel launch");
}

static int dispatch_srm_delayed(const SrmArgs &a, const DelayArgs &da)
{
    const int window = a.nuEff > 1 ? a.nuEff - 1 : 0;     // history bits needed
    if (window <= 2) return launch_srm_delayed<2, 1>(a, da);
    if (window <= 4) return launch_srm_delayed<4, 1>(a, da);
    if (window <= 6) return launch_srm_delayed<6, 1>(a, da);
    if (window <= 8) return launch_srm_delayed<8, 1>(a, da);
    if (window <= 10) return launch_srm_delayed<10, 1>(a, da);
    if (window <= 12) return launch_srm_delayed<12, 1>(a, da);
    if (window <= 16) return launch_srm_delayed<16, 1>(a, da);
    if (window <= 24) return launch_srm_delayed<24, 1>(a, da);
    if (window <= 32) return launch_srm_delayed<32, 1>(a, da);
    if (window <= 64) return launch_srm_delayed<0, 2>(a, da);
    if (window <= 128) return launch_srm_delayed<0, 4>(a, da);
    return launch_srm_delayed<0, 8>(a, da);
}

// Spikes written as bits (slayer_b200_srm_get_spikes_packed): the bulk-tensor kernel with its
// spike output replaced by two word stores per row and tile.
template <int NB, int W>
static int launch_srm_packed(const SrmArgs &a)
{
    const int64_t nblocks = ceil_div(a.rows, kTile);
    CUtensorMap map_u;
    int *status = device_status_word();
    if (!status || a.rows * (int64_t)kTile >= (1LL << 31) ||
        !encode_rows_tensor_map(&map_u, a.u, a.rows, a.T, kBoxT, kTile, CU_TENSOR_MAP_SWIZZLE_128B)) {
        set_error("srm_get_spikes_packed: cannot describe the buffers for bulk tensor copies");
        return SLAYER_B200_EUNSUPPORTED;
    }
    const int sms = sm_count();
    const int64_t warps_per_sm = ceil_div(nblocks, sms);
    int ustages = (int)((208 * 1024) / (warps_per_sm * kStageBytes));
    if (ustages > kMaxUStages) ustages = kMaxUStages;
    if (ustages < g_srm_stages.load()) ustages = g_srm_stages.load();
    int warps, grid;
    spike_launch_shape(nblocks, (size_t)ustages * kStageBytes + 512, warps, grid);
    const size_t smem = srm_tma_smem(warps, ustages, a.nuEff, NB == 0);
    auto kern = srm_get_spikes_tma_kernel<NB, W, false, false, true>;
    int rc = reserve_dynamic_smem((const void *)kern, smem);
    if (rc) return rc;
    kern<<<(unsigned)grid, warps * 32, smem, a.stream>>>(map_u, a.s, a.u, a.nu, a.rows, a.nuEff, a.T, a.theta,
                                                         a.spikeVal, status, ustages, DelayArgs{});
    return check_launch("srm_get_spikes_packed kernel launch");
}

static int dispatch_srm_packed(const SrmArgs &a)
{
    const int window = a.nuEff > 1 ? a.nuEff - 1 : 0;     // history bits needed
    if (window <= 2) return launch_srm_packed<2, 1>(a);
    if (window <= 4) return launch_srm_packed<4, 1>(a);
    if (window <= 6) return launch_srm_packed<6, 1>(a);
    if (window <= 8) return launch_srm_packed<8, 1>(a);
    if (window <= 10) return launch_srm_packed<10, 1>(a);
    if (window <= 12) return launch_srm_packed<12, 1>(a);
    if (window <= 16) return launch_srm_packed<16, 1>(a);
    if (window <= 24) return launch_srm_packed<24, 1>(a);
    if (window <= 32) return launch_srm_packed<32, 1>(a);
    if (window <= 64) return launch_srm_packed<0, 2>(a);
    if (window <= 128) return launch_srm_packed<0, 4>(a);
    return launch_srm_packed<0, 8>(a);
}

// ---------------------------------------------------------------------------------------
// Entry point that allocates nothing (slayer_b200_srm_get_spikes_noalloc).
//
// The bulk-tensor kernel needs a little global memory of its own to leave a trace when a wait
// runs out.  The regular entry point gets that word from cudaMalloc the first time a device is
// used.  Some callers must not allocate device memory at all - a host application that has
// handed all of its device memory to its own pool, code running where the allocator may not be
// entered (inside another library's callback, or after the process has frozen its memory
// footprint) - so this variant keeps its scratch in a fixed array that is part of the loaded
// library image: one int per block of 32 rows, kNoAllocMaxRowBlocks of them (256 KB, held by
// every GPU that loads the library until the process exits).
//
// In host code the array's name is only a handle; the device address is obtained once per
// device with cudaGetSymbolAddress while that device is current, and that address is what the
// kernel receives.
// ---------------------------------------------------------------------------------------
constexpr int kNoAllocMaxRowBlocks = 65536;                 // 2,097,152 rows
static __device__ __align__(256) int g_noalloc_block_status[kNoAllocMaxRowBlocks];

struct NoAllocDevice {
    bool ready;
    int *scratch;            // device address of g_noalloc_block_status on this device
};
static NoAllocDevice g_noalloc_dev[64];
static std::mutex g_noalloc_mu;

// Raise the shared-memory limit of one instantiation to the largest request any of its launches
// can make (8 warps, 257 taps).  Setting the attribute also loads the kernel's code onto the
// device, so after the set-up no later call has anything left to load.
template <int NB, int W>
static cudaError_t noalloc_prepare_one()
{
    const int most = (int)srm_tma_smem(8, kUStages, 260, true);
    return cudaFuncSetAttribute(srm_get_spikes_tma_kernel<NB, W, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
}

static cudaError_t noalloc_prepare_all()
{
    cudaError_t e;
    if ((e = noalloc_prepare_one<2, 1>()) != cudaSuccess) return e;
    if ((e = noalloc_prepare_one<4, 1>()) != cudaSuccess) return e;
    if ((e = noalloc_prepare_one<6, 1>()) != cudaSuccess) return e;
    if ((e = noalloc_prepare_one<8, 1>()) != cudaSuccess) return e;
    if ((e = noalloc_prepare_one<10, 1>()) != cudaSuccess) return e;
    if ((e = noalloc_prepare_one<12, 1>()) != cudaSuccess) return e;
    if ((e = noalloc_prepare_one<16, 1>()) != cudaSuccess) return e;
    if ((e = noalloc_prepare_one<24, 1>()) != cudaSuccess) return e;
    if ((e = noalloc_prepare_one<32, 1>()) != cudaSuccess) return e;
    if ((e = noalloc_prepare_one<0, 2>()) != cudaSuccess) return e;
    if ((e = noalloc_prepare_one<0, 4>()) != cudaSuccess) return e;
    return noalloc_prepare_one<0, 8>();
}

template <int NB, int W>
static int launch_srm_noalloc(const SrmArgs &a, NoAllocDevice &dev)
{
    const int64_t nblocks = ceil_div(a.rows, kTile);
    CUtensorMap map_u;
    if (!encode_rows_tensor_map(&map_u, a.u, a.rows, a.T, kBoxT, kTile, CU_TENSOR_MAP_SWIZZLE_128B)) {
        set_error("srm_get_spikes_noalloc: cannot describe the buffers for bulk tensor copies");
        return SLAYER_B200_EUNSUPPORTED;
    }
    int warps, grid;
    spike_launch_shape(nblocks, (size_t)kUStages * kStageBytes + 512, warps, grid);
    const size_t smem = srm_tma_smem(warps, kUStages, a.nuEff, NB == 0);
    auto kern = srm_get_spikes_tma_kernel<NB, W, true>;
    kern<<<(unsigned)grid, warps * 32, smem, a.stream>>>(map_u, a.s, a.u, a.nu, a.rows, a.nuEff, a.T, a.theta,
                                                         a.spikeVal, dev.scratch, kUStages, DelayArgs{});
    return check_launch("srm_get_spikes_noalloc kernel launch");
}

}  // namespace sb200

extern "C" int slayer_b200_srm_get_spikes_noalloc(float *s, float *u, const float *nu,
                                                  int64_t rows, int64_t nuSize, int64_t T,
                                                  float theta, float Ts, void *stream_)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(rows >= 0 && nuSize >= 0 && T >= 0, "srm_get_spikes_noalloc: negative size");
    if (rows == 0 || T == 0) return SLAYER_B200_OK;
    SB200_REQUIRE(s && u && (nu || nuSize == 0), "srm_get_spikes_noalloc: null pointer");
    SB200_REQUIRE(s != u, "srm_get_spikes_noalloc: s must not alias u");
    const int64_t nblocks = ceil_div(rows, kTile);
    if (nblocks > kNoAllocMaxRowBlocks) {
        set_error("srm_get_spikes_noalloc: %lld rows exceed the %lld this entry point has scratch for",
                  (long long)rows, (long long)kNoAllocMaxRowBlocks * kTile);
        return SLAYER_B200_EUNSUPPORTED;
    }
    const int64_t nuEff = nuSize < T ? nuSize : T;
    if (T >= (1LL << 31) - 64 || (T & 3) || !aligned16(s) || !aligned16(u) || nuEff - 1 > 32 * kMaxHistWords) {
        set_error("srm_get_spikes_noalloc: needs T %% 4 == 0, 16-byte aligned buffers and at most %d taps",
                  32 * kMaxHistWords + 1);
        return SLAYER_B200_EUNSUPPORTED;
    }

    // set-up, once per device, with that device current
    int d = 0;
    cudaError_t e = cudaGetDevice(&d);
    if (e != cudaSuccess || d < 0 || d >= 64) {
        set_error("srm_get_spikes_noalloc: no usable current device");
        return SLAYER_B200_ECUDA;
    }
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    NoAllocDevice &dev = g_noalloc_dev[d];
    if (!dev.ready) {
        int *ptr = nullptr;
        e = cudaGetSymbolAddress((void **)&ptr, g_noalloc_block_status);
        if (e != cudaSuccess || ptr == nullptr) {
            set_error("srm_get_spikes_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return SLAYER_B200_ECUDA;
        }
        e = noalloc_prepare_all();
        if (e != cudaSuccess) {
            set_error("srm_get_spikes_noalloc: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
            return SLAYER_B200_ECUDA;
        }
        dev.scratch = ptr;
        dev.ready = true;
    }

    const SrmArgs a = {s, u, nu, rows, (int)nuEff, (int)T, theta, 1.0f / Ts, (cudaStream_t)stream_, true};
    const int window = a.nuEff > 1 ? a.nuEff - 1 : 0;
    if (window <= 2) return launch_srm_noalloc<2, 1>(a, dev);
    if (window <= 4) return launch_srm_noalloc<4, 1>(a, dev);
    if (window <= 6) return launch_srm_noalloc<6, 1>(a, dev);
    if (window <= 8) return launch_srm_noalloc<8, 1>(a, dev);
    if (window <= 10) return launch_srm_noalloc<10, 1>(a, dev);
    if (window <= 12) return launch_srm_noalloc<12, 1>(a, dev);
    if (window <= 16) return launch_srm_noalloc<16, 1>(a, dev);
    if (window <= 24) return launch_srm_noalloc<24, 1>(a, dev);
    if (window <= 32) return launch_srm_noalloc<32, 1>(a, dev);
    if (window <= 64) return launch_srm_noalloc<0, 2>(a, dev);
    if (window <= 128) return launch_srm_noalloc<0, 4>(a, dev);
    return launch_srm_noalloc<0, 8>(a, dev);
}

extern "C" int slayer_b200_srm_get_spikes_noalloc_status(int64_t rows, int64_t T, int64_t *first_bad_block)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(rows >= 0 && T >= 0, "srm_get_spikes_noalloc_status: negative size");
    if (first_bad_block) *first_bad_block = -1;
    if (rows == 0 || T == 0) return SLAYER_B200_OK;
    const int64_t nblocks = ceil_div(rows, kTile);
    SB200_REQUIRE(nblocks <= kNoAllocMaxRowBlocks, "srm_get_spikes_noalloc_status: %lld rows exceed the %lld the array covers",
                  (long long)rows, (long long)kNoAllocMaxRowBlocks * kTile);
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) {
        set_error("srm_get_spikes_noalloc_status: no usable current device");
        return SLAYER_B200_ECUDA;
    }
    const int *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mu);
        if (g_noalloc_dev[d].ready) scratch = g_noalloc_dev[d].scratch;
    }
    SB200_REQUIRE(scratch != nullptr, "srm_get_spikes_noalloc_status: slayer_b200_srm_get_spikes_noalloc has not run on this device");
    const int want = (int)ceil_div(T, (int64_t)kWide);        // wide tiles per row block
    int chunk[1024];                                           // on the stack: nothing is allocated
    for (int64_t b0 = 0; b0 < nblocks; b0 += 1024) {
        const int64_t n = nblocks - b0 < 1024 ? nblocks - b0 : 1024;
        cudaError_t e = cudaMemcpy(chunk, scratch + b0, (size_t)n * sizeof(int), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) {
            set_error("srm_get_spikes_noalloc_status: %s", cudaGetErrorString(e));
            return SLAYER_B200_ECUDA;
        }
        for (int64_t i = 0; i < n; ++i) {
            if (chunk[i] != want) {
                if (first_bad_block) *first_bad_block = b0 + i;
                set_error("srm_get_spikes_noalloc_status: row block %lld %s (entry %d, expected %d)", (long long)(b0 + i),
                          chunk[i] == -kStatusSrmLoadTimeout ? "gave up waiting for a load" : "did not finish",
                          chunk[i], want);
                return SLAYER_B200_EDEVICE;
            }
        }
    }
    return SLAYER_B200_OK;
}

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
    const SrmArgs a = {s, u, nu, rows, (int)nuEff, (int)T, theta, spikeVal, stream, tma_enabled()};
    // 16-byte aligned buffers: row-skewed 16-byte tiles (or bulk tensor copies when rows are
    // sector aligned); otherwise the widest access the alignment allows
    switch (all_aligned16({s, u}) ? 4 : tile_vec_width(T, {s, u})) {
        case 4: return dispatch_srm<4>(a);
        case 2: return dispatch_srm<2>(a);
        default: return dispatch_srm<1>(a);
    }
}

extern "C" int slayer_b200_srm_get_spikes_packed(uint32_t *bits, float *u, const float *nu,
                                                 int64_t rows, int64_t nuSize, int64_t T, float theta, void *stream_)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(rows >= 0 && nuSize >= 0 && T >= 0, "srm_get_spikes_packed: negative size");
    SB200_REQUIRE(T < (1LL << 31) - 64, "srm_get_spikes_packed: T=%lld too large", (long long)T);
    if (rows == 0 || T == 0) return SLAYER_B200_OK;
    SB200_REQUIRE(bits && u && (nu || nuSize == 0), "srm_get_spikes_packed: null pointer");
    SB200_REQUIRE((void *)bits != (void *)u, "srm_get_spikes_packed: bits must not alias u");
    const int64_t nuEff = nuSize < T ? nuSize : T;
    if ((T & 3) || !aligned16(u) || (reinterpret_cast<uintptr_t>(bits) & 3u) || nuEff - 1 > 32 * kMaxHistWords || !tma_enabled()) {
        set_error("srm_get_spikes_packed: needs T %% 4 == 0, a 16-byte aligned potential and at most %d taps; "
                  "otherwise run slayer_b200_srm_get_spikes and slayer_b200_pack_spikes", 32 * kMaxHistWords + 1);
        return SLAYER_B200_EUNSUPPORTED;
    }
    const SrmArgs a = {reinterpret_cast<float *>(bits), u, nu, rows, (int)nuEff, (int)T, theta, 1.0f, (cudaStream_t)stream_, true};
    return dispatch_srm_packed(a);
}

extern "C" int slayer_b200_shift_lut(float *out, const float *in, const float *lut,
                                     int64_t nBatch, int64_t nNeurons, int64_t T, float Ts, void *stream);
extern "C" int slayer_b200_shift_scalar(float *out, const float *in, float shift,
                                        int64_t rows, int64_t T, float Ts, void *stream);

extern "C" int slayer_b200_srm_get_spikes_delayed(float *delayed, float *s_scratch, float *u, const float *nu,
                                                  const float *shift_lut, float shift,
                                                  int64_t nBatch, int64_t nNeurons, int64_t nuSize, int64_t T,
                                                  float theta, float Ts, void *stream_)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(nBatch >= 0 && nNeurons >= 0 && nuSize >= 0 && T >= 0, "srm_get_spikes_delayed: negative size");
    SB200_REQUIRE(T < (1LL << 31) - 64, "srm_get_spikes_delayed: T=%lld too large", (long long)T);
    const int64_t rows = nBatch * nNeurons;
    if (rows == 0 || T == 0) return SLAYER_B200_OK;
    SB200_REQUIRE(delayed && u && (nu || nuSize == 0), "srm_get_spikes_delayed: null pointer");
    SB200_REQUIRE(delayed != u && s_scratch != u && s_scratch != delayed, "srm_get_spikes_delayed: buffers must not alias");
    const int64_t nuEff = nuSize < T ? nuSize : T;
    const bool fused = tma_enabled() && (T & 3) == 0 && aligned16(delayed) && aligned16(u) &&
                       nuEff - 1 <= 32 * kMaxHistWords && ceil_div(T, (int64_t)kWide) <= kDelayedMaxTiles;
    if (fused) {
        const SrmArgs a = {nullptr, u, nu, rows, (int)nuEff, (int)T, theta, 1.0f / Ts, (cudaStream_t)stream_, true};
        const DelayArgs da = {delayed, shift_lut, shift, Ts, shift_lut ? nNeurons : 1};
        const int rc = dispatch_srm_delayed(a, da);
        if (rc != SLAYER_B200_EUNSUPPORTED) return rc;
    }
    if (!s_scratch) {
        set_error("srm_get_spikes_delayed: these sizes need a scratch buffer for the undelayed spikes "
                  "(fused path: T %% 4 == 0, T <= %d, 16-byte aligned buffers)", kDelayedMaxTiles * kWide);
        return SLAYER_B200_EUNSUPPORTED;
    }
    int rc = slayer_b200_srm_get_spikes(s_scratch, u, nu, rows, nuSize, T, theta, Ts, stream_);
    if (rc) return rc;
    if (shift_lut) return slayer_b200_shift_lut(delayed, s_scratch, shift_lut, nBatch, nNeurons, T, Ts, stream_);
    return slayer_b200_shift_scalar(delayed, s_scratch, shift, rows, T, Ts, stream_);
}

extern "C" int slayer_b200_set_srm_stages(int stages)
{
    if (stages < 2 || stages > sb200::kMaxUStages) return sb200::g_srm_stages.load();
    return sb200::g_srm_stages.exchange(stages);
}
