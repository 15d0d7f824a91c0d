// Loihi CUBA neuron: fixed-point current / voltage decay, threshold and refractory delay.
//
// Per row, with integer state uOld = vOld = 0 and the neuron not refractory:
//   t = 0:  s = v = u = 0 (the input sample is ignored)
//   t >= 1: uT = sgn(uOld) * ((|uOld| * (4096 - iDecay)) >> 12) + (64 << wgtExp) * int(w[t])
//           vT = sgn(vOld) * ((|vOld| * (4096 - vDecay)) >> 12) + uT
//           the refractory state set by a spike at t' is cleared at the top of step t'+refDelay
//           spike = vT > theta and not refractory
//           vOld  = vT if neither refractory nor spiking, else 0;   uOld = uT
//           outputs: s = spike, u = uT, v = vDecay at a spike else vOld
// All products and the >> 12 are evaluated modulo 2^32 with a logical shift (the reference's
// expressions mix int and unsigned operands), sgn(0) = +1, and outputs are float images of
// the int32 values.  The reference re-reads its own spike output from refDelay steps back to
// clear the refractory state; because a neuron cannot spike while refractory, that is
// equivalent to the countdown kept in a register here.
//
// Memory: 16 algorithmic bytes per element (read w; write s, v, u), bound by HBM.  A warp owns
// 32 rows and walks them in time tiles staged in swizzled shared memory (lane = row), as in the
// SRM kernel.  Two kernels: 16-byte aligned buffers take loihi_get_spikes_wide_kernel (64-step
// row-skewed tiles, spikes kept as bit masks); other alignments take loihi_get_spikes_kernel
// (32-step tiles, 8- or 4-byte accesses), described first.
#include "common.cuh"
#include "tile.cuh"

namespace sb200 {

template <int V>
__global__ void __launch_bounds__(256)
loihi_get_spikes_kernel(float *s, float *v, float *u, const float *w,
                        int64_t rows, int T, unsigned weightScale, int theta,
                        unsigned iKeep, unsigned vKeep, int vDecayMark, unsigned refDelay)
{
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps_per_block = blockDim.x >> 5;
    float *tiles_u = smem + warp * (4 * kTileWords);     // two input/current tiles (prefetch ring)
    float *tile_v = tiles_u + 2 * kTileWords;            // voltage tile
    float *tile_s = tiles_u + 3 * kTileWords;            // spike tile
    const float vMarkF = (float)vDecayMark;

    // The warp's work is one stream of tiles: all time tiles of its first block of 32 rows, then
    // of its next block, ...  The tile after the current one - possibly the first tile of the
    // next row block - is always in flight, so a change of row block costs no memory latency.
    // V == 4 uses row-skewed tiles (tile.cuh): 16-byte accesses on 32-byte boundaries for any T.
    // Samples before a row's start are padded with zeros and the sample at t = 0 is replaced by
    // zero: with zero input the neuron's state stays zero and its outputs are zero, which is
    // exactly what the definition prescribes for t = 0 (the host only picks this variant when
    // theta is non-negative as a signed int, so that 0 > theta cannot fire).
    const int ntiles = V == 4 ? skew_tiles(T) : (T + kTile - 1) / kTile;
    const unsigned phase = (unsigned)(reinterpret_cast<uintptr_t>(w) >> 2) & 7u;
    const int64_t nblocks = (rows + kTile - 1) / kTile;
    const int64_t wstride = (int64_t)gridDim.x * warps_per_block;
    int64_t rb = (int64_t)blockIdx.x * warps_per_block + warp;
    if (rb >= nblocks) return;
    int64_t rb_next = rb;           // (row block, tile) of the tile to prefetch next
    int it_next = 0;
    int skew = V == 4 ? block_skew(rb * kTile, T, phase) : 0;
    int skew_next = skew;
    int uOld = 0, vOld = 0;
    unsigned refLeft = 0;           // steps until the refractory state clears

    auto prefetch = [&](float *dst) {
        if (V == 4) tile_prefetch_skew(dst, w, rb_next * kTile, rows, it_next, T, lane, skew_next, 0.0f);
        else tile_prefetch<V>(dst, w, rb_next * kTile, rows, it_next * kTile, T, lane);
        if (++it_next == ntiles) {
            it_next = 0;
            rb_next += wstride;
            if (V == 4 && rb_next < nblocks) skew_next = block_skew(rb_next * kTile, T, phase);
        }
    };
    prefetch(tiles_u);
    cp_async_commit();

    {
        int it = 0;
        for (unsigned q = 0; rb < nblocks; ++q) {
            const int64_t row0 = rb * kTile;
            const int t0 = it * kTile;
            float *tile_u = tiles_u + (q & 1) * kTileWords;
            if (it == 0) {
                uOld = 0;
                vOld = 0;
                refLeft = 0;
            }
            if (rb_next < nblocks) prefetch(tiles_u + ((q + 1) & 1) * kTileWords);
            cp_async_commit();
            cp_async_wait<1>();
            __syncwarp();
            if (V == 4 && it == 0) tile_u[tile_word(lane, row_skew(skew, lane, T))] = 0.0f;   // w[t = 0] is ignored

            // walk the 32 steps; the next chunk is fetched before the current one is processed
            float4 cur = *reinterpret_cast<const float4 *>(tile_u + tile_chunk(lane, 0));
#pragma unroll 2
            for (int c4 = 0; c4 < kTile / 4; ++c4) {
                float4 nxt = cur;
                if (c4 + 1 < kTile / 4) nxt = *reinterpret_cast<const float4 *>(tile_u + tile_chunk(lane, c4 + 1));
                const float wv[4] = {cur.x, cur.y, cur.z, cur.w};
                float uo[4], vo[4], so[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (V != 4 && it == 0 && c4 == 0 && j == 0) {   // t = 0
                        uo[j] = 0.0f;
                        vo[j] = 0.0f;
                        so[j] = 0.0f;
                        continue;
                    }
                    const unsigned uSign = uOld >= 0 ? 1u : 0xffffffffu;
                    const unsigned vSign = vOld >= 0 ? 1u : 0xffffffffu;
                    const unsigned uT = uSign * ((uSign * (unsigned)uOld * iKeep) >> 12)
                                      + weightScale * (unsigned)__float2int_rz(wv[j]);
                    const unsigned vT = vSign * ((vSign * (unsigned)vOld * vKeep) >> 12) + uT;
                    const int vTemp = (int)vT;

                    if (refLeft != 0) --refLeft;
                    const bool refractory = refLeft != 0;
                    const bool spk = (vTemp > theta) && !refractory;
                    vOld = (refractory || spk) ? 0 : vTemp;
                    if (spk) refLeft = refDelay;
                    uOld = (int)uT;

                    so[j] = spk ? 1.0f : 0.0f;
                    uo[j] = (float)uOld;
                    vo[j] = spk ? vMarkF : (float)vOld;
                }
                *reinterpret_cast<float4 *>(tile_u + tile_chunk(lane, c4)) = make_float4(uo[0], uo[1], uo[2], uo[3]);
                *reinterpret_cast<float4 *>(tile_v + tile_chunk(lane, c4)) = make_float4(vo[0], vo[1], vo[2], vo[3]);
                *reinterpret_cast<float4 *>(tile_s + tile_chunk(lane, c4)) = make_float4(so[0], so[1], so[2], so[3]);
                cur = nxt;
            }
            __syncwarp();

            if (V == 4) {
                tile_store3_skew(tile_u, tile_v, tile_s, u, v, s, row0, rows, it, T, lane, skew);
            } else {
                tile_store<V>(tile_u, u, row0, rows, t0, T, lane);
                tile_store<V>(tile_v, v, row0, rows, t0, T, lane);
                tile_store<V>(tile_s, s, row0, rows, t0, T, lane);
            }
            __syncwarp();
            if (++it == ntiles) {
                it = 0;
                rb += wstride;
                if (V == 4 && rb < nblocks) skew = block_skew(rb * kTile, T, phase);
            }
        }
    }
}


// One time step of the neuron for one row.  The decays are written on the magnitude with the
// sign folded back in by xor / subtract (sm = 0 or -1): for every 32-bit state, INT_MIN
// included, this is the reference's expression sgn(x) * ((sgn(x) * x * keep) >> 12) evaluated
// modulo 2^32 with a logical shift.
struct LoihiRow {
    int uOld, vOld;
    unsigned refLeft;           // steps until the refractory state clears (0 = not refractory)

    __device__ __forceinline__ void reset() { uOld = 0; vOld = 0; refLeft = 0; }

    // wv: weighted input sample; returns the spike flag, writes the float images of u and v
    __device__ __forceinline__ bool step(float wv, unsigned weightScale, int theta, unsigned iKeep, unsigned vKeep,
                                         float vMarkF, unsigned refDelay, float &uo, float &vo)
    {
        const int us = uOld >> 31, vs = vOld >> 31;
        const unsigned udec = (((unsigned)((uOld ^ us) - us) * iKeep) >> 12);
        const unsigned vdec = (((unsigned)((vOld ^ vs) - vs) * vKeep) >> 12);
        const unsigned uT = (unsigned)(((int)udec ^ us) - us) + weightScale * (unsigned)__float2int_rz(wv);
        const int vT = (int)((unsigned)(((int)vdec ^ vs) - vs) + uT);
        if (refLeft != 0) --refLeft;
        const bool quiet = refLeft == 0;
        const bool spk = (vT > theta) && quiet;
        vOld = (quiet && !spk) ? vT : 0;
        if (spk) refLeft = refDelay;
        uOld = (int)uT;
        uo = (float)uOld;
        vo = spk ? vMarkF : (float)vOld;
        return spk;
    }
};

// Two wide tiles of the same rows and steps to two arrays of the same shape: the row, its skew,
// the bounds and the offset are worked out once per pass and shared by the two stores; the
// spike samples of the same tile are expanded from bit masks in the same pass.
template <bool SKEW, bool WRITE_U>
__device__ __forceinline__ void wide_store_loihi(const float *tile_u, const float *tile_v, const unsigned *masks,
                                                 float *gu, float *gv, float *gs, int64_t row0, int64_t rows,
                                                 int j, int T, int lane, int skew0)
{
    const int c16 = lane & 15;
    const int rsub = lane >> 4;
    const int hoff = (c16 >> 3) * kTileWords;
    const unsigned *mhalf = masks + (c16 >> 3) * kTile;
    const int c = (c16 & 7) * 4;
    const int64_t nrow = rows - row0;
#pragma unroll
    for (int i = 0; i < kTile / 2; ++i) {
        const int r = i * 2 + rsub;
        if (r >= nrow) continue;
        const int t = kWide * j - (SKEW ? row_skew(skew0, r, T) : 0) + c16 * 4;
        if (t >= T || t + 4 <= 0) continue;
        const int wd = hoff + tile_word(r, c);
        const float4 vu = WRITE_U ? *reinterpret_cast<const float4 *>(tile_u + wd) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const float4 vv = *reinterpret_cast<const float4 *>(tile_v + wd);
        const unsigned m = mhalf[r] >> c;
        const float4 vs = make_float4((m & 1u) ? 1.0f : 0.0f, (m & 2u) ? 1.0f : 0.0f, (m & 4u) ? 1.0f : 0.0f, (m & 8u) ? 1.0f : 0.0f);
        const int64_t off = (row0 + r) * (int64_t)T + t;
        if (t >= 0 && t + 4 <= T) {
            if (WRITE_U) *reinterpret_cast<float4 *>(gu + off) = vu;
            *reinterpret_cast<float4 *>(gv + off) = vv;
            *reinterpret_cast<float4 *>(gs + off) = vs;
        } else {
            const float eu[4] = {vu.x, vu.y, vu.z, vu.w};
            const float ev[4] = {vv.x, vv.y, vv.z, vv.w};
            const float es[4] = {vs.x, vs.y, vs.z, vs.w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (t + k >= 0 && t + k < T) {
                    if (WRITE_U) gu[off + k] = eu[k];
                    gv[off + k] = ev[k];
                    gs[off + k] = es[k];
                }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Wide-tile kernel (16-byte aligned buffers, threshold below 2^31, any T): row-skewed tiles of
// 64 steps, so that every global request covers 256 contiguous bytes of a row - DRAM on this
// part runs measurably closer to its peak on 256-byte row segments than on 128-byte ones.
// Per warp: `depth` input tiles (8 KB each; the current u overwrites the input in place), one
// tile for v, and the spike bits of the tile being walked (256 bytes), expanded to samples on
// their way out.  Samples before a row's start are padded with zeros and the sample at t = 0
// is replaced by zero: with zero input the state stays zero and all outputs are zero, which is
// what the definition prescribes for t = 0 (0 > theta cannot fire because theta >= 0 here).
//
// WRITE_U = false leaves the current out (callers that only keep spikes and voltage: 12 instead
// of 16 bytes per element).  `delay` (0 .. 63 steps) writes the spikes already delayed,
// s_out[t] = s[t - delay]: a Loihi layer is always followed by a delay of one step, and the
// spike bits of a tile only need a 64-bit shift with carry from the previous tile for that, so
// the separate shift pass (8 bytes per element) disappears.
// ---------------------------------------------------------------------------------------
template <bool SKEW, bool WRITE_U>
__global__ void __launch_bounds__(256)
loihi_get_spikes_wide_kernel(float *s, float *v, float *u, const float *w,
                             int64_t rows, int T, unsigned weightScale, int theta,
                             unsigned iKeep, unsigned vKeep, int vDecayMark, unsigned refDelay, int depth, int delay)
{
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps_per_block = blockDim.x >> 5;
    float *tiles = smem + warp * ((depth + 1) * kWideWords + 2 * kTile);
    float *tile_v = tiles + depth * kWideWords;
    unsigned *masks = reinterpret_cast<unsigned *>(tile_v + kWideWords);
    const float vMarkF = (float)vDecayMark;

    const int ntiles = SKEW ? skew_wide_tiles(T) : (T + kWide - 1) / kWide;
    const unsigned phase = (unsigned)(reinterpret_cast<uintptr_t>(w) >> 2) & 7u;
    const int64_t nblocks = (rows + kTile - 1) / kTile;
    const int64_t wstride = (int64_t)gridDim.x * warps_per_block;
    int64_t rb = (int64_t)blockIdx.x * warps_per_block + warp;
    if (rb >= nblocks) return;
    int64_t rb_next = rb;           // (row block, tile) of the tile to prefetch next
    int it_next = 0;
    int skew = SKEW ? block_skew(rb * kTile, T, phase) : 0;
    int skew_next = skew;
    unsigned q = 0;                 // tiles walked so far: buffer = q & (depth - 1)
    const unsigned dmask = (unsigned)depth - 1u;
    LoihiRow st;
    st.reset();
    unsigned long long prev_bits = 0ull;      // spike bits of the previous tile of this lane's row

    auto prefetch = [&](float *dst) {
        wide_prefetch_skew<SKEW>(dst, w, rb_next * kTile, rows, it_next, T, lane, skew_next, 0.0f);
        if (++it_next == ntiles) {
            it_next = 0;
            rb_next += wstride;
            if (SKEW && rb_next < nblocks) skew_next = block_skew(rb_next * kTile, T, phase);
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
            prev_bits = 0ull;
        }
        if (rb_next < nblocks) prefetch(tiles + ((q + dmask) & dmask) * kWideWords);
        cp_async_commit();
        if (depth == 2) cp_async_wait<1>();
        else cp_async_wait<3>();
        __syncwarp();
        if (it == 0) tile[tile_word(lane, SKEW ? row_skew(skew, lane, T) : 0)] = 0.0f;      // w[t = 0] is ignored

        // the second half lies wholly past the end of every row when even the most skewed row
        // (7 steps behind) has run out of samples there
        const bool second = kWide * it + kTile - (SKEW ? 7 : 0) < T;
        unsigned m[2] = {0u, 0u};
#pragma unroll 1
        for (int h = 0; h < (second ? 2 : 1); ++h) {
            float *th = tile + h * kTileWords;
            float *tv = tile_v + h * kTileWords;
            unsigned mh = 0u;
            float4 cur = *reinterpret_cast<const float4 *>(th + tile_chunk(lane, 0));
#pragma unroll
            for (int c4 = 0; c4 < kTile / 4; ++c4) {
                float4 nxt = cur;       // the next chunk is fetched before the current one is processed
                if (c4 + 1 < kTile / 4) nxt = *reinterpret_cast<const float4 *>(th + tile_chunk(lane, c4 + 1));
                const float wv[4] = {cur.x, cur.y, cur.z, cur.w};
                float uo[4], vo[4];
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (st.step(wv[k], weightScale, theta, iKeep, vKeep, vMarkF, refDelay, uo[k], vo[k])) mh |= 1u << (c4 * 4 + k);
                if (WRITE_U) *reinterpret_cast<float4 *>(th + tile_chunk(lane, c4)) = make_float4(uo[0], uo[1], uo[2], uo[3]);
                *reinterpret_cast<float4 *>(tv + tile_chunk(lane, c4)) = make_float4(vo[0], vo[1], vo[2], vo[3]);
                cur = nxt;
            }
            if (h == 0) m[0] = mh;
            else m[1] = mh;
        }
        {
            // the tile's 64 spike bits, delayed: bits that leave at the top come back in at the
            // bottom of the next tile
            const unsigned long long cur_bits = ((unsigned long long)m[1] << 32) | m[0];
            const unsigned long long out_bits = delay ? (cur_bits << delay) | (prev_bits >> (64 - delay)) : cur_bits;
            prev_bits = cur_bits;
            masks[lane] = (unsigned)out_bits;
            masks[kTile + lane] = (unsigned)(out_bits >> 32);
        }
        __syncwarp();

        wide_store_loihi<SKEW, WRITE_U>(tile, tile_v, masks, u, v, s, row0, rows, it, T, lane, skew);
        __syncwarp();
        if (++it == ntiles) {
            it = 0;
            rb += wstride;
            if (SKEW && rb < nblocks) skew = block_skew(rb * kTile, T, phase);
        }
    }
}

struct LoihiArgs {
    float *s, *v, *u;
    const float *w;
    int64_t rows;
    int T;
    unsigned weightScale;
    int theta;
    unsigned iKeep, vKeep;
    int vMark;
    unsigned refDelay;
    cudaStream_t stream;
};

template <int V>
static int launch_loihi(const LoihiArgs &a)
{
    const int64_t nblocks = ceil_div(a.rows, kTile);
    int warps, grid;
    spike_launch_shape(nblocks, 4 * kTileWords * sizeof(float), warps, grid);
    const size_t smem = (size_t)warps * 4 * kTileWords * sizeof(float);
    auto kern = loihi_get_spikes_kernel<V>;
    int rc = reserve_dynamic_smem((const void *)kern, smem);
    if (rc) return rc;
    kern<<<(unsigned)grid, warps * 32, smem, a.stream>>>(a.s, a.v, a.u, a.w, a.rows, a.T, a.weightScale, a.theta,
                                                         a.iKeep, a.vKeep, a.vMark, a.refDelay);
    return check_launch("loihi_get_spikes kernel launch");
}

static int launch_loihi_wide(const LoihiArgs &a, int delay = 0)
{
    const int64_t nblocks = ceil_div(a.rows, kTile);
    // prefetch depth 4 when every warp of the launch is resident at once even with the larger
    // footprint (then latency, not bandwidth, bounds the launch), depth 2 otherwise
    const size_t deep_bytes = (5 * kWideWords + 2 * kTile) * sizeof(float);
    const int depth = nblocks <= (int64_t)((216 * 1024) / deep_bytes) * sm_count() ? 4 : 2;
    const size_t warp_bytes = (size_t)((depth + 1) * kWideWords + 2 * kTile) * sizeof(float);
    int warps, grid;
    spike_launch_shape(nblocks, warp_bytes, warps, grid);
    const size_t smem = (size_t)warps * warp_bytes;
    // rows that start on 32-byte boundaries need no skew
    const bool skew = (a.T & 7) != 0 || (reinterpret_cast<uintptr_t>(a.w) & 31u) != 0;
    auto kern = a.u ? (skew ? loihi_get_spikes_wide_kernel<true, true> : loihi_get_spikes_wide_kernel<false, true>)
                    : (skew ? loihi_get_spikes_wide_kernel<true, false> : loihi_get_spikes_wide_kernel<false, false>);
    int rc = reserve_dynamic_smem((const void *)kern, smem);
    if (rc) return rc;
    kern<<<(unsigned)grid, warps * 32, smem, a.stream>>>(a.s, a.v, a.u, a.w, a.rows, a.T, a.weightScale, a.theta,
                                                         a.iKeep, a.vKeep, a.vMark, a.refDelay, depth, delay);
    return check_launch("loihi_get_spikes (wide tile) kernel launch");
}

}  // namespace sb200

extern "C" int slayer_b200_loihi_get_spikes(float *s, float *v, float *u, const float *w,
                                            int64_t rows, int64_t T,
                                            uint32_t wgtExp, uint32_t theta, uint32_t iDecay,
                                            uint32_t vDecay, uint32_t refDelay, void *stream_)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(rows >= 0 && T >= 0, "loihi_get_spikes: negative size");
    SB200_REQUIRE(T < (1LL << 31) - 64, "loihi_get_spikes: T=%lld too large", (long long)T);
    SB200_REQUIRE(refDelay >= 1, "loihi_get_spikes: refDelay must be >= 1");
    SB200_REQUIRE(wgtExp <= 25, "loihi_get_spikes: wgtExp=%u out of range", wgtExp);
    if (rows == 0 || T == 0) return SLAYER_B200_OK;
    SB200_REQUIRE(s && v && u && w, "loihi_get_spikes: null pointer");
    SB200_REQUIRE(s != v && s != u && v != u && s != w && v != w,
                  "loihi_get_spikes: output buffers must be distinct");
    const LoihiArgs a = {s, v, u, w, rows, (int)T, 1u << (6 + wgtExp), (int)theta,
                         4096u - iDecay, 4096u - vDecay, (int)vDecay, refDelay, (cudaStream_t)stream_};
    // 16-byte aligned buffers and a threshold below 2^31: row-skewed 16-byte tiles for any T;
    // otherwise the widest access the alignment allows
    int vw = tile_vec_width(T, {s, v, u, w});
    if (all_aligned16({s, v, u, w}) && theta < 0x80000000u) vw = 4;
    else if (vw == 4) vw = 2;
    switch (vw) {
        case 4: return launch_loihi_wide(a);
        case 2: return launch_loihi<2>(a);
        default: return launch_loihi<1>(a);
    }
}

extern "C" int slayer_b200_loihi_get_spikes_delayed(float *delayed, float *v, float *u, const float *w,
                                                    int64_t rows, int64_t T,
                                                    uint32_t wgtExp, uint32_t theta, uint32_t iDecay,
                                                    uint32_t vDecay, uint32_t refDelay, int64_t delay, void *stream_)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(rows >= 0 && T >= 0, "loihi_get_spikes_delayed: negative size");
    SB200_REQUIRE(T < (1LL << 31) - 64, "loihi_get_spikes_delayed: T=%lld too large", (long long)T);
    SB200_REQUIRE(refDelay >= 1, "loihi_get_spikes_delayed: refDelay must be >= 1");
    SB200_REQUIRE(wgtExp <= 25, "loihi_get_spikes_delayed: wgtExp=%u out of range", wgtExp);
    if (rows == 0 || T == 0) return SLAYER_B200_OK;
    SB200_REQUIRE(delayed && v && w, "loihi_get_spikes_delayed: null pointer");
    SB200_REQUIRE(delayed != v && delayed != u && v != u && delayed != w && v != w && u != w,
                  "loihi_get_spikes_delayed: buffers must be distinct");
    if (delay < 0 || delay > 63 || theta >= 0x80000000u || !all_aligned16({delayed, v, w}) || (u && !aligned16(u))) {
        set_error("loihi_get_spikes_delayed: needs a delay of 0 .. 63 steps, 16-byte aligned buffers and a threshold "
                  "below 2^31; otherwise run slayer_b200_loihi_get_spikes and slayer_b200_shift_scalar");
        return SLAYER_B200_EUNSUPPORTED;
    }
    const LoihiArgs a = {delayed, v, u, w, rows, (int)T, 1u << (6 + wgtExp), (int)theta,
                         4096u - iDecay, 4096u - vDecay, (int)vDecay, refDelay, (cudaStream_t)stream_};
    return launch_loihi_wide(a, (int)delay);
}
