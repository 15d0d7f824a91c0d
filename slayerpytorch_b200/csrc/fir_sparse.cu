// Event-driven form of the temporal filter (slayer_b200_conv / _corr / _conv_packed) for inputs
// that are mostly zeros - spike tensors.  Replaces, for such inputs, the dense tiled kernels of
// fir.cu, which restate convKernel / corrKernel of the reference (src/cuda/convKernels.h:9-44).
//
// A dense filter spends K multiply-adds per output sample whatever the input holds; at the spike
// rates of a trained network (a few percent) almost all of them multiply a zero.  Here a warp
// takes one row: it turns the row into a list of its non-zero samples (time, value) in shared
// memory - one ballot per 32 samples - and then walks the outputs 128 at a time, lane l owning the
// samples t0 + l, t0 + 32 + l, t0 + 64 + l and t0 + 96 + l, adding the contributions of the events
// that can reach that window in the order the dense sum visits them.  Skipped terms are products with zero, so the
// result has the bits of the dense kernel's (taps must be finite: the launcher falls back to
// the dense kernel otherwise; a row that holds a non-finite sample takes a predicated loop so
// that the zero padding of the taps never meets an infinity).  Work is proportional to
// events x taps / 32 + outputs, and at a few percent of events the kernel is bound by HBM.
//
// Which kernel runs is decided on the device: a probe kernel samples the input, counts
// non-zeros and writes a flag; the event-driven kernel and the dense kernel are both enqueued
// and the one the flag rules out returns at once.  Nothing synchronises with the host.
#include <atomic>
#include <cfloat>
#include <mutex>

#include "common.cuh"
#include "fir_sparse.cuh"
#include "tile.cuh"

namespace sb200 {

namespace {

constexpr int kPad = 160;               // zero taps in front of and behind the filter
constexpr int kProbeThreads = 256;
constexpr int64_t kProbeSamples = 1 << 18;

// One decision per call: non-zeros counted, samples seen, blocks that have finished, the decision.
struct ProbeSlot {
    int nnz, seen, done, sparse;
};
constexpr int kProbeSlots = 64;

std::mutex g_slots_mu;
ProbeSlot *g_slots[64] = {nullptr};
std::atomic<unsigned> g_next_slot{0};

// The next slot of the current device's ring.  Calls in flight at the same time on different
// streams use different slots as long as there are fewer than kProbeSlots of them.
ProbeSlot *next_probe_slot()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    {
        std::lock_guard<std::mutex> lock(g_slots_mu);
        if (!g_slots[dev]) {
            ProbeSlot *p = nullptr;
            if (cudaMalloc(&p, kProbeSlots * sizeof(ProbeSlot)) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
            if (cudaMemset(p, 0, kProbeSlots * sizeof(ProbeSlot)) != cudaSuccess) { (void)cudaGetLastError(); cudaFree(p); return nullptr; }
            g_slots[dev] = p;
        }
    }
    return g_slots[dev] + (g_next_slot.fetch_add(1) % kProbeSlots);
}

// Samples whole rows - every time step of a row, since spike rates depend on the time step -
// picked at even spacing with a hashed offset inside each stride, about 2^18 samples in all;
// counts the non-zero samples (set bits when BITS: the input is then 32-bit words of packed
// spikes, `row_len` words per row) and lets the last block to finish decide: event-driven if at
// most `max_per_1024` of 1024 sampled samples are non-zero and every tap is finite.  A warp
// takes one run of up to 256 words of one row, all loads in flight at once.  The counters are
// back at zero when the kernel ends.
template <bool BITS>
__global__ void __launch_bounds__(kProbeThreads)
fir_probe_kernel(const void *__restrict__ in_, int64_t rows, int row_len, int64_t rows_sampled,
                 const float *__restrict__ filt, int K, int max_per_1024, ProbeSlot *slot)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (kProbeThreads / 32) + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * (kProbeThreads / 32);
    const int runs_per_row = (row_len + 255) / 256;
    const int64_t spacing = rows / rows_sampled;        // >= 1
    int count = 0, seen = 0;
    for (int64_t unit = warp; unit < rows_sampled * runs_per_row; unit += nwarps) {
        const int64_t i = unit / runs_per_row;
        const int run = (int)(unit - i * runs_per_row);
        const int64_t row = i * spacing + (int64_t)(((uint64_t)i * 2654435761ull >> 8) % (uint64_t)spacing);
        const int64_t base = row * (int64_t)row_len + run * 256;
        const int left = row_len - run * 256;
        unsigned v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int o = 32 * u + lane;
            v[u] = o < left ? __ldg(static_cast<const unsigned *>(in_) + base + o) : 0u;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            // fp32 samples: anything but +0.0 / -0.0 counts (denormals too: the estimate may err on that side)
            count += BITS ? __popc(v[u]) : ((v[u] << 1) != 0u ? 1 : 0);
            if (32 * u + lane < left) seen += BITS ? 32 : 1;
        }
    }
    int bad_tap = 0;
    if (blockIdx.x == 0) {
        for (int i = threadIdx.x; i < K; i += kProbeThreads)
            if (!(fabsf(__ldg(filt + i)) <= FLT_MAX)) bad_tap = 1;
    }
    bad_tap = __syncthreads_or(bad_tap);
    __shared__ int s_count[kProbeThreads / 32], s_seen[kProbeThreads / 32];
    __shared__ bool s_last;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        count += __shfl_xor_sync(0xffffffffu, count, o);
        seen += __shfl_xor_sync(0xffffffffu, seen, o);
    }
    if (lane == 0) {
        s_count[threadIdx.x >> 5] = count;
        s_seen[threadIdx.x >> 5] = seen;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int c = bad_tap ? 1 << 28 : 0, s = 0;       // a non-finite tap rules the event-driven kernel out
        for (int w = 0; w < kProbeThreads / 32; ++w) {
            c += s_count[w];
            s += s_seen[w];
        }
        atomicAdd(&slot->nnz, c);
        atomicAdd(&slot->seen, s);
        __threadfence();
        s_last = atomicAdd(&slot->done, 1) == (int)gridDim.x - 1;
    }
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        __threadfence();
        const long long nz = atomicAdd(&slot->nnz, 0), sm = atomicAdd(&slot->seen, 0);
        slot->sparse = (sm > 0 && nz * 1024 <= (long long)max_per_1024 * sm) ? 1 : 0;
        slot->nnz = 0;
        slot->seen = 0;
        slot->done = 0;
        __threadfence();
    }
}

// One event of a row: its time step and its value.
struct __align__(8) Event {
    int t;
    float x;
};

// Shared memory of one warp: the event list (one slot per sample: a row may be all events),
// nwords + 1 prefix counts, and - fp32 input - the staging buffer of the row.
__host__ __device__ inline size_t sparse_warp_bytes(int nwords, bool bits)
{
    return (size_t)nwords * 32 * sizeof(Event) + (size_t)((nwords + 4) & ~3) * sizeof(int) +
           (bits ? 0 : (size_t)nwords * 32 * sizeof(float));
}

// DIR = -1: conv (out[t] = Ts * sum_i filt[i] * in[t - i], i ascending), DIR = +1: corr
// (out[t] = Ts * sum_i filt[i] * in[t + i]).  BITS: the input is a bit-packed spike tensor
// (32-bit words, ceil(T / 32) per row, bit b of word w = "sample 32 w + b is spike_value").
// run_flag: NULL, or a word that must be non-zero for the kernel to do anything.
// The next row of a warp is on its way while the current one is filtered: fp32 rows by
// asynchronous copies into the staging buffer (16 bytes each when `vec4`: T % 4 == 0 and a
// 16-byte aligned base), packed rows in up to four registers per lane.
template <int DIR, bool BITS, int NACC>
__global__ void __launch_bounds__(256)
fir_sparse_kernel(float *__restrict__ out, const void *__restrict__ in_, const float *__restrict__ filt,
                  int64_t rows, int T, int K, float Ts, float spike_value, bool vec4, const int *run_flag)
{
    if (run_flag != nullptr && *run_flag == 0) return;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    const int nwords = (T + 31) >> 5;
    const int wp_len = (2 * kPad + K + 3) & ~3;
    float *wp = reinterpret_cast<float *>(smem_raw);        // taps with kPad zeros on either side
    unsigned char *mine = smem_raw + sizeof(float) * wp_len + (size_t)warp * sparse_warp_bytes(nwords, BITS);
    float *xbuf = reinterpret_cast<float *>(mine);                                  // fp32 input only
    Event *list = reinterpret_cast<Event *>(mine + (BITS ? 0 : (size_t)nwords * 32 * sizeof(float)));
    int *cnt = reinterpret_cast<int *>(reinterpret_cast<unsigned char *>(list) + (size_t)nwords * 32 * sizeof(Event));

    for (int i = threadIdx.x; i < wp_len; i += blockDim.x) wp[i] = (i >= kPad && i < kPad + K) ? __ldg(filt + (i - kPad)) : 0.0f;
    __syncthreads();

    const int H = (K + 30) >> 5;                            // words of the past (conv) or future (corr) that reach a word
    const unsigned lt = (1u << lane) - 1u;
    const float *wl = wp + kPad + (DIR < 0 ? lane : -lane); // this lane's view of the taps (see the walk below)
    const int64_t stride = (int64_t)gridDim.x * nwarps;
    int64_t row = (int64_t)blockIdx.x * nwarps + warp;

    unsigned held[4] = {0u, 0u, 0u, 0u};                    // BITS: words lane, lane + 32, ... of the row on its way
    auto fetch = [&](int64_t r) {
        if (BITS) {
            const unsigned *bw = static_cast<const unsigned *>(in_) + r * (int64_t)nwords;
#pragma unroll
            for (int j = 0; j < 4; ++j) held[j] = 32 * j + lane < nwords ? __ldg(bw + 32 * j + lane) : 0u;
        } else {
            const float *x = static_cast<const float *>(in_) + r * (int64_t)T;
            if (vec4) {
                for (int q = lane; q < nwords * 8; q += 32) cp_async<16>(xbuf + 4 * q, 4 * q < T ? x + 4 * q : x, 4 * q < T);
            } else {
                for (int t = lane; t < nwords * 32; t += 32) cp_async<4>(xbuf + t, t < T ? x + t : x, t < T);
            }
            cp_async_commit();
        }
    };
    if (row < rows) fetch(row);

    for (; row < rows; row += stride) {
        // ---- the row's events, in time order
        int running = 0;
        unsigned bad = 0u;
        if (!BITS) {
            cp_async_wait<0>();
            __syncwarp();
            for (int c = 0; c < nwords; ++c) {
                const float v = xbuf[32 * c + lane];
                const bool nz = v != 0.0f;
                const unsigned m = __ballot_sync(0xffffffffu, nz);
                bad |= __ballot_sync(0xffffffffu, !(fabsf(v) <= FLT_MAX));
                if (lane == 0) cnt[c] = running;
                if (nz) list[running + __popc(m & lt)] = Event{32 * c + lane, v};
                running += __popc(m);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (32 * j < nwords) {
                    const int c = 32 * j + lane;
                    unsigned w = held[j];
                    if (c == nwords - 1 && (T & 31)) w &= (1u << (T & 31)) - 1u;       // bits past the row end
                    const int pc = __popc(w);
                    int incl = pc;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const int up = __shfl_up_sync(0xffffffffu, incl, o);
                        if (lane >= o) incl += up;
                    }
                    int p = running + incl - pc;
                    if (c < nwords) cnt[c] = p;
                    while (w) {
                        const int b = __ffs(w) - 1;
                        w &= w - 1u;
                        list[p++] = Event{32 * c + b, spike_value};
                    }
                    running += __shfl_sync(0xffffffffu, incl, 31);
                }
            }
        }
        if (lane == 0) cnt[nwords] = running;
        __syncwarp();           // the list is complete and the staging buffer has been read
        if (row + stride < rows) fetch(row + stride);

        // ---- outputs, 32 NACC at a time: lane l owns t0 + l, t0 + 32 + l, ...
        float *o = out + row * (int64_t)T;
        for (int c = 0; c < nwords; c += NACC) {
            int lo, hi;
            if (DIR < 0) {
                lo = cnt[c - H > 0 ? c - H : 0];
                hi = cnt[c + NACC < nwords ? c + NACC : nwords];
            } else {
                lo = cnt[c];
                hi = cnt[c + NACC + H < nwords ? c + NACC + H : nwords];
            }
            float acc[NACC];
#pragma unroll
            for (int j = 0; j < NACC; ++j) acc[j] = 0.0f;
            if (bad == 0u) {
                // tap index of this lane's first sample for an event at t: k = (32 c + lane) - t
                // (conv) or t - (32 c + lane) (corr); its sample j is 32 j taps further on (conv)
                // or back (corr); taps outside the filter read as zero
                const float *wb = wl + (DIR < 0 ? 32 * c : -32 * c);
                if (DIR < 0) {
#pragma unroll 2
                    for (int i = hi - 1; i >= lo; --i) {
                        const Event e = list[i];
                        const float *we = wb - e.t;
#pragma unroll
                        for (int j = 0; j < NACC; ++j) acc[j] = fmaf(e.x, we[32 * j], acc[j]);
                    }
                } else {
#pragma unroll 2
                    for (int i = lo; i < hi; ++i) {
                        const Event e = list[i];
                        const float *we = wb + e.t;
#pragma unroll
                        for (int j = 0; j < NACC; ++j) acc[j] = fmaf(e.x, we[-32 * j], acc[j]);
                    }
                }
            } else {
                // a non-finite sample in this row: only the terms of the definition
                const int t0 = 32 * c + lane;
                for (int n = 0; n < hi - lo; ++n) {
                    const Event e = list[DIR < 0 ? hi - 1 - n : lo + n];
                    const int k0 = DIR < 0 ? t0 - e.t : e.t - t0;
#pragma unroll
                    for (int j = 0; j < NACC; ++j) {
                        const int k = DIR < 0 ? k0 + 32 * j : k0 - 32 * j;
                        if ((unsigned)k < (unsigned)K) acc[j] = fmaf(e.x, wp[kPad + k], acc[j]);
                    }
                }
            }
            const int t0 = 32 * c + lane;
#pragma unroll
            for (int j = 0; j < NACC; ++j)
                if (t0 + 32 * j < T) o[t0 + 32 * j] = acc[j] * Ts;
        }
        __syncwarp();           // the list is rebuilt for the next row
    }
}

template <int DIR, bool BITS, int NACC>
int launch_sparse(float *out, const void *in, const float *filt, int64_t rows, int64_t T, int64_t K, float Ts,
                  float spike_value, const int *run_flag, cudaStream_t stream)
{
    const int nwords = (int)((T + 31) >> 5);
    const size_t per_warp = sparse_warp_bytes(nwords, BITS);
    const size_t taps = sizeof(float) * (size_t)((2 * kPad + K + 3) & ~3LL);
    // the largest CTA of which two still fit an SM; one CTA per SM for the longest rows
    int nwarps = 8;
    while (nwarps > 1 && taps + nwarps * per_warp > 100 * 1024) nwarps >>= 1;
    const size_t smem = taps + nwarps * per_warp;
    auto kern = fir_sparse_kernel<DIR, BITS, NACC>;
    int rc = reserve_dynamic_smem((const void *)kern, smem);
    if (rc) return rc;
    // a persistent grid: exactly the CTAs that are resident at once
    int ctas_per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas_per_sm, kern, nwarps * 32, smem) != cudaSuccess) {
        (void)cudaGetLastError();
        ctas_per_sm = 1;
    }
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    int64_t grid = (int64_t)ctas_per_sm * sm_count();
    const int64_t need = ceil_div(rows, nwarps);
    if (grid > need) grid = need;
    const bool vec4 = !BITS && (T & 3) == 0 && aligned16(in);
    kern<<<(unsigned)grid, nwarps * 32, smem, stream>>>(out, in, filt, rows, (int)T, (int)K, Ts, spike_value, vec4, run_flag);
    return check_launch("fir (event-driven) kernel launch");
}

}  // namespace

bool fir_sparse_eligible(int64_t rows, int64_t T, int64_t K)
{
    // rows of at least two words, short enough for the event list of a warp (8 bytes per sample)
    // to fit shared memory, and taps that fit next to it
    return rows > 0 && T >= 64 && T <= kFirSparseMaxT && K >= 1 && K <= kFirSparseMaxTaps;
}

int fir_sparse_probe(const void *in, int64_t rows, int64_t T, bool bits, const float *filt, int64_t K,
                     cudaStream_t stream, const int **flag)
{
    *flag = nullptr;
    ProbeSlot *slot = next_probe_slot();
    if (!slot) return SLAYER_B200_OK;               // no scratch: the caller runs the dense kernel alone
    int64_t rows_sampled = ceil_div(kProbeSamples, T);
    if (rows_sampled > rows) rows_sampled = rows;
    const int row_len = (int)(bits ? (T + 31) / 32 : T);
    const int64_t units = rows_sampled * ((row_len + 255) / 256);
    int64_t blocks = ceil_div(units, kProbeThreads / 32);
    if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
    if (bits) fir_probe_kernel<true><<<(unsigned)blocks, kProbeThreads, 0, stream>>>(in, rows, row_len, rows_sampled, filt, (int)K,
                                                                                      kFirSparseMaxPer1024Bits, slot);
    else fir_probe_kernel<false><<<(unsigned)blocks, kProbeThreads, 0, stream>>>(in, rows, row_len, rows_sampled, filt, (int)K,
                                                                                  kFirSparseMaxPer1024, slot);
    const int rc = check_launch("fir (density probe) kernel launch");
    if (rc == SLAYER_B200_OK) *flag = &slot->sparse;
    return rc;
}

int fir_sparse_launch(int dir, bool bits, float *out, const void *in, const float *filt, int64_t rows, int64_t T,
                      int64_t K, float Ts, float spike_value, const int *run_flag, cudaStream_t stream)
{
    if (bits) return launch_sparse<-1, true, 4>(out, in, filt, rows, T, K, Ts, spike_value, run_flag, stream);
    if (dir < 0) return launch_sparse<-1, false, 4>(out, in, filt, rows, T, K, Ts, 0.0f, run_flag, stream);
    return launch_sparse<1, false, 4>(out, in, filt, rows, T, K, Ts, 0.0f, run_flag, stream);
}

}  // namespace sb200
