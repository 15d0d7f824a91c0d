// Address events -> spike tensor (binning in time), on the device.
//
// An event is (x, y, p, t): pixel, polarity / channel and a timestamp in milliseconds.  The
// tensor is [C, H, W, T] (or [N, C, H, W, T] with a sample index per event); event e lands at
//   [p, y, x, rint(t / samplingTime) - tStart]          (rint: double precision, half to even)
// if every index is inside the tensor, and is dropped otherwise.  Two modes, as the host
// routine this replaces has them:
//   OR   the element becomes 1 / samplingTime;
//   SUM  the element becomes its ORIGINAL value + 1 / samplingTime, once, however many events
//        share the bin (an indexed "+=" evaluates its right-hand side from the original tensor
//        and assigns once per index), which is why SUM reads `base` and writes `out`.
// One thread per event; events that share a bin all store the same value, so the result does
// not depend on the order in which they arrive.  The packed form sets bits (32 bins per word)
// with an atomic OR.  Memory: 20-28 bytes read per event and one scattered 4-byte store; the
// tensor itself is only touched where events land.
#include "common.cuh"

namespace sb200 {

struct EventArgs {
    const int32_t *n, *x, *y, *p;      // n and y may be null (one sample; one spatial dimension)
    const double *t;
    int64_t count;
    int64_t N, C, H, W, T;
    double samplingTime;
    int64_t tStart;
};

// flat element index of event e, or -1 if it falls outside the tensor
__device__ __forceinline__ int64_t event_index(const EventArgs &a, int64_t e, int64_t &tbin)
{
    const int64_t n = a.n ? a.n[e] : 0;
    const int64_t x = a.x[e];
    const int64_t y = a.y ? a.y[e] : 0;
    const int64_t p = a.p[e];
    const double q = rint(a.t[e] / a.samplingTime);
    if (!(q > -9.0e18 && q < 9.0e18)) return -1;           // NaN or out of any tensor's range
    tbin = (int64_t)q - a.tStart;
    if (n < 0 || n >= a.N || x < 0 || x >= a.W || y < 0 || y >= a.H || p < 0 || p >= a.C || tbin < 0 || tbin >= a.T)
        return -1;
    return (((n * a.C + p) * a.H + y) * a.W + x);          // row; the element is row * T + tbin
}

template <bool SUM>
__global__ void __launch_bounds__(256)
bin_events_kernel(float *__restrict__ out, const float *__restrict__ base, EventArgs a, float value)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < a.count; e += stride) {
        int64_t tbin;
        const int64_t row = event_index(a, e, tbin);
        if (row < 0) continue;
        const int64_t i = row * a.T + tbin;
        out[i] = SUM ? base[i] + value : value;
    }
}

__global__ void __launch_bounds__(256)
bin_events_packed_kernel(unsigned *__restrict__ bits, EventArgs a, int words)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < a.count; e += stride) {
        int64_t tbin;
        const int64_t row = event_index(a, e, tbin);
        if (row < 0) continue;
        atomicOr(bits + row * words + (tbin >> 5), 1u << (tbin & 31));
    }
}

static int check_event_args(const char *name, const EventArgs &a, const void *out)
{
    SB200_REQUIRE(a.count >= 0 && a.N >= 0 && a.C >= 0 && a.H >= 0 && a.W >= 0 && a.T >= 0, "%s: negative size", name);
    SB200_REQUIRE(a.samplingTime > 0.0, "%s: samplingTime must be positive", name);
    if (a.count == 0 || a.N * a.C * a.H * a.W * a.T == 0) return 1;       // nothing to do
    SB200_REQUIRE(out && a.x && a.p && a.t, "%s: null pointer", name);
    return SLAYER_B200_OK;
}

static unsigned event_grid(int64_t count)
{
    int64_t blocks = ceil_div(count, 256);
    const int64_t cap = (int64_t)sm_count() * 16;
    return (unsigned)(blocks > cap ? cap : blocks);
}

}  // namespace sb200

extern "C" int slayer_b200_bin_events(float *out, const float *base, const int32_t *n, const int32_t *x, const int32_t *y,
                                      const int32_t *p, const double *t, int64_t nEvents,
                                      int64_t N, int64_t C, int64_t H, int64_t W, int64_t T,
                                      double samplingTime, int64_t tStart, int sum_mode, void *stream)
{
    using namespace sb200;
    clear_error();
    const EventArgs a = {n, x, y, p, t, nEvents, N, C, H, W, T, samplingTime, tStart};
    int rc = check_event_args("bin_events", a, out);
    if (rc) return rc < 0 ? rc : SLAYER_B200_OK;
    SB200_REQUIRE(!sum_mode || (base && base != out), "bin_events: SUM mode reads the original tensor from `base`, which must not be `out`");
    const float value = (float)(1.0 / samplingTime);
    if (sum_mode) bin_events_kernel<true><<<event_grid(nEvents), 256, 0, (cudaStream_t)stream>>>(out, base, a, value);
    else bin_events_kernel<false><<<event_grid(nEvents), 256, 0, (cudaStream_t)stream>>>(out, nullptr, a, value);
    return check_launch("bin_events kernel launch");
}

extern "C" int slayer_b200_bin_events_packed(uint32_t *bits, const int32_t *n, const int32_t *x, const int32_t *y,
                                             const int32_t *p, const double *t, int64_t nEvents,
                                             int64_t N, int64_t C, int64_t H, int64_t W, int64_t T,
                                             double samplingTime, int64_t tStart, void *stream)
{
    using namespace sb200;
    clear_error();
    const EventArgs a = {n, x, y, p, t, nEvents, N, C, H, W, T, samplingTime, tStart};
    int rc = check_event_args("bin_events_packed", a, bits);
    if (rc) return rc < 0 ? rc : SLAYER_B200_OK;
    bin_events_packed_kernel<<<event_grid(nEvents), 256, 0, (cudaStream_t)stream>>>(bits, a, (int)((T + 31) >> 5));
    return check_launch("bin_events_packed kernel launch");
}
