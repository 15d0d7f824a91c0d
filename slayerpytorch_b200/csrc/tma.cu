// Host side of the bulk-tensor-copy support: descriptor encoding through the driver entry
// point (no link-time dependency on the driver library), the per-device status word, and the
// switch that lets callers and tests turn the bulk-tensor path off.
#include <atomic>
#include <mutex>

#include "tma.cuh"

namespace sb200 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            (void)cudaGetLastError();
    });
    return fn;
}

bool encode_rows_tensor_map(CUtensorMap *map, const float *base, int64_t rows, int64_t T,
                            unsigned box_cols, unsigned box_rows, CUtensorMapSwizzle swizzle)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn || rows <= 0 || T <= 0 || (T & 3) || !aligned16(base)) return false;
    if (rows > 0xffffffffLL || T > 0xffffffffLL) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)T, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)T * sizeof(float)};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

static std::mutex g_status_mu;
static int *g_status[64] = {nullptr};

int *device_status_word()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_status_mu);
    if (!g_status[dev]) {
        int *p = nullptr;
        if (cudaMalloc(&p, 256) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
        if (cudaMemset(p, 0, 256) != cudaSuccess) { (void)cudaGetLastError(); cudaFree(p); return nullptr; }
        g_status[dev] = p;
    }
    return g_status[dev];
}

// One thread waits, a bounded number of polls, for a barrier phase that nothing will ever
// complete (it expects 16 bytes that no copy sends), then records the code a lost bulk copy
// would record and returns.  No copy is in flight and nothing faults or spins without limit:
// this is how the give-up branch of the bounded waits is exercised on real hardware.
__global__ void bounded_wait_selftest_kernel(int *status, int polls)
{
    __shared__ uint64_t bar;
    if (threadIdx.x != 0) return;
    mbar_init(&bar, 1);
    mbar_init_fence();
    mbar_expect_tx(&bar, 16);
    if (!mbar_wait_bounded(&bar, 0u, polls)) atomicExch(status, kStatusSrmLoadTimeout);
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
}

static std::atomic<int> g_use_tma{1};

bool tma_enabled() { return g_use_tma.load() != 0; }

}  // namespace sb200

extern "C" int slayer_b200_set_tma(int enable)
{
    return sb200::g_use_tma.exchange(enable ? 1 : 0);
}

extern "C" int slayer_b200_device_status(int *status_out)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(status_out != nullptr, "device_status: null pointer");
    int *word = device_status_word();
    if (!word) { set_error("device_status: no status word on this device"); return SLAYER_B200_ECUDA; }
    int value = 0;
    cudaError_t e = cudaMemcpy(&value, word, sizeof(int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && value != 0) e = cudaMemset(word, 0, sizeof(int));
    if (e != cudaSuccess) { set_error("device_status: %s", cudaGetErrorString(e)); return SLAYER_B200_ECUDA; }
    *status_out = value;
    return SLAYER_B200_OK;
}

extern "C" int slayer_b200_selftest_bounded_wait(int polls, void *stream)
{
    using namespace sb200;
    clear_error();
    SB200_REQUIRE(polls >= 1 && polls <= (1 << 20), "selftest_bounded_wait: polls must be in [1, 2^20]");
    int *word = device_status_word();
    if (!word) { set_error("selftest_bounded_wait: no status word on this device"); return SLAYER_B200_ECUDA; }
    bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(word, polls);
    return check_launch("selftest_bounded_wait kernel launch");
}
