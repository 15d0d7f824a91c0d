// Tensor-memory-accelerator (bulk tensor copy) helpers: host-side descriptor encoding and the
// PTX wrappers the kernels use.  Everything here moves tiles of a GPU's own memory; nothing is
// multicast and no descriptor ever covers another GPU's memory.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace sb200 {

// Describe a row-major [rows, T] fp32 array for 2-D tiled copies of [box_rows x box_cols]
// boxes with the given shared-memory swizzle.  Requires a 16-byte aligned base and T % 4 == 0
// (the row pitch must be a multiple of 16 bytes).  Returns false when the driver entry point
// is unavailable or the encoding is rejected, in which case callers use their cp.async path.
bool encode_rows_tensor_map(CUtensorMap *map, const float *base, int64_t rows, int64_t T,
                            unsigned box_cols, unsigned box_rows, CUtensorMapSwizzle swizzle);

// Device-side status word (one per device, owned by the library).  Kernels that wait on a
// barrier give up after a bounded number of polls and record a non-zero code here instead of
// hanging; slayer_b200_device_status() reads and clears it.
int *device_status_word();

constexpr int kStatusSrmLoadTimeout = 0x5101;

// false after slayer_b200_set_tma(0): kernels then use their cp.async paths
bool tma_enabled();

#ifdef __CUDACC__
__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// make barrier initialisation visible to the asynchronous proxy before the first copy uses it
__device__ __forceinline__ void mbar_init_fence()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, unsigned parity)
{
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Poll a barrier at most `limit` times.  Returns false if the phase did not complete.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, unsigned parity, int limit)
{
    for (int i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// global -> shared box load; completion is signalled on `bar` as transferred bytes
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// order this thread's shared-memory accesses before later asynchronous-proxy accesses to the
// same locations (a bulk load that refills a tile this thread has just read)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
#endif

}  // namespace sb200
