// Helpers shared by the two Python extension modules (slayerCuda, slayerLoihiCuda).
#pragma once

#include <torch/extension.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include "slayer_b200.h"

namespace sb200py {

// The reference's CHECK_INPUT / CHECK_DEVICE (src/cuda/slayerKernels.cu:7-10) plus an explicit
// dtype check (the reference fails later, inside .data<float>(), for other dtypes).
inline void check_input(const torch::Tensor &x, const char *name)
{
    TORCH_CHECK(x.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(x.is_contiguous(), name, " must be contiguous");
    TORCH_CHECK(x.scalar_type() == torch::kFloat32, name, " must be a float32 tensor");
}

inline void check_device(const torch::Tensor &x, const torch::Tensor &y, const char *xn, const char *yn)
{
    TORCH_CHECK(x.device().index() == y.device().index(), xn, " and ", yn, " must be in same CUDA device");
}

inline void check_rc(int rc, const char *op)
{
    TORCH_CHECK(rc == SLAYER_B200_OK, op, " failed (", rc, "): ", slayer_b200_last_error());
}

inline void *current_stream() { return (void *)c10::cuda::getCurrentCUDAStream().stream(); }

}  // namespace sb200py
