// Python module `slayerLoihiCuda`: the reference's Loihi operator
// (src/cuda/slayerLoihiKernels.cu:12-51) on top of the slayer_b200 C ABI.
#include <vector>

#include "bindings_common.h"

using namespace sb200py;

static std::vector<torch::Tensor> getSpikesCuda(torch::Tensor weightedSpikes, const unsigned wgtExp,
                                                const unsigned theta, const unsigned iDecay,
                                                const unsigned vDecay, const unsigned refDelay)
{
    check_input(weightedSpikes, "weightedSpikes");
    c10::cuda::CUDAGuard guard(weightedSpikes.device());
    auto current = torch::empty_like(weightedSpikes);
    auto voltage = torch::empty_like(weightedSpikes);
    auto spike = torch::empty_like(weightedSpikes);
    const int64_t T = weightedSpikes.size(-1);
    const int64_t rows = T ? weightedSpikes.numel() / T : 0;
    check_rc(slayer_b200_loihi_get_spikes(spike.data_ptr<float>(), voltage.data_ptr<float>(),
                                          current.data_ptr<float>(), weightedSpikes.data_ptr<float>(),
                                          rows, T, wgtExp, theta, iDecay, vDecay, refDelay, current_stream()),
             "getSpikes");
    return {spike, voltage, current};
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
    m.def("getSpikes", &getSpikesCuda, "Get spikes for Loihi neuron (CUDA)");
    m.attr("backend") = "slayer_b200";
}
