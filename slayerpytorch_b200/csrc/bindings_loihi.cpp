// Python module `slayerLoihiCuda`: the reference's Loihi operator
// (src/cuda/slayerLoihiKernels.cu:12-51) on top of the slayer_b200 C ABI, plus getSpikesDelayed
// (the operator followed by the delay every Loihi layer applies, as one launch).
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

// getSpikes followed by a delay of `delay` >= 0 time steps on the spikes, which are written once,
// already delayed; returns [delayedSpike, voltage] or, with wantCurrent, [delayedSpike, voltage,
// current].  Sizes the fused kernel does not take run as getSpikes + shift.
static std::vector<torch::Tensor> getSpikesDelayedCuda(torch::Tensor weightedSpikes, const unsigned wgtExp,
                                                       const unsigned theta, const unsigned iDecay,
                                                       const unsigned vDecay, const unsigned refDelay,
                                                       const int64_t delay, const bool wantCurrent)
{
    check_input(weightedSpikes, "weightedSpikes");
    TORCH_CHECK(delay >= 0, "delay must be >= 0 time steps");
    c10::cuda::CUDAGuard guard(weightedSpikes.device());
    auto voltage = torch::empty_like(weightedSpikes);
    auto delayed = torch::empty_like(weightedSpikes);
    torch::Tensor current;
    if (wantCurrent) current = torch::empty_like(weightedSpikes);
    const int64_t T = weightedSpikes.size(-1);
    const int64_t rows = T ? weightedSpikes.numel() / T : 0;
    int rc = slayer_b200_loihi_get_spikes_delayed(delayed.data_ptr<float>(), voltage.data_ptr<float>(),
                                                  wantCurrent ? current.data_ptr<float>() : nullptr,
                                                  weightedSpikes.data_ptr<float>(), rows, T, wgtExp, theta, iDecay, vDecay,
                                                  refDelay, delay, current_stream());
    if (rc == SLAYER_B200_EUNSUPPORTED) {
        if (!wantCurrent) current = torch::empty_like(weightedSpikes);
        auto spike = torch::empty_like(weightedSpikes);
        check_rc(slayer_b200_loihi_get_spikes(spike.data_ptr<float>(), voltage.data_ptr<float>(), current.data_ptr<float>(),
                                              weightedSpikes.data_ptr<float>(), rows, T, wgtExp, theta, iDecay, vDecay,
                                              refDelay, current_stream()),
                 "getSpikesDelayed");
        rc = slayer_b200_shift_scalar(delayed.data_ptr<float>(), spike.data_ptr<float>(), (float)delay, rows, T, 1.0f,
                                      current_stream());
    }
    check_rc(rc, "getSpikesDelayed");
    if (wantCurrent) return {delayed, voltage, current};
    return {delayed, voltage};
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
    m.def("getSpikes", &getSpikesCuda, "Get spikes for Loihi neuron (CUDA)");
    m.def("getSpikesDelayed", &getSpikesDelayedCuda, "Get spikes for Loihi neuron, written already delayed (CUDA)",
          pybind11::arg("weightedSpikes"), pybind11::arg("wgtExp"), pybind11::arg("theta"), pybind11::arg("iDecay"),
          pybind11::arg("vDecay"), pybind11::arg("refDelay"), pybind11::arg("delay"), pybind11::arg("wantCurrent") = false);
    m.attr("backend") = "slayer_b200";
}
