// Python module `slayerCuda`: the reference's operator names and signatures
// (src/cuda/slayerKernels.cu:136-145) on top of the slayer_b200 C ABI.
//
// Differences from the reference shim, all deliberate:
//   - work is enqueued on PyTorch's current stream under a device guard (the reference uses
//     the legacy default stream and leaves the device switched);
//   - a one-element shift tensor is read on the device (no host synchronisation);
//   - the per-neuron shift covers the whole batch in one launch;
//   - dtype is checked explicitly;
//   - additional operators are exported: spikeGrad, spikeGrad_ (in place), spikeGradShift, corrSpikeGrad,
//     getSpikesDelayed, delayGrad, the bit-packed spike operators packSpikes, unpackSpikes,
//     getSpikesPacked and convPacked (packed tensors are int32, [..., ceil(T / 32)]), and the
//     event binning binEvents / binEventsPacked.
#include "bindings_common.h"

using namespace sb200py;

static torch::Tensor getSpikesCuda(torch::Tensor d_u, const torch::Tensor &d_nu, const float theta, const float Ts)
{
    check_input(d_u, "d_u");
    check_input(d_nu, "d_nu");
    check_device(d_u, d_nu, "d_u", "d_nu");
    TORCH_CHECK_INDEX(d_u.dim() >= 4, "getSpikes expects a tensor with at least 4 dimensions (NCHWT), got ", d_u.dim());
    c10::cuda::CUDAGuard guard(d_u.device());
    auto d_s = torch::empty_like(d_u);
    const int64_t Ns = d_u.size(-1);
    const int64_t rows = Ns ? d_u.numel() / Ns : 0;
    const int64_t nuSize = d_nu.dim() ? d_nu.size(-1) : 1;
    check_rc(slayer_b200_srm_get_spikes(d_s.data_ptr<float>(), d_u.data_ptr<float>(), d_nu.data_ptr<float>(),
                                        rows, nuSize, Ns, theta, Ts, current_stream()),
             "getSpikes");
    return d_s;
}

// shift(getSpikes(d_u, d_nu, theta, Ts), delayLUT, Ts) with the spikes written once, already
// delayed; d_u is updated in place like getSpikes does.  delayLUT: one value per neuron or a
// single value.  Sizes the fused kernel does not take run as the two operators.
static torch::Tensor getSpikesDelayedCuda(torch::Tensor d_u, const torch::Tensor &d_nu, const float theta, const float Ts,
                                          torch::Tensor delayLUT)
{
    check_input(d_u, "d_u");
    check_input(d_nu, "d_nu");
    check_input(delayLUT, "delayLUT");
    check_device(d_u, d_nu, "d_u", "d_nu");
    check_device(d_u, delayLUT, "d_u", "delayLUT");
    TORCH_CHECK_INDEX(d_u.dim() >= 4, "getSpikesDelayed expects a tensor with at least 4 dimensions (NCHWT), got ", d_u.dim());
    c10::cuda::CUDAGuard guard(d_u.device());
    auto delayed = torch::empty_like(d_u);
    const int64_t Ns = d_u.size(-1);
    const int64_t rows = Ns ? d_u.numel() / Ns : 0;
    const int64_t nuSize = d_nu.dim() ? d_nu.size(-1) : 1;
    int64_t nBatch = rows, nNeurons = 1;
    if (delayLUT.numel() != 1) {
        nBatch = d_u.size(0);
        nNeurons = nBatch ? rows / nBatch : 0;
        TORCH_CHECK(delayLUT.numel() == nNeurons, "shift and number of neurons must be same");
    }
    int rc = slayer_b200_srm_get_spikes_delayed(delayed.data_ptr<float>(), nullptr, d_u.data_ptr<float>(),
                                                d_nu.data_ptr<float>(), delayLUT.data_ptr<float>(), 0.0f,
                                                nBatch, nNeurons, nuSize, Ns, theta, Ts, current_stream());
    if (rc == SLAYER_B200_EUNSUPPORTED) {
        auto scratch = torch::empty_like(d_u);
        rc = slayer_b200_srm_get_spikes_delayed(delayed.data_ptr<float>(), scratch.data_ptr<float>(), d_u.data_ptr<float>(),
                                                d_nu.data_ptr<float>(), delayLUT.data_ptr<float>(), 0.0f,
                                                nBatch, nNeurons, nuSize, Ns, theta, Ts, current_stream());
    }
    check_rc(rc, "getSpikesDelayed");
    return delayed;
}

static torch::Tensor convCuda(torch::Tensor input, torch::Tensor filter, float Ts)
{
    check_input(input, "input");
    check_input(filter, "filter");
    check_device(input, filter, "input", "filter");
    c10::cuda::CUDAGuard guard(input.device());
    auto output = torch::empty_like(input);
    const int64_t T = input.size(-1);
    const int64_t rows = T ? input.numel() / T : 0;
    check_rc(slayer_b200_conv(output.data_ptr<float>(), input.data_ptr<float>(), filter.data_ptr<float>(),
                              rows, T, filter.numel(), Ts, current_stream()),
             "conv");
    return output;
}

static torch::Tensor corrCuda(torch::Tensor input, torch::Tensor filter, float Ts)
{
    check_input(input, "input");
    check_input(filter, "filter");
    check_device(input, filter, "input", "filter");
    c10::cuda::CUDAGuard guard(input.device());
    auto output = torch::empty_like(input);
    const int64_t T = input.size(-1);
    const int64_t rows = T ? input.numel() / T : 0;
    check_rc(slayer_b200_corr(output.data_ptr<float>(), input.data_ptr<float>(), filter.data_ptr<float>(),
                              rows, T, filter.numel(), Ts, current_stream()),
             "corr");
    return output;
}

// spikeGrad(corr(gradOutput, filter, Ts), membranePotential, ...) in one pass: the backward step
// of a psp filter that follows a spike layer (src/slayer.py:892, then :862).
static torch::Tensor corrSpikeGradCuda(torch::Tensor gradOut, torch::Tensor filter, torch::Tensor u,
                                       float theta, float tau, float scale, float Ts)
{
    check_input(gradOut, "gradOutput");
    check_input(filter, "filter");
    check_input(u, "membranePotential");
    check_device(gradOut, filter, "gradOutput", "filter");
    check_device(gradOut, u, "gradOutput", "membranePotential");
    TORCH_CHECK(gradOut.sizes() == u.sizes(), "gradOutput and membranePotential must have the same shape");
    c10::cuda::CUDAGuard guard(gradOut.device());
    auto output = torch::empty_like(gradOut);
    const int64_t T = gradOut.dim() ? gradOut.size(-1) : 0;
    const int64_t rows = T ? gradOut.numel() / T : 0;
    check_rc(slayer_b200_corr_spike_grad(output.data_ptr<float>(), gradOut.data_ptr<float>(), filter.data_ptr<float>(),
                                         u.data_ptr<float>(), rows, T, filter.numel(), Ts, theta, tau, scale, current_stream()),
             "corrSpikeGrad");
    return output;
}

static torch::Tensor shiftCuda(torch::Tensor input, torch::Tensor shiftLUT, float Ts)
{
    check_input(input, "input");
    check_input(shiftLUT, "shiftLUT");
    check_device(input, shiftLUT, "input", "shiftLUT");
    c10::cuda::CUDAGuard guard(input.device());
    auto output = torch::empty_like(input);
    const int64_t T = input.size(-1);
    const int64_t rows = T ? input.numel() / T : 0;
    if (shiftLUT.numel() == 1) {
        // same amount for every row; the value stays on the device
        check_rc(slayer_b200_shift_lut(output.data_ptr<float>(), input.data_ptr<float>(),
                                       shiftLUT.data_ptr<float>(), rows, 1, T, Ts, current_stream()),
                 "shift");
    } else {
        const int64_t nBatch = input.size(0);
        const int64_t nNeurons = nBatch ? rows / nBatch : 0;
        TORCH_CHECK(shiftLUT.numel() == nNeurons, "shift and number of neurons must be same");
        check_rc(slayer_b200_shift_lut(output.data_ptr<float>(), input.data_ptr<float>(),
                                       shiftLUT.data_ptr<float>(), nBatch, nNeurons, T, Ts, current_stream()),
                 "shift");
    }
    return output;
}

static torch::Tensor shift1Cuda(torch::Tensor input, torch::Tensor shiftLUT) { return shiftCuda(input, shiftLUT, 1.0f); }

static torch::Tensor shiftFlCuda(torch::Tensor input, float shiftValue, float Ts)
{
    check_input(input, "input");
    c10::cuda::CUDAGuard guard(input.device());
    auto output = torch::empty_like(input);
    const int64_t T = input.size(-1);
    const int64_t rows = T ? input.numel() / T : 0;
    check_rc(slayer_b200_shift_scalar(output.data_ptr<float>(), input.data_ptr<float>(), shiftValue,
                                      rows, T, Ts, current_stream()),
             "shift");
    return output;
}

static torch::Tensor shiftFl1Cuda(torch::Tensor input, float shiftValue) { return shiftFlCuda(input, shiftValue, 1.0f); }

static torch::Tensor spikeGradImpl(torch::Tensor out, const torch::Tensor &gradOut, const torch::Tensor &u,
                                   float theta, float tau, float scale)
{
    check_input(gradOut, "gradOutput");
    check_input(u, "membranePotential");
    check_device(gradOut, u, "gradOutput", "membranePotential");
    TORCH_CHECK(gradOut.numel() == u.numel(), "gradOutput and membranePotential must have the same number of elements");
    c10::cuda::CUDAGuard guard(gradOut.device());
    check_rc(slayer_b200_spike_grad(out.data_ptr<float>(), gradOut.data_ptr<float>(), u.data_ptr<float>(),
                                    gradOut.numel(), theta, tau, scale, current_stream()),
             "spikeGrad");
    return out;
}

static torch::Tensor spikeGradCuda(torch::Tensor gradOut, torch::Tensor u, float theta, float tau, float scale)
{
    return spikeGradImpl(torch::empty_like(gradOut), gradOut, u, theta, tau, scale);
}

static torch::Tensor spikeGradInplaceCuda(torch::Tensor gradOut, torch::Tensor u, float theta, float tau, float scale)
{
    return spikeGradImpl(gradOut, gradOut, u, theta, tau, scale);
}

// spikeGrad(shift(gradOutput, shiftLUT, Ts), membranePotential, ...) in one pass: the backward
// step of a spike layer followed by a delay.  shiftLUT is the shift to apply to the gradient
// (minus the forward delay): one value per neuron, or a single value for all rows.
static torch::Tensor spikeGradShiftCuda(torch::Tensor gradOut, torch::Tensor u, torch::Tensor shiftLUT,
                                        float theta, float tau, float scale, float Ts)
{
    check_input(gradOut, "gradOutput");
    check_input(u, "membranePotential");
    check_input(shiftLUT, "shiftLUT");
    check_device(gradOut, u, "gradOutput", "membranePotential");
    check_device(gradOut, shiftLUT, "gradOutput", "shiftLUT");
    TORCH_CHECK(gradOut.sizes() == u.sizes(), "gradOutput and membranePotential must have the same shape");
    TORCH_CHECK(gradOut.dim() >= 2, "spikeGradShift expects [batch, ..., time] tensors");
    c10::cuda::CUDAGuard guard(gradOut.device());
    auto output = torch::empty_like(gradOut);
    const int64_t T = gradOut.size(-1);
    const int64_t rows = T ? gradOut.numel() / T : 0;
    int64_t nBatch = rows, nNeurons = 1;
    if (shiftLUT.numel() != 1) {
        nBatch = gradOut.size(0);
        nNeurons = nBatch ? rows / nBatch : 0;
        TORCH_CHECK(shiftLUT.numel() == nNeurons, "shift and number of neurons must be same");
    }
    check_rc(slayer_b200_spike_grad_shift(output.data_ptr<float>(), gradOut.data_ptr<float>(), u.data_ptr<float>(),
                                          shiftLUT.data_ptr<float>(), 0.0f, nBatch, nNeurons, T, Ts, theta, tau, scale,
                                          current_stream()),
             "spikeGradShift");
    return output;
}

// gradDelay of _delayFunction.backward (src/slayer.py:950-954) in one pass; the result has the
// shape of gradOutput without its first (batch) and last (time) dimension.
static torch::Tensor delayGradCuda(torch::Tensor gradOut, torch::Tensor output, float Ts)
{
    check_input(gradOut, "gradOutput");
    check_input(output, "output");
    check_device(gradOut, output, "gradOutput", "output");
    TORCH_CHECK(gradOut.sizes() == output.sizes(), "gradOutput and output must have the same shape");
    TORCH_CHECK(gradOut.dim() >= 2, "delayGrad expects [batch, ..., time] tensors");
    c10::cuda::CUDAGuard guard(gradOut.device());
    const int64_t nBatch = gradOut.size(0), T = gradOut.size(-1);
    auto shape = gradOut.sizes().slice(1, gradOut.dim() - 2);
    if (nBatch == 0 || T == 0) return torch::zeros(shape, gradOut.options());
    const int64_t nNeurons = gradOut.numel() / (nBatch * T);
    auto result = torch::empty(shape, gradOut.options());   // every element is written by the kernel
    if (nNeurons > 0)
        check_rc(slayer_b200_delay_grad(result.data_ptr<float>(), gradOut.data_ptr<float>(), output.data_ptr<float>(),
                                        nBatch, nNeurons, T, Ts, current_stream()),
                 "delayGrad");
    return result;
}

// ---------------------------------------------------------------- bit-packed spike tensors
static std::vector<int64_t> packed_shape(const torch::Tensor &like)
{
    auto shape = like.sizes().vec();
    shape.back() = (shape.back() + 31) / 32;
    return shape;
}

static void check_packed(const torch::Tensor &bits, const char *name)
{
    TORCH_CHECK(bits.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(bits.is_contiguous(), name, " must be contiguous");
    TORCH_CHECK(bits.scalar_type() == torch::kInt32, name, " must be an int32 tensor");
}

// bit i of word w of a row = (spikes[..., 32 w + i] != 0)
static torch::Tensor packSpikesCuda(torch::Tensor spikes)
{
    check_input(spikes, "spikes");
    TORCH_CHECK(spikes.dim() >= 1, "packSpikes expects a tensor with a time dimension");
    c10::cuda::CUDAGuard guard(spikes.device());
    auto bits = torch::empty(packed_shape(spikes), spikes.options().dtype(torch::kInt32));
    const int64_t T = spikes.size(-1);
    const int64_t rows = T ? spikes.numel() / T : 0;
    check_rc(slayer_b200_pack_spikes(reinterpret_cast<uint32_t *>(bits.data_ptr<int32_t>()), spikes.data_ptr<float>(),
                                     rows, T, current_stream()),
             "packSpikes");
    return bits;
}

// fp32 view of a packed spike tensor: `value` where a bit is set, 0 elsewhere; T = row length
static torch::Tensor unpackSpikesCuda(torch::Tensor bits, int64_t T, float value)
{
    check_packed(bits, "bits");
    TORCH_CHECK(bits.dim() >= 1 && bits.size(-1) == (T + 31) / 32, "unpackSpikes: the last dimension must be ceil(T / 32)");
    c10::cuda::CUDAGuard guard(bits.device());
    auto shape = bits.sizes().vec();
    shape.back() = T;
    auto spikes = torch::empty(shape, bits.options().dtype(torch::kFloat32));
    const int64_t words = bits.size(-1);
    const int64_t rows = words ? bits.numel() / words : 0;
    check_rc(slayer_b200_unpack_spikes(spikes.data_ptr<float>(), reinterpret_cast<const uint32_t *>(bits.data_ptr<int32_t>()),
                                       rows, T, value, current_stream()),
             "unpackSpikes");
    return spikes;
}

// getSpikes with the spikes returned packed; d_u is updated in place like getSpikes does
static torch::Tensor getSpikesPackedCuda(torch::Tensor d_u, const torch::Tensor &d_nu, const float theta, const float Ts)
{
    check_input(d_u, "d_u");
    check_input(d_nu, "d_nu");
    check_device(d_u, d_nu, "d_u", "d_nu");
    TORCH_CHECK_INDEX(d_u.dim() >= 4, "getSpikesPacked expects a tensor with at least 4 dimensions (NCHWT), got ", d_u.dim());
    c10::cuda::CUDAGuard guard(d_u.device());
    auto bits = torch::empty(packed_shape(d_u), d_u.options().dtype(torch::kInt32));
    const int64_t Ns = d_u.size(-1);
    const int64_t rows = Ns ? d_u.numel() / Ns : 0;
    const int64_t nuSize = d_nu.dim() ? d_nu.size(-1) : 1;
    uint32_t *words = reinterpret_cast<uint32_t *>(bits.data_ptr<int32_t>());
    int rc = slayer_b200_srm_get_spikes_packed(words, d_u.data_ptr<float>(), d_nu.data_ptr<float>(), rows, nuSize, Ns, theta,
                                               current_stream());
    if (rc == SLAYER_B200_EUNSUPPORTED) {       // sizes the packed kernel does not take: the two steps
        auto d_s = torch::empty_like(d_u);
        check_rc(slayer_b200_srm_get_spikes(d_s.data_ptr<float>(), d_u.data_ptr<float>(), d_nu.data_ptr<float>(),
                                            rows, nuSize, Ns, theta, Ts, current_stream()),
                 "getSpikesPacked");
        rc = slayer_b200_pack_spikes(words, d_s.data_ptr<float>(), rows, Ns, current_stream());
    }
    check_rc(rc, "getSpikesPacked");
    return bits;
}

// conv(unpackSpikes(bits, T, value), filter, Ts) without the fp32 spike tensor
static torch::Tensor convPackedCuda(torch::Tensor bits, int64_t T, torch::Tensor filter, float Ts, float value)
{
    check_packed(bits, "bits");
    check_input(filter, "filter");
    TORCH_CHECK(bits.device().index() == filter.device().index(), "bits and filter must be in same CUDA device");
    TORCH_CHECK(bits.dim() >= 1 && bits.size(-1) == (T + 31) / 32, "convPacked: the last dimension must be ceil(T / 32)");
    c10::cuda::CUDAGuard guard(bits.device());
    auto shape = bits.sizes().vec();
    shape.back() = T;
    auto output = torch::empty(shape, bits.options().dtype(torch::kFloat32));
    const int64_t words = bits.size(-1);
    const int64_t rows = words ? bits.numel() / words : 0;
    const uint32_t *w = reinterpret_cast<const uint32_t *>(bits.data_ptr<int32_t>());
    int rc = slayer_b200_conv_packed(output.data_ptr<float>(), w, filter.data_ptr<float>(), rows, T, filter.numel(), value, Ts,
                                     current_stream());
    if (rc == SLAYER_B200_EUNSUPPORTED) {       // very long filter: the two steps
        auto spikes = torch::empty_like(output);
        check_rc(slayer_b200_unpack_spikes(spikes.data_ptr<float>(), w, rows, T, value, current_stream()), "convPacked");
        rc = slayer_b200_conv(output.data_ptr<float>(), spikes.data_ptr<float>(), filter.data_ptr<float>(), rows, T,
                              filter.numel(), Ts, current_stream());
    }
    check_rc(rc, "convPacked");
    return output;
}

// ------------------------------------------------------------------------ spike-count loss
// Returns (sum over rows and time of e^2 as a float64 0-dim tensor, d loss / d spikes for a unit
// upstream gradient); the caller scales by Ts / 2.  desiredCount: one value per [batch, class] row.
static std::vector<torch::Tensor> numSpikesLossCuda(torch::Tensor spikes, torch::Tensor desiredCount, torch::Tensor filter,
                                                    int64_t start, int64_t stop, float Ts, float scale)
{
    check_input(spikes, "spikes");
    check_input(desiredCount, "desiredCount");
    check_input(filter, "filter");
    check_device(spikes, desiredCount, "spikes", "desiredCount");
    check_device(spikes, filter, "spikes", "filter");
    TORCH_CHECK(spikes.dim() >= 2, "numSpikesLoss expects [batch, ..., time] spikes");
    const int64_t T = spikes.size(-1);
    const int64_t rows = T ? spikes.numel() / T : 0;
    TORCH_CHECK(desiredCount.numel() == rows, "desiredCount must hold one value per row of spikes");
    c10::cuda::CUDAGuard guard(spikes.device());
    auto grad = torch::empty_like(spikes);
    auto row_sq = torch::empty({rows}, spikes.options().dtype(torch::kFloat64));
    check_rc(slayer_b200_num_spikes_loss(grad.data_ptr<float>(), row_sq.data_ptr<double>(), spikes.data_ptr<float>(),
                                         desiredCount.data_ptr<float>(), filter.data_ptr<float>(), rows, T, filter.numel(),
                                         start, stop, Ts, scale, current_stream()),
             "numSpikesLoss");
    return {row_sq.sum(), grad};
}

// ------------------------------------------------------------------ address events -> tensor
static void check_events(const torch::Tensor &v, const char *name, torch::ScalarType dtype, int64_t count, const torch::Tensor &like)
{
    TORCH_CHECK(v.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(v.is_contiguous(), name, " must be contiguous");
    TORCH_CHECK(v.scalar_type() == dtype, name, " has the wrong dtype (x, y, p, n: int32; t: float64)");
    TORCH_CHECK(v.numel() == count, name, " must have one entry per event");
    TORCH_CHECK(v.device().index() == like.device().index(), name, " must be on the device of the tensor");
}

// Events (x, y, p, t [, n]) binned into `tensor` ([C, H, W, T], or [N, C, H, W, T] with a sample
// index n per event): mode 0 sets bins to 1/samplingTime in place and returns `tensor`; mode 1
// returns a new tensor with 1/samplingTime added once to every bin that receives events.
static torch::Tensor binEventsCuda(torch::Tensor tensor, torch::Tensor x, c10::optional<torch::Tensor> y, torch::Tensor p,
                                   torch::Tensor t, c10::optional<torch::Tensor> n, double samplingTime, int64_t tStart,
                                   int64_t mode)
{
    check_input(tensor, "tensor");
    TORCH_CHECK(tensor.dim() == 4 || tensor.dim() == 5, "binEvents expects a CHWT or NCHWT tensor");
    TORCH_CHECK(mode == 0 || mode == 1, "mode must be 0 (OR) or 1 (SUM)");
    const int64_t count = x.numel();
    check_events(x, "x", torch::kInt32, count, tensor);
    check_events(p, "p", torch::kInt32, count, tensor);
    check_events(t, "t", torch::kFloat64, count, tensor);
    if (y.has_value()) check_events(*y, "y", torch::kInt32, count, tensor);
    if (n.has_value()) check_events(*n, "n", torch::kInt32, count, tensor);
    TORCH_CHECK(tensor.dim() == 5 || !n.has_value(), "a sample index needs an NCHWT tensor");
    c10::cuda::CUDAGuard guard(tensor.device());
    const int d = tensor.dim() == 5 ? 1 : 0;
    const int64_t N = d ? tensor.size(0) : 1;
    auto out = mode == 1 ? tensor.clone() : tensor;
    check_rc(slayer_b200_bin_events(out.data_ptr<float>(), mode == 1 ? tensor.data_ptr<float>() : nullptr,
                                    n.has_value() ? n->data_ptr<int32_t>() : nullptr, x.data_ptr<int32_t>(),
                                    y.has_value() ? y->data_ptr<int32_t>() : nullptr, p.data_ptr<int32_t>(), t.data_ptr<double>(),
                                    count, N, tensor.size(d), tensor.size(d + 1), tensor.size(d + 2), tensor.size(d + 3),
                                    samplingTime, tStart, (int)mode, current_stream()),
             "binEvents");
    return out;
}

// The same binning ('OR') into a bit-packed spike tensor of the given CHWT / NCHWT shape.
static torch::Tensor binEventsPackedCuda(std::vector<int64_t> shape, torch::Tensor x, c10::optional<torch::Tensor> y,
                                         torch::Tensor p, torch::Tensor t, c10::optional<torch::Tensor> n,
                                         double samplingTime, int64_t tStart)
{
    TORCH_CHECK(shape.size() == 4 || shape.size() == 5, "binEventsPacked expects a CHWT or NCHWT shape");
    TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor");
    const int64_t count = x.numel();
    check_events(x, "x", torch::kInt32, count, x);
    check_events(p, "p", torch::kInt32, count, x);
    check_events(t, "t", torch::kFloat64, count, x);
    if (y.has_value()) check_events(*y, "y", torch::kInt32, count, x);
    if (n.has_value()) check_events(*n, "n", torch::kInt32, count, x);
    TORCH_CHECK(shape.size() == 5 || !n.has_value(), "a sample index needs an NCHWT shape");
    c10::cuda::CUDAGuard guard(x.device());
    const int d = shape.size() == 5 ? 1 : 0;
    const int64_t N = d ? shape[0] : 1;
    const int64_t T = shape.back();
    auto wshape = shape;
    wshape.back() = (T + 31) / 32;
    auto bits = torch::zeros(wshape, x.options().dtype(torch::kInt32));
    check_rc(slayer_b200_bin_events_packed(reinterpret_cast<uint32_t *>(bits.data_ptr<int32_t>()),
                                           n.has_value() ? n->data_ptr<int32_t>() : nullptr, x.data_ptr<int32_t>(),
                                           y.has_value() ? y->data_ptr<int32_t>() : nullptr, p.data_ptr<int32_t>(),
                                           t.data_ptr<double>(), count, N, shape[d], shape[d + 1], shape[d + 2], T,
                                           samplingTime, tStart, current_stream()),
             "binEventsPacked");
    return bits;
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
    m.def("getSpikes", &getSpikesCuda, "Get spikes (CUDA)");
    m.def("conv", &convCuda, "Convolution in time (CUDA)");
    m.def("corr", &corrCuda, "Correlation in time (CUDA)");
    m.def("shift", &shiftCuda, "Element shift in time (CUDA)");
    m.def("shift", &shift1Cuda, "Element shift in time (CUDA)");
    m.def("shift", &shiftFlCuda, "Element shift in time (CUDA)");
    m.def("shift", &shiftFl1Cuda, "Element shift in time (CUDA)");
    m.def("getSpikesDelayed", &getSpikesDelayedCuda, "Get spikes, written once and already delayed (CUDA)");
    m.def("spikeGrad", &spikeGradCuda,
          "gradOutput * scale/tau * exp(-|u - theta| / tau) in one pass (CUDA)");
    m.def("spikeGrad_", &spikeGradInplaceCuda, "In-place variant of spikeGrad (overwrites gradOutput)");
    m.def("spikeGradShift", &spikeGradShiftCuda, "Surrogate gradient of the time-shifted gradient in one pass (CUDA)");
    m.def("corrSpikeGrad", &corrSpikeGradCuda, "Correlation in time, then the surrogate gradient on its result, in one pass (CUDA)");
    m.def("delayGrad", &delayGradCuda, "Ts * sum over batch and time of gradOutput * d(output)/dt per neuron (CUDA)");
    m.def("packSpikes", &packSpikesCuda, "Spike tensor -> bit-packed int32 words, ceil(T / 32) per row (CUDA)");
    m.def("unpackSpikes", &unpackSpikesCuda, "Bit-packed spike tensor -> fp32 (value where a bit is set) (CUDA)");
    m.def("getSpikesPacked", &getSpikesPackedCuda, "Get spikes, returned bit-packed (CUDA)");
    m.def("convPacked", &convPackedCuda, "Convolution in time of a bit-packed spike tensor (CUDA)");
    m.def("numSpikesLoss", &numSpikesLossCuda, "Spike-count loss: sum of squared errors and gradient in one pass (CUDA)");
    m.def("binEvents", &binEventsCuda, "Address events -> spike tensor (CUDA)");
    m.def("binEventsPacked", &binEventsPackedCuda, "Address events -> bit-packed spike tensor (CUDA)");
    m.attr("backend") = "slayer_b200";
}
