"""Host-side mirror of the reference's spiking-layer interface for the hot path.

Same method names, argument meaning and tensor layout (``NCHWT`` float32, time last) as
``spikeLayer`` in the reference (src/slayer.py:47-391, src/slayerLoihi.py:16-210), restricted
to what the hot path needs: ``psp``, ``spike``, ``delayShift``, ``delay``, ``spikeLoihi``,
``spikeLoihiFull`` and a ``dense`` weight layer (plain PyTorch, as in the reference).

The autograd Functions below do what the reference's do (src/slayer.py:817-979,
src/slayerLoihi.py:243-283) on the operators of ``slayerCuda`` / ``slayerLoihiCuda``, with two
differences that do not change results beyond fp32 rounding of ``exp``:

* the surrogate-gradient backward is one fused kernel (``slayerCuda.spikeGrad``) instead of a
  chain of elementwise tensor operations;
* the delay gradient is one fused reduction (``slayerCuda.delayGrad``) instead of a two-tap
  conv, a product and a tensor sum;
* ``spikeDelayed`` (an addition to the interface) runs spike generation and the delay that
  follows it as one autograd node whose backward is a single pass (``slayerCuda.spikeGradShift``);
* scalars (``Ts``, ``theta`` ...) stay Python floats, so no backward pass synchronises the host
  to read a 0-dim device tensor.

The reference's own ``slayer.py`` / ``slayerLoihi.py`` also run unchanged on the same operator
modules; this mirror exists so that the package is usable (and benchmarkable) on its own.
"""
import math

import numpy as np
import torch
import torch.nn.functional as F

from . import load_ops

slayerCuda, slayerLoihiCuda = load_ops()


# ----------------------------------------------------------------------------- kernels
def alpha_kernel(tau, Ts, tSample, mult=1.0, epsilon=0.01):
    """Samples of mult * t/tau * exp(1 - t/tau) at t = 0, Ts, 2Ts, ..., cut where the tail
    drops below epsilon (src/slayer.py:114-123)."""
    taps = []
    for t in np.arange(0, tSample, Ts):
        value = mult * t / tau * math.exp(1 - t / tau)
        if abs(value) < epsilon and t > tau:
            break
        taps.append(value)
    return taps


def loihi_psp_kernel(neuron):
    """Impulse response of the Loihi current/voltage filter pair (src/slayerLoihi.py:66-79)."""
    keep_i = (1 << 12) - neuron['iDecay']
    keep_v = (1 << 12) - neuron['vDecay']
    u = 1 << (6 + neuron['wgtExp'] + 1)
    v = u
    out = [v]
    while v > 0:
        u = (u * keep_i) >> 12
        v = ((v * keep_v) >> 12) + u
        out.append(v)
    return [x / 2 for x in out]


def loihi_ref_kernel(neuron, scale=1000):
    """Refractory kernel equivalent of the Loihi reset (src/slayerLoihi.py:81-89)."""
    keep_v = (1 << 12) - neuron['vDecay']
    absolute = np.ones(neuron['refDelay']) * (-scale * neuron['theta'])
    absolute[0] = 0
    relative = [neuron['theta']]
    while relative[-1] > 0:
        relative.append((relative[-1] * keep_v) >> 12)
    return np.concatenate((absolute, -2 * np.array(relative))).astype('float32')


# ----------------------------------------------------------------------------- autograd
class _PspFunction(torch.autograd.Function):
    """psp forward = causal FIR, backward = its adjoint (src/slayer.py:875-899)."""

    @staticmethod
    def forward(ctx, spike, kernel, Ts):
        ctx.save_for_backward(kernel)
        ctx.Ts = float(Ts)
        return slayerCuda.conv(spike.contiguous(), kernel, ctx.Ts)

    @staticmethod
    def backward(ctx, grad):
        (kernel,) = ctx.saved_tensors
        return slayerCuda.corr(grad.contiguous(), kernel, ctx.Ts), None, None


class _SpikeFunction(torch.autograd.Function):
    """Spike generation; the membrane potential is updated in place and kept for the
    surrogate gradient (src/slayer.py:817-873)."""

    @staticmethod
    def forward(ctx, u, refKernel, neuron, Ts):
        u = u.contiguous()
        spikes = slayerCuda.getSpikes(u, refKernel, neuron['theta'], Ts)
        ctx.save_for_backward(u)
        ctx.theta = float(neuron['theta'])
        ctx.tau = float(neuron['tauRho'] * neuron['theta'])
        ctx.scale = float(neuron['scaleRho'])
        return spikes

    @staticmethod
    def backward(ctx, grad):
        (u,) = ctx.saved_tensors
        return slayerCuda.spikeGrad(grad.contiguous(), u, ctx.theta, ctx.tau, ctx.scale), None, None, None


class PackedSpikes:
    """A spike tensor stored as bits: ``bits`` is int32 of shape ``[..., ceil(T / 32)]``, bit i of
    word w = "spike at step 32 w + i"; a spike has the value ``value`` (1 / Ts).  1/32 of the
    bytes of the fp32 form; ``dense()`` gives that form back."""

    def __init__(self, bits, T, value):
        self.bits, self.T, self.value = bits, int(T), float(value)

    @property
    def shape(self):
        return tuple(self.bits.shape[:-1]) + (self.T,)

    def dense(self):
        return slayerCuda.unpackSpikes(self.bits, self.T, self.value)


class _SpikePspFunction(torch.autograd.Function):
    """psp(spike(u)) as one autograd node: the spikes go from the spike kernel to the psp filter
    as bits (1/8 byte per element instead of two fp32 passes) and are returned packed as a second,
    non-differentiable output.  Backward is the reference's - corr of the incoming gradient
    (src/slayer.py:892), then the surrogate gradient on the updated potential (src/slayer.py:862) -
    as one launch (corrSpikeGrad).  Same results as _PspFunction applied to _SpikeFunction."""

    @staticmethod
    def forward(ctx, u, srmKernel, refKernel, neuron, Ts):
        u = u.contiguous()
        Ts = float(Ts)
        bits = slayerCuda.getSpikesPacked(u, refKernel, neuron['theta'], Ts)
        out = slayerCuda.convPacked(bits, u.shape[-1], srmKernel, Ts, 1.0 / Ts)
        ctx.save_for_backward(u, srmKernel)
        ctx.theta = float(neuron['theta'])
        ctx.tau = float(neuron['tauRho'] * neuron['theta'])
        ctx.scale = float(neuron['scaleRho'])
        ctx.Ts = Ts
        ctx.mark_non_differentiable(bits)
        return out, bits

    @staticmethod
    def backward(ctx, grad, _grad_bits):
        u, srmKernel = ctx.saved_tensors
        g = slayerCuda.corrSpikeGrad(grad.contiguous(), srmKernel, u, ctx.theta, ctx.tau, ctx.scale, ctx.Ts)
        return g, None, None, None, None


class _DelayFunction(torch.autograd.Function):
    """Learnable per-neuron delay (src/slayer.py:930-957): forward shifts by the delay, backward
    shifts the gradient back and integrates gradient x finite-difference of the output."""

    @staticmethod
    def forward(ctx, x, delay, Ts):
        out = slayerCuda.shift(x.contiguous(), delay.data, Ts)
        ctx.save_for_backward(out, delay.data)
        ctx.Ts = float(Ts)
        return out

    @staticmethod
    def backward(ctx, grad):
        out, delay = ctx.saved_tensors
        Ts = ctx.Ts
        grad = grad.contiguous()
        grad_delay = slayerCuda.delayGrad(grad, out, Ts)      # one fused pass, no temporaries
        return slayerCuda.shift(grad, -delay, Ts), grad_delay.reshape(delay.shape), None


class _SpikeDelayFunction(torch.autograd.Function):
    """Spike generation followed by a per-neuron (or uniform) delay as one autograd node.

    Forward is ``getSpikesDelayed`` (the spikes are written once, already delayed); backward is one fused pass
    ``spikeGradShift`` (shifted gradient times surrogate gradient, src/slayer.py:957 and :862
    combined) plus, when the delay is learnable, the fused delay gradient.  Results equal those
    of ``_SpikeFunction`` followed by ``_DelayFunction`` / ``_DelayShiftFunction`` bit for bit."""

    @staticmethod
    def forward(ctx, u, refKernel, neuron, Ts, delay):
        u = u.contiguous()
        Ts = float(Ts)
        d = delay.detach().contiguous()
        out = slayerCuda.getSpikesDelayed(u, refKernel, neuron['theta'], Ts, d)
        ctx.learn_delay = bool(delay.requires_grad)
        ctx.delay_shape = delay.shape
        ctx.save_for_backward(u, d, out if ctx.learn_delay else d)
        ctx.theta = float(neuron['theta'])
        ctx.tau = float(neuron['tauRho'] * neuron['theta'])
        ctx.scale = float(neuron['scaleRho'])
        ctx.Ts = Ts
        return out

    @staticmethod
    def backward(ctx, grad):
        u, d, out = ctx.saved_tensors
        grad = grad.contiguous()
        grad_delay = None
        if ctx.learn_delay:
            grad_delay = slayerCuda.delayGrad(grad, out, ctx.Ts).reshape(ctx.delay_shape)
        grad_u = slayerCuda.spikeGradShift(grad, u, -d, ctx.theta, ctx.tau, ctx.scale, ctx.Ts)
        return grad_u, None, None, None, grad_delay


class _DelayShiftFunction(torch.autograd.Function):
    """Fixed delay without a delay gradient (src/slayer.py:959-979)."""

    @staticmethod
    def forward(ctx, x, delay, Ts=1):
        if torch.is_tensor(delay):
            ctx.delay = delay.detach()
        else:
            ctx.delay = float(delay)
        ctx.Ts = float(Ts)
        return slayerCuda.shift(x.contiguous(), ctx.delay, ctx.Ts)

    @staticmethod
    def backward(ctx, grad):
        return slayerCuda.shift(grad.contiguous(), -ctx.delay, ctx.Ts), None, None


class _LoihiSpikeFunction(torch.autograd.Function):
    """Loihi neuron forward, surrogate gradient x psp-adjoint backward (src/slayerLoihi.py:243-283)."""

    @staticmethod
    def loihi(weightedSpikes, neuron, Ts):
        if weightedSpikes.dtype == torch.int32:
            Ts = 1
        w = weightedSpikes if Ts == 1 and weightedSpikes.dtype == torch.float32 else (weightedSpikes * Ts).float()
        spike, voltage, current = slayerLoihiCuda.getSpikes(
            w.contiguous(), neuron['wgtExp'], neuron['theta'], neuron['iDecay'], neuron['vDecay'],
            neuron['refDelay'])
        if Ts != 1:
            spike = spike / Ts
        return spike, voltage, current

    @staticmethod
    def forward(ctx, weightedSpikes, srmKernel, neuron, Ts):
        spike, voltage, _ = _LoihiSpikeFunction.loihi(weightedSpikes, neuron, Ts)
        ctx.save_for_backward(voltage, srmKernel)
        ctx.theta = float(neuron['theta'])
        ctx.tau = float(neuron['tauRho'] * neuron['theta'])
        ctx.scale = float(neuron['scaleRho'])
        ctx.Ts = float(Ts)
        return spike

    @staticmethod
    def backward(ctx, grad):
        voltage, srmKernel = ctx.saved_tensors
        g = slayerCuda.spikeGrad(grad.contiguous(), voltage, ctx.theta, ctx.tau, ctx.scale)
        return slayerCuda.corr(g, srmKernel, ctx.Ts), None, None, None


class _LoihiSpikeDelayFunction(torch.autograd.Function):
    """Loihi neuron followed by a delay of a whole number of steps, as one autograd node: the
    forward is one launch that writes the spikes already delayed and skips the current
    (``slayerLoihiCuda.getSpikesDelayed``), the backward is the fused shift-back + surrogate
    gradient (``slayerCuda.spikeGradShift``) followed by corr.  Same results as
    ``_LoihiSpikeFunction`` followed by ``_DelayShiftFunction`` (src/slayerLoihi.py:243-283,
    src/slayer.py:959-979)."""

    @staticmethod
    def forward(ctx, weightedSpikes, srmKernel, neuron, Ts, delaySteps):
        if weightedSpikes.dtype == torch.int32:
            Ts = 1
        w = weightedSpikes if Ts == 1 and weightedSpikes.dtype == torch.float32 else (weightedSpikes * Ts).float()
        delayed, voltage = slayerLoihiCuda.getSpikesDelayed(
            w.contiguous(), neuron['wgtExp'], neuron['theta'], neuron['iDecay'], neuron['vDecay'], neuron['refDelay'],
            int(delaySteps))
        if Ts != 1:
            delayed = delayed / Ts
        ctx.save_for_backward(voltage, srmKernel)
        ctx.theta = float(neuron['theta'])
        ctx.tau = float(neuron['tauRho'] * neuron['theta'])
        ctx.scale = float(neuron['scaleRho'])
        ctx.Ts = float(Ts)
        ctx.shift_back = torch.tensor([-float(delaySteps) * float(Ts)], device=voltage.device)
        return delayed

    @staticmethod
    def backward(ctx, grad):
        voltage, srmKernel = ctx.saved_tensors
        g = slayerCuda.spikeGradShift(grad.contiguous(), voltage, ctx.shift_back, ctx.theta, ctx.tau, ctx.scale, ctx.Ts)
        return slayerCuda.corr(g, srmKernel, ctx.Ts), None, None, None, None


# ----------------------------------------------------------------------------- modules
class _DenseLayer(torch.nn.Conv3d):
    """Fully connected layer over NCHWT tensors: a 1x1x1 3-D convolution.  This class restates the
    reference's dense layer (src/slayer.py:393-437) - same argument forms, same branches, same
    exception texts - because it is the interface the reference's networks are written against;
    weighting is not part of the hot path."""

    def __init__(self, inFeatures, outFeatures, weightScale=1):
        if isinstance(inFeatures, int):
            kernel, channels = (1, 1, 1), inFeatures
        elif len(inFeatures) == 2:
            kernel, channels = (inFeatures[1], inFeatures[0], 1), 1
        elif len(inFeatures) == 3:
            kernel, channels = (inFeatures[1], inFeatures[0], 1), inFeatures[2]
        else:
            raise Exception('inFeatures should not be more than 3 dimension. It was: {}'.format(inFeatures))
        if not isinstance(outFeatures, int):
            raise Exception('outFeatures should not be more than 1 dimesnion. It was: {}'.format(outFeatures))
        super().__init__(channels, outFeatures, kernel, bias=False)
        if weightScale != 1:
            self.weight = torch.nn.Parameter(weightScale * self.weight)

    def forward(self, x):
        return F.conv3d(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups)


class _DelayLayer(torch.nn.Module):
    """Learnable axonal delay per neuron or per channel.  Restates the reference's delay layer
    (src/slayer.py:901-928: same argument forms and exception text, delays drawn from U(0, 1),
    per-channel delays repeated over H and W); the arithmetic behind it is _DelayFunction."""

    def __init__(self, inputSize, Ts):
        super().__init__()
        if isinstance(inputSize, int):
            shape = (inputSize, 1, 1)
        elif len(inputSize) == 3:
            shape = tuple(inputSize)
        else:
            raise Exception('inputSize can only be 1 or 2 dimension. It was: {}'.format(inputSize))
        self.delay = torch.nn.Parameter(torch.rand(shape), requires_grad=True)
        self.Ts = Ts

    def forward(self, x):
        N, C, H, W, Ns = x.shape
        if x.numel() != self.delay.numel() * Ns * N:
            return _DelayFunction.apply(x, self.delay.repeat((1, H, W)), self.Ts)
        return _DelayFunction.apply(x, self.delay, self.Ts)


class spikeLayer(torch.nn.Module):
    """SRM spiking layer: response kernels as buffers plus the hot-path methods."""

    def __init__(self, neuronDesc, simulationDesc, fullRefKernel=False):
        super().__init__()
        self.neuron = neuronDesc
        self.simulation = simulationDesc
        self.fullRefKernel = fullRefKernel
        self.register_buffer('srmKernel', self.calculateSrmKernel())
        self.register_buffer('refKernel', self.calculateRefKernel())

    def calculateSrmKernel(self):
        return torch.FloatTensor(alpha_kernel(self.neuron['tauSr'], self.simulation['Ts'],
                                              self.simulation['tSample']))

    def calculateRefKernel(self):
        mult = -self.neuron['scaleRef'] * self.neuron['theta']
        eps = 0.0001 if self.fullRefKernel else 0.01
        return torch.FloatTensor(alpha_kernel(self.neuron['tauRef'], self.simulation['Ts'],
                                              self.simulation['tSample'], mult=mult, epsilon=eps))

    def psp(self, spike):
        if isinstance(spike, PackedSpikes):      # bit-packed spikes (no gradient flows into them)
            return slayerCuda.convPacked(spike.bits, spike.T, self.srmKernel, self.simulation['Ts'], spike.value)
        return _PspFunction.apply(spike, self.srmKernel, self.simulation['Ts'])

    def spikePsp(self, membranePotential):
        """``psp(spike(u))`` as one autograd node with the spikes kept bit-packed in between;
        returns ``(psp output, PackedSpikes)``.  For layers of the form ``spike(W(psp(.)))``, where
        the spikes of one layer are only ever read by the psp filter of the next.  Not part of
        the reference's interface."""
        Ts = self.simulation['Ts']
        out, bits = _SpikePspFunction.apply(membranePotential, self.srmKernel, self.refKernel, self.neuron, Ts)
        return out, PackedSpikes(bits, membranePotential.shape[-1], 1.0 / Ts)

    def spike(self, membranePotential):
        return _SpikeFunction.apply(membranePotential, self.refKernel, self.neuron, self.simulation['Ts'])

    def delayShift(self, input, delay, Ts=1):
        return _DelayShiftFunction.apply(input, delay, Ts)

    def spikeDelayed(self, membranePotential, delay):
        """``spike`` followed by a delay, as one autograd node with a fused backward pass.

        ``delay`` is a delay layer made by ``self.delay(...)`` (learnable: its parameter
        receives the delay gradient), or a tensor with one value per neuron or a single value
        (fixed, like ``delayShift``).  Not part of the reference's interface."""
        if isinstance(delay, _DelayLayer):
            d = delay.delay
            N, C, H, W, Ns = membranePotential.shape
            if membranePotential.numel() != d.numel() * Ns * N:
                d = d.repeat((1, H, W))
        else:
            d = torch.as_tensor(delay, dtype=torch.float32, device=membranePotential.device)
        return _SpikeDelayFunction.apply(membranePotential, self.refKernel, self.neuron, self.simulation['Ts'], d)

    def delay(self, inputSize):
        return _DelayLayer(inputSize, self.simulation['Ts'])

    def dense(self, inFeatures, outFeatures, weightScale=10):
        return _DenseLayer(inFeatures, outFeatures, weightScale)


class loihiLayer(spikeLayer):
    """Loihi CUBA spiking layer (src/slayerLoihi.py:16-122)."""

    def __init__(self, neuronDesc, simulationDesc):
        if neuronDesc['type'] == 'LOIHI':
            neuronDesc['theta'] = neuronDesc['vThMant'] * 2 ** 6
        super().__init__(neuronDesc, simulationDesc)
        self.maxPspKernel = torch.max(self.srmKernel).item()
        # as in the reference, the caller's descriptor is rescaled in place
        neuronDesc['scaleRho'] /= self.maxPspKernel

    def calculateSrmKernel(self):
        return torch.tensor(loihi_psp_kernel(self.neuron))

    def calculateRefKernel(self, SCALE=1000):
        return torch.tensor(loihi_ref_kernel(self.neuron, SCALE))

    def spikeLoihi(self, weightedSpikes):
        return _LoihiSpikeFunction.apply(weightedSpikes, self.srmKernel, self.neuron, self.simulation['Ts'])

    def spikeLoihiDelayed(self, weightedSpikes, delaySteps=1):
        """``delayShift(spikeLoihi(w), delaySteps * Ts, Ts)`` - a Loihi layer and the delay that
        always follows it - as one autograd node with a one-launch forward.  ``delaySteps`` is a
        whole number of time steps.  Not part of the reference's interface."""
        return _LoihiSpikeDelayFunction.apply(weightedSpikes, self.srmKernel, self.neuron, self.simulation['Ts'],
                                              int(delaySteps))

    def spikeLoihiFull(self, weightedSpikes):
        return _LoihiSpikeFunction.loihi(weightedSpikes, self.neuron, self.simulation['Ts'])

    def dense(self, inFeatures, outFeatures, weightScale=100):
        return _DenseLayer(inFeatures, outFeatures, weightScale)
