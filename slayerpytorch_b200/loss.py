"""Spike losses and the spike-count classifier, resident on the device.

Same names, arguments and results as ``spikeLoss`` (src/spikeLoss.py:7-104) and
``spikeClassifier`` (src/spikeClassifier.py:4-22) of the reference, which the layers of the
hot path feed in every training step.  The reference computes the spike counts, the desired
counts and the target-region mask with NumPy on the host, which costs a device-to-host copy of
the full output spike tensor, a host-to-device copy of two tensors of the same size and two
synchronisations per step (src/spikeLoss.py:91-102).  Here every term is a tensor expression
on the device of ``spikeOut``; nothing is copied and nothing waits.

Arithmetic follows the reference closely enough for identical results: the spike-count error
is formed in float64 (NumPy promotes ``float32 - int64`` to float64 there) and rounded to
float32 once, and the part of the output inside the target region is treated as a constant
in the backward pass, exactly as the reference's ``spikeDesired`` built from ``.data`` is.
"""
import numpy as np
import torch

from .layer import slayerCuda, spikeLayer


class _NumSpikesFunction(torch.autograd.Function):
    """Value and gradient of the spike-count loss from one kernel (``slayerCuda.numSpikesLoss``):
    forward keeps the gradient for a unit upstream gradient, backward scales it."""

    @staticmethod
    def forward(ctx, spikeOut, desiredCount, srmKernel, start, stop, Ts, scale):
        sq, grad = slayerCuda.numSpikesLoss(spikeOut.contiguous(), desiredCount, srmKernel, start, stop, Ts, scale)
        ctx.save_for_backward(grad)
        return (sq * (0.5 * Ts)).float()

    @staticmethod
    def backward(ctx, gradLoss):
        (grad,) = ctx.saved_tensors
        return grad * gradLoss, None, None, None, None, None, None


class spikeLoss(torch.nn.Module):
    """``spikeLoss(networkDescriptor, slayerClass=spikeLayer)`` with ``networkDescriptor`` holding
    ``'neuron'``, ``'simulation'`` and ``'training': {'error': ...}`` (src/spikeLoss.py:30-37)."""

    def __init__(self, networkDescriptor, slayerClass=spikeLayer):
        super().__init__()
        self.neuron = networkDescriptor['neuron']
        self.simulation = networkDescriptor['simulation']
        self.errorDescriptor = networkDescriptor['training']['error']
        self.slayer = slayerClass(self.neuron, self.simulation)
        self.fused = True          # numSpikes: one fused kernel; False = the tensor expressions

    def spikeTime(self, spikeOut, spikeDesired):
        """Van Rossum-like distance between two spike trains (src/spikeLoss.py:39-59)."""
        assert self.errorDescriptor['type'] == 'SpikeTime', "Error type is not SpikeTime"
        error = self.slayer.psp(spikeOut - spikeDesired)
        return 1 / 2 * torch.sum(error ** 2) * self.simulation['Ts']

    def numSpikes(self, spikeOut, desiredClass, numSpikesScale=1):
        """Spike-count loss inside the target region, spike-time loss outside of it
        (src/spikeLoss.py:61-104).  ``desiredClass`` is one-hot with a time dimension of 1."""
        assert self.errorDescriptor['type'] == 'NumSpikes', "Error type is not NumSpikes"
        region = self.errorDescriptor['tgtSpikeRegion']
        count = self.errorDescriptor['tgtSpikeCount']
        Ts = self.simulation['Ts']
        start = int(np.rint(region['start'] / Ts))
        stop = int(np.rint(region['stop'] / Ts))
        T = spikeOut.shape[-1]
        lo, hi = slice(start, stop).indices(T)[:2]        # the slice the reference takes, made explicit

        if spikeOut.is_cuda and spikeOut.dtype == torch.float32 and self.fused and stop != start and T <= 8192:
            # one kernel for the loss and its gradient (same arithmetic as the expressions below)
            onehot = desiredClass.to(spikeOut.device)
            desired = torch.where(onehot == True, float(count[True]), float(count[False]))    # noqa: E712
            desired = desired.to(torch.float32).expand(spikeOut.shape[:-1] + (1,)).reshape(-1).contiguous()
            return _NumSpikesFunction.apply(spikeOut, desired, self.slayer.srmKernel, start, stop, float(Ts),
                                            float(numSpikesScale))

        with torch.no_grad():
            inside = torch.zeros(T, dtype=spikeOut.dtype, device=spikeOut.device)
            inside[lo:hi] = 1
            actual = torch.sum(spikeOut[..., start:stop], 4, keepdim=True) * Ts          # float32, as the reference
            desired = torch.where(desiredClass.to(spikeOut.device) == True,              # noqa: E712 (tensor compare)
                                  torch.tensor(float(count[True]), dtype=torch.float64, device=spikeOut.device),
                                  torch.tensor(float(count[False]), dtype=torch.float64, device=spikeOut.device))
            count_error = (actual.double() - desired) / (stop - start) * numSpikesScale  # float64
            count_term = (count_error * inside.double()).float()                         # rounded once
            spikeDesired = inside * spikeOut                                             # constant in backward

        error = self.slayer.psp(spikeOut - spikeDesired)
        error = error + count_term
        return 1 / 2 * torch.sum(error ** 2) * Ts


class spikeClassifier:
    """Class label = the output neuron with the most spikes (src/spikeClassifier.py:9-20).

    As in the reference the labels come back as a CPU tensor, so that the reference's training
    scripts, which compare them with the CPU labels of a DataLoader
    (``torch.sum(getClass(output) == label)``), run unchanged; the counting itself stays on the
    device and only one index per sample crosses.  ``host=False`` keeps the result on the device
    of ``spike`` (no synchronisation)."""

    @staticmethod
    def getClass(spike, host=True):
        numSpikes = torch.sum(spike, 4, keepdim=True)
        labels = torch.max(numSpikes.reshape((numSpikes.shape[0], -1)), 1)[1]
        return labels.cpu() if host else labels
