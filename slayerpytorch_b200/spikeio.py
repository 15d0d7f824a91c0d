"""Address events on the device: the step before the hot path in a training loop.

``event`` mirrors the reference's ``spikeFileIO.event`` (src/spikeFileIO.py:6-144) for what a
training loop does with it - turning a list of (x, y, p, t) events into the spike tensor a
network consumes - but bins on the GPU: the events travel to the device once (20-28 bytes per
event instead of 4 bytes per tensor element) and ``toSpikeTensor`` fills a device tensor in one
kernel.  ``toPackedSpikes`` bins straight into the bit-packed form that ``spikeLayer.psp``
accepts.  File reading, plotting and animation are not part of this module.
"""
import numpy as np
import torch

from . import load_ops
from .layer import PackedSpikes

slayerCuda, _ = load_ops()


class event:
    """``event(xEvent, yEvent, pEvent, tEvent, device='cuda')``: x, y, p integer arrays (y may be
    ``None`` for one spatial dimension), t timestamps in ms.  As in the reference, polarities
    are shifted so that the smallest is 0 (src/spikeFileIO.py:35)."""

    def __init__(self, xEvent, yEvent, pEvent, tEvent, device="cuda"):
        self.dim = 1 if yEvent is None else 2
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("event binning runs on a CUDA device; there is no CPU path")
        as_int = lambda v: torch.as_tensor(np.asarray(v).astype(np.int64), dtype=torch.int32).to(self.device).contiguous()
        self.x = as_int(xEvent)
        self.y = None if yEvent is None else as_int(yEvent)
        p = np.asarray(pEvent).astype(np.int64)
        self.p = as_int(p - (p.min() if p.size else 0))
        self.t = torch.as_tensor(np.asarray(tEvent, dtype=np.float64)).to(self.device).contiguous()

    def _start(self, bins, samplingTime, randomShift):
        if not randomShift or self.t.numel() == 0:
            return 0
        tmin, tmax = float(self.t.min()), float(self.t.max())         # the draw of src/spikeFileIO.py:82-93
        return int(np.random.randint(max(int(tmin / samplingTime), int(tmax / samplingTime) - bins,
                                         bins - int(tmax / samplingTime), 1)))

    def toSpikeTensor(self, emptyTensor, samplingTime=1, randomShift=False, binningMode="OR"):
        """Bins the events into ``emptyTensor`` ([C, H, W, T] float32 on the device) and returns
        it ('OR': filled in place; 'SUM': a new tensor), src/spikeFileIO.py:66-144."""
        mode = {"OR": 0, "SUM": 1}.get(str(binningMode).upper())
        if mode is None:
            raise Exception("Unsupported binningMode. It was {}".format(binningMode))
        if not (torch.is_tensor(emptyTensor) and emptyTensor.is_cuda):
            raise RuntimeError("toSpikeTensor needs a CUDA tensor; there is no CPU path")
        start = self._start(emptyTensor.shape[3], samplingTime, randomShift)
        return slayerCuda.binEvents(emptyTensor, self.x, self.y, self.p, self.t, None, float(samplingTime), start, mode)

    def toPackedSpikes(self, shape, samplingTime=1, randomShift=False):
        """The same binning ('OR') into bit-packed spikes of the given CHWT shape."""
        start = self._start(shape[3], samplingTime, randomShift)
        bits = slayerCuda.binEventsPacked(list(shape), self.x, self.y, self.p, self.t, None, float(samplingTime), start)
        return PackedSpikes(bits, shape[-1], 1.0 / samplingTime)
