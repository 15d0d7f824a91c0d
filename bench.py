#!/usr/bin/env python
"""Benchmark of the SLAYER spiking-neuron hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 1..5] [--impl ours|reference]

A "step" is one forward + backward pass of the hot-path operators of one of five synthetic
workloads (``--config``, default 3) over one batch:

  1  single SRM layer chain, batch 4, 2312 -> 512 neurons, T = 300, fixed delays U(0, 5) ms
  2  SRM MLP 2312-512-10, batch 64, T = 300, learnable delays after the hidden layer
  3  SRM CNN on 34x34x2 frames, batch 128, T = 300, seven spiking layers (2.1 M ... 1.3 k rows)
  4  long-sequence SRM 200-256-200, batch 32, T = 2000, learnable delays U(0, 10) ms after both layers
  5  Loihi CUBA CNN on 32x32x2 frames, batch 64, T = 1450, five spiking layers (1.05 M ... 704 rows)

The weight layers (dense / conv / pool) are PyTorch and run once, during set-up, to produce the
tensors the hot path consumes and the gradients that arrive at it; the timed step is the
operators of this package only: psp (conv), getSpikes, delay shift, their backward (shift back,
surrogate gradient, corr) and, where a delay is learnable, the delay gradient.

Metric: neuron-timesteps per second = (rows of every spiking layer) x T per step / step time,
summed over all GPUs.  With N GPUs the batch is split (``--scaling strong``, the default: the
batch of the configuration is divided over the ranks) or repeated (``--scaling weak``); no
operator communicates, and the step ends with one NCCL all-reduce(SUM) of the parameter
gradients (weight gradients of the rank's shard, computed during set-up, and the delay gradients
the step has just produced).

One JSON line is printed by rank 0.  ``value`` is measured with inputs resident in HBM, L2
flushed between steps, CUDA events around each step, the step's launches replayed from a CUDA
graph; ``e2e`` is the same chain through the package's public layer API with host (pinned)
buffers, copies inside the timed region, streamed in batch chunks by ``HostPipeline``;
``roofline`` describes the kernel with the largest share of the step; ``cpu_baseline`` is the C
oracle on the host cores on a stated batch subsample; ``configs`` holds the resident-input
numbers of all five workloads.  ``--impl reference`` times the explicit time-loop formulation
(the C oracle, all host threads) on a batch subsample of the same workload and, when the
reference's own CUDA operators were built, adds their timing on this GPU as ``reference_cuda``.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np
import torch
import torch.nn.functional as F

METRIC = "neuron-timesteps/s, SRM/Loihi getSpikes+psp+shift forward/backward"
UNIT = "neuron-timesteps/s"
SRM_NEURON = {"type": "SRMALPHA", "theta": 10, "tauSr": 10.0, "tauRef": 1.0, "scaleRef": 2,
              "tauRho": 1, "scaleRho": 1}
LOIHI_NEURON = {"type": "LOIHI", "vThMant": 80, "vDecay": 128, "iDecay": 1024, "refDelay": 1, "wgtExp": 0,
                "tauRho": 1, "scaleRho": 1}
TGT_TRUE, TGT_FALSE = 60, 10
FMA_LANES = 148 * 128 * 2            # fp32 flops per clock of the whole GPU (148 SMs x 128 FMA lanes x 2)

# algorithmic bytes per neuron-timestep of each operator (reads + writes of fp32 tensors)
ALG_BYTES = {"conv": 8, "corr": 8, "getSpikes": 12, "shift": 8, "spikeGrad": 12, "spikeGradShift": 12,
             "getSpikesDelayed": 12, "delayGrad": 8, "loihi": 16, "loihiDelayed": 12,
             "getSpikesPacked": 8.125, "convPacked": 4.125, "corrSpikeGrad": 12}
# DRAM bytes per element measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum of one
# launch over its element count) on launches too large for L2; see the summaries under profiles/.
NCU_TRAFFIC_PER_ELEMENT = {"fir_flow_kernel": 7.36, "fir_flow_kernel<surrogate-gradient epilogue>": 11.6, "srm_get_spikes_tma_kernel": 9.85, "shift_vec4_kernel": 7.4,
                           "spike_grad_shift_rows_kernel": 11.6, "loihi_get_spikes_wide_kernel": 11.9,
                           "delay_grad_kernel": 8.0}


# conv inputs of at least this many samples are probed on the device and go to the event-driven
# kernel when at most SPARSE_DENSITY of the sampled samples are non-zero (csrc/fir.cu, fir_sparse.cuh)
PROBE_MIN_ELEMENTS = 1 << 25
SPARSE_DENSITY = {"conv": 61 / 1024, "convPacked": 92 / 1024}


def conv_is_probed(el, T, taps):
    return el >= PROBE_MIN_ELEMENTS and 64 <= T <= 4096 and 1 <= taps <= 1024


def kernel_of(op, T):
    """Name of the kernel an operator launches for 16-byte aligned fp32 tensors of row length T
    (conv on a mostly-zero input: fir_sparse_kernel instead, see conv_is_probed)."""
    quad = T % 4 == 0
    return {"conv": "fir_flow_kernel", "corr": "fir_flow_kernel", "convPacked": "fir_flow_kernel<packed input>",
            "corrSpikeGrad": "fir_flow_kernel<surrogate-gradient epilogue>",
            "getSpikes": "srm_get_spikes_tma_kernel" if quad else "srm_get_spikes_wide_kernel",
            "getSpikesPacked": "srm_get_spikes_tma_kernel" if quad else "srm_get_spikes_wide_kernel",
            "getSpikesDelayed": "srm_get_spikes_tma_kernel" if quad else "srm_get_spikes_wide_kernel",
            "shift": "shift_vec4_kernel" if quad else "shift_flat4_kernel",
            "spikeGrad": "spike_grad_vec4_kernel", "spikeGradShift": "spike_grad_shift_rows_kernel",
            "delayGrad": "delay_grad_kernel", "loihi": "loihi_get_spikes_wide_kernel",
            "loihiDelayed": "loihi_get_spikes_wide_kernel"}[op]


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ------------------------------------------------------------------------ response kernels
def srm_kernels(T, Ts=1.0, tauSr=None):
    from slayerpytorch_b200.layer import alpha_kernel
    n = SRM_NEURON
    srm = torch.tensor(alpha_kernel(tauSr or n["tauSr"], Ts, T * Ts), dtype=torch.float32)
    ref = torch.tensor(alpha_kernel(n["tauRef"], Ts, T * Ts, mult=-n["scaleRef"] * n["theta"]), dtype=torch.float32)
    return srm, ref


def loihi_kernel():
    from slayerpytorch_b200.layer import loihi_psp_kernel
    return torch.tensor(loihi_psp_kernel(LOIHI_NEURON), dtype=torch.float32)


# ------------------------------------------------------------- operator sets (same names)
class OracleOps:
    """The CPU oracle behind the operator names of slayerCuda / slayerLoihiCuda (torch CPU tensors
    in and out).  Used only by the cpu_baseline leg and the reference arm."""
    fused = False

    def __init__(self, threads=None):
        from oracle import cpu_oracle as co
        self.co = co
        co.set_threads(threads or os.cpu_count() or 1)
        self.threads = co.max_threads()

    def conv(self, x, f, Ts):
        return torch.from_numpy(self.co.conv(x.numpy(), f.numpy(), Ts))

    def corr(self, x, f, Ts):
        return torch.from_numpy(self.co.corr(x.numpy(), f.numpy(), Ts))

    def getSpikes(self, u, nu, theta, Ts):
        s, u_new = self.co.srm_get_spikes(u.numpy(), nu.numpy(), theta, Ts)
        u.copy_(torch.from_numpy(u_new))
        return torch.from_numpy(s)

    def shift(self, x, d, Ts):
        return torch.from_numpy(self.co.shift(x.numpy(), d.numpy() if torch.is_tensor(d) else d, Ts))

    def spikeGrad(self, g, u, theta, tau, scale):
        return torch.from_numpy(self.co.spike_grad(g.numpy(), u.numpy(), theta, tau, scale))

    def delayGrad(self, g, out, Ts):
        return torch.from_numpy(np.asarray(self.co.delay_grad(g.numpy(), out.numpy(), Ts), dtype=np.float32))

    def loihi(self, w, wgtExp, theta, iDecay, vDecay, refDelay):
        return tuple(torch.from_numpy(a) for a in self.co.loihi_get_spikes(w.numpy(), wgtExp, theta, iDecay, vDecay, refDelay))


class OurOps:
    """The operator modules of this package, with the fused operators switched on or off."""

    def __init__(self, fused=True):
        import slayerpytorch_b200
        self.sc, self.lc = slayerpytorch_b200.load_ops()
        self.fused = fused
        for name in ("conv", "corr", "getSpikes", "shift", "spikeGrad", "delayGrad", "getSpikesDelayed", "spikeGradShift"):
            setattr(self, name, getattr(self.sc, name))
        # spikes that only feed the next layer's psp stay bit-packed (spike(W(psp(.))) networks)
        self.packed_spikes = fused
        self.packSpikes, self.getSpikesPacked = self.sc.packSpikes, self.sc.getSpikesPacked
        # ... and the backward of psp(spike(.)) is one launch: corr, then the surrogate gradient
        self.corr_spike_grad = fused
        self.corrSpikeGrad = self.sc.corrSpikeGrad

    def convPacked(self, bits, T, filt, Ts):
        return self.sc.convPacked(bits, T, filt, Ts, 1.0 / Ts)

    def loihi(self, w, wgtExp, theta, iDecay, vDecay, refDelay):
        return tuple(self.lc.getSpikes(w, wgtExp, theta, iDecay, vDecay, refDelay))

    def loihiDelayed(self, w, wgtExp, theta, iDecay, vDecay, refDelay, delay):
        return tuple(self.lc.getSpikesDelayed(w, wgtExp, theta, iDecay, vDecay, refDelay, delay))


class RefCudaOps:
    """The reference's own CUDA operators plus the tensor expressions its Python uses for the
    surrogate gradient (src/slayer.py:862) and the delay gradient (src/slayer.py:950-954)."""
    fused = False

    def __init__(self, mod, loihi_mod):
        self.m, self.lm = mod, loihi_mod
        self.conv, self.corr, self.getSpikes, self.shift = mod.conv, mod.corr, mod.getSpikes, mod.shift

    def spikeGrad(self, g, u, theta, tau, scale):
        th, ta, sc = (torch.tensor(v, device=g.device, dtype=g.dtype) for v in (theta, tau, scale))
        return g * (sc / ta * torch.exp(-torch.abs(u - th) / ta))

    def delayGrad(self, g, out, Ts):
        diff = torch.tensor([-1.0, 1.0], device=g.device) / Ts
        return torch.sum(g * self.m.conv(out, diff, 1), [0, -1], keepdim=True).reshape(out.shape[1:-1]) * Ts

    def loihi(self, w, wgtExp, theta, iDecay, vDecay, refDelay):
        return tuple(self.lm.getSpikes(w, wgtExp, theta, iDecay, vDecay, refDelay))


# ------------------------------------------------------- weight layers (PyTorch, set-up only)
class Weight:
    """A dense / conv / pool layer over NCHWT tensors as the reference builds them: 3-D
    convolutions with a singleton time extent (src/slayer.py:393-585).  Not part of the hot path."""

    def __init__(self, kind, weight=None, padding=0, pool=1, pool_weight=1.0):
        self.kind, self.weight, self.padding, self.pool, self.pool_weight = kind, weight, padding, pool, pool_weight

    def __call__(self, x):
        if self.kind == "pool":
            k = self.pool
            return F.avg_pool3d(x, (k, k, 1)) * (k * k * self.pool_weight)
        if self.kind == "dense":
            n = x.shape[0]
            flat = x.reshape(n, -1, 1, 1, x.shape[-1])
            return F.conv3d(flat, self.weight)
        return F.conv3d(x, self.weight, padding=(self.padding, self.padding, 0))

    def vjp(self, x, g):
        """(gradient w.r.t. x, gradient w.r.t. the weight or None) for an output gradient g."""
        with torch.enable_grad():
            xr = x.detach().requires_grad_(True)
            wr = self.weight.detach().requires_grad_(True) if self.weight is not None else None
            saved, self.weight = self.weight, wr
            try:
                out = self(xr)
            finally:
                self.weight = saved
            wanted = [xr] + ([wr] if wr is not None else [])
            grads = torch.autograd.grad(out, wanted, g)
        return grads[0], (grads[1] if wr is not None else None)


def conv_init(gen, cout, cin, k, std=None, integer=False):
    shape = (cout, cin, k, k, 1)
    if integer:
        return torch.randint(-128, 128, shape, generator=gen).float()
    if std is not None:
        return torch.randn(shape, generator=gen) * std
    bound = 1.0 / (cin * k * k) ** 0.5          # PyTorch Conv3d default init (uniform +-1/sqrt(fan_in))
    return torch.empty(shape).uniform_(-bound, bound, generator=gen)


# -------------------------------------------------------------------------------- workloads
class Workload:
    """Operands of one configuration's hot path on one device, and the step that runs it.

    ``layers`` is a list of dicts, one per spiking layer, with ``kind`` in
      "psp_spike"  u = psp(a); spike(u) [+ delay]               (configs 1, 2, 4)
      "spike_w"    p = psp(s_in); spike(u) with u = W(p) given  (config 3)
      "loihi"      spikeLoihi(w) then delayShift(., 1)           (config 5)
    and the operand tensors of that layer."""

    def __init__(self, cfg, name, T, Ts, layers, kernels, neuron, param_grads, rates, batch):
        self.cfg, self.name, self.T, self.Ts, self.layers = cfg, name, T, Ts, layers
        self.kernels, self.neuron, self.param_grads, self.rates, self.batch = kernels, neuron, param_grads, rates, batch
        self.units = sum(L["rows"] for L in layers) * T
        self.delay_grads = []            # filled by step(): delay gradients produced in this step

    def prep(self):
        """Untimed, between steps: give the in-place operators their original input back."""
        for L in self.layers:
            if L["kind"] == "spike_w":
                L["u"].copy_(L["u0"])

    def step(self, ops, run=None):
        """One forward + backward pass of the hot path; `run(op, layer, rows, fn)` wraps every
        operator call (per-launch timing).  Returns every output so that nothing is freed - and
        no buffer reused - inside the step."""
        run = run or (lambda op, layer, rows, fn: fn())
        Ts, T = self.Ts, self.T
        n = self.neuron
        theta = float(n["theta"])
        tau, scale = float(n["tauRho"] * n["theta"]), float(n["scaleRho"])
        outs, self.delay_grads = [], []
        for i, L in enumerate(self.layers):
            rows = L["rows"]
            if L["kind"] == "psp_spike":
                srm, ref = self.kernels
                u = run("conv", i, rows, lambda: ops.conv(L["a"], srm, Ts))
                delay = L.get("delay")
                if delay is None:
                    s = run("getSpikes", i, rows, lambda: ops.getSpikes(u, ref, theta, Ts))
                    b = run("spikeGrad", i, rows, lambda: ops.spikeGrad(L["g"], u, theta, tau, scale))
                    outs += [s]
                elif ops.fused:
                    d = run("getSpikesDelayed", i, rows, lambda: ops.getSpikesDelayed(u, ref, theta, Ts, delay))
                    if L["learn_delay"]:
                        self.delay_grads.append(run("delayGrad", i, rows, lambda: ops.delayGrad(L["g"], d, Ts)))
                    b = run("spikeGradShift", i, rows,
                            lambda: ops.spikeGradShift(L["g"], u, L["neg_delay"], theta, tau, scale, Ts))
                    outs += [d]
                else:
                    s = run("getSpikes", i, rows, lambda: ops.getSpikes(u, ref, theta, Ts))
                    d = run("shift", i, rows, lambda: ops.shift(s, delay, Ts))
                    if L["learn_delay"]:
                        self.delay_grads.append(run("delayGrad", i, rows, lambda: ops.delayGrad(L["g"], d, Ts)))
                    b0 = run("shift", i, rows, lambda: ops.shift(L["g"], L["neg_delay"], Ts))
                    b = run("spikeGrad", i, rows, lambda: ops.spikeGrad(b0, u, theta, tau, scale))
                    outs += [s, d, b0]
                c = run("corr", i, rows, lambda: ops.corr(b, srm, Ts))
                outs += [u, b, c]
            elif L["kind"] == "spike_w":
                srm, ref = self.kernels
                if getattr(ops, "packed_spikes", False) and "s_bits" in L:
                    # the spikes of a layer are only read by the next layer's psp: they cross as bits
                    p = run("convPacked", i, L["rows_in"], lambda: ops.convPacked(L["s_bits"], T, srm, Ts))
                    if i + 1 < len(self.layers):
                        s = run("getSpikesPacked", i, rows, lambda: ops.getSpikesPacked(L["u"], ref, theta, Ts))
                    else:               # the loss reads the output spikes as fp32
                        s = run("getSpikes", i, rows, lambda: ops.getSpikes(L["u"], ref, theta, Ts))
                else:
                    p = run("conv", i, L["rows_in"], lambda: ops.conv(L["s_in"], srm, Ts))
                    s = run("getSpikes", i, rows, lambda: ops.getSpikes(L["u"], ref, theta, Ts))
                outs += [p, s]
                corr_rho = getattr(ops, "corr_spike_grad", False)
                if not (corr_rho and i + 1 < len(self.layers)):
                    # (fused: the surrogate gradient of this layer rides on the corr of the next one, below)
                    outs.append(run("spikeGrad", i, rows, lambda: ops.spikeGrad(L["g_s"], L["u"], theta, tau, scale)))
                if L["g_p"] is not None:         # the network input needs no gradient
                    if corr_rho:
                        # psp backward of this layer, then spike backward of the layer that produced
                        # its input spikes: one launch
                        below = self.layers[i - 1]
                        outs.append(run("corrSpikeGrad", i, L["rows_in"],
                                        lambda: ops.corrSpikeGrad(L["g_p"], srm, below["u"], theta, tau, scale, Ts)))
                    else:
                        outs.append(run("corr", i, L["rows_in"], lambda: ops.corr(L["g_p"], srm, Ts)))
            else:
                k = self.kernels[0]
                if ops.fused:
                    # the spikes are written once, already delayed by one step, and the current (which
                    # the layer does not keep) is not written; shift back + surrogate gradient in one pass
                    d, v = run("loihiDelayed", i, rows, lambda: ops.loihiDelayed(L["w"], n["wgtExp"], n["theta"], n["iDecay"],
                                                                                 n["vDecay"], n["refDelay"], 1))
                    gu = run("spikeGradShift", i, rows,
                             lambda: ops.spikeGradShift(L["g"], v, L["minus_one"], theta, tau, scale, Ts))
                    outs += [v, d, gu]
                else:
                    s, v, u = run("loihi", i, rows, lambda: ops.loihi(L["w"], n["wgtExp"], n["theta"], n["iDecay"],
                                                                      n["vDecay"], n["refDelay"]))
                    d = run("shift", i, rows, lambda: ops.shift(s, 1.0, Ts))
                    b0 = run("shift", i, rows, lambda: ops.shift(L["g"], -1.0, Ts))
                    gu = run("spikeGrad", i, rows, lambda: ops.spikeGrad(b0, v, theta, tau, scale))
                    outs += [s, v, u, d, b0, gu]
                outs.append(run("corr", i, rows, lambda: ops.corr(gu, k, Ts)))
        return outs

    def op_list(self, fused):
        """(op, layer, elements, taps) of every launch of a step, without running anything."""
        class Dry:
            pass
        calls = []
        dry = Dry()
        dry.fused = fused
        dry.packed_spikes = fused
        dry.corr_spike_grad = fused
        for name in ("conv", "corr", "getSpikes", "shift", "spikeGrad", "delayGrad", "getSpikesDelayed",
                     "spikeGradShift", "loihi", "loihiDelayed", "convPacked", "getSpikesPacked", "corrSpikeGrad"):
            setattr(dry, name, (lambda *a, **k: (None, None, None)) if name == "loihi" else
                    ((lambda *a, **k: (None, None)) if name == "loihiDelayed" else (lambda *a, **k: None)))

        def run(op, layer, rows, fn):
            taps = 0
            if op in ("conv", "corr", "convPacked", "corrSpikeGrad"):
                taps = int(self.kernels[0].numel())
            calls.append((op, layer, rows * self.T, taps))
            return fn()
        if not hasattr(self, "conv_density"):
            # fraction of non-zero samples of every conv input (what the probe kernel estimates)
            self.conv_density = {}
            for i, L in enumerate(self.layers):
                a = L.get("a") if L["kind"] == "psp_spike" else L.get("s_in")
                if a is not None:
                    self.conv_density[i] = float((a != 0).float().mean())
        self.step(dry, run)
        self.delay_grads = []
        return calls

    def launches_per_step(self, fused):
        """Kernels launched per step: one per operator call, three for a conv that is probed (the
        probe, the event-driven kernel and the dense kernel, one of the two returning at once)."""
        return sum(3 if (op in SPARSE_DENSITY and conv_is_probed(el, self.T, taps)) else 1
                   for op, _, el, taps in self.op_list(fused))

    def sparse_convs(self, fused):
        """Layers whose conv goes to the event-driven kernel, with the density of its input."""
        return {layer: self.conv_density[layer] for op, layer, el, taps in self.op_list(fused)
                if op in SPARSE_DENSITY and conv_is_probed(el, self.T, taps)
                and self.conv_density.get(layer, 1.0) <= SPARSE_DENSITY[op]}

    def chain_bound_ms(self, fused, peak_gbs, sm_mhz):
        """Sum over the step's launches of max(algorithmic bytes / HBM peak, flops / fp32 FMA peak);
        a conv on a mostly-zero input that the event-driven kernel takes only owes the products
        with non-zero samples (2 K flop x density per element)."""
        fma = FMA_LANES * sm_mhz * 1e6
        sparse = self.sparse_convs(fused)
        total = 0.0
        for op, layer, el, taps in self.op_list(fused):
            flops = 2.0 * taps * el * (sparse[layer] if (op in SPARSE_DENSITY and layer in sparse) else 1.0)
            total += max(ALG_BYTES[op] * el / (peak_gbs * 1e9), flops / fma)
        return total * 1e3


def bernoulli(gen, shape, p):
    return (torch.rand(shape, generator=gen) < p).float()


def count_loss_grad(ops, s_out, label, srm, Ts, T):
    """Gradient of a spike-count loss (src/spikeLoss.py:60-104, target region = whole sample)
    at the output spikes: the per-step error (count - target) / T sent back through psp."""
    batch, n_out = s_out.shape[0], s_out.shape[1]
    count = s_out.sum(-1, keepdim=True) * Ts
    target = torch.full((batch, n_out, 1, 1, 1), float(TGT_FALSE), device=count.device)
    target[torch.arange(batch), label.to(count.device)] = float(TGT_TRUE)
    err = ((count - target) / T).expand(-1, -1, -1, -1, T).contiguous()
    return ops.corr(err * Ts, srm, Ts)


def shard(t, rank, world, scaling):
    if world == 1 or scaling == "weak":
        return t
    from slayerpytorch_b200.sharding import shard_batch
    return shard_batch(t, rank, world)


def build_mlp(cfg, ops, device, rank, world, scaling, batch_override=None):
    """Configs 1, 2 and 4: layers of the form spike(psp(fc(x))) with an optional delay."""
    spec = {1: dict(batch=4, sizes=[2312, 512], T=300, delay_after=[0], delay_max=5.0, learn=False, tauSr=10.0,
                    inp="bernoulli", w="normal"),
            2: dict(batch=64, sizes=[2312, 512, 10], T=300, delay_after=[0], delay_max=5.0, learn=True, tauSr=10.0,
                    inp="bernoulli", w="default"),
            4: dict(batch=32, sizes=[200, 256, 200], T=2000, delay_after=[0, 1], delay_max=10.0, learn=True, tauSr=10.0,
                    inp="one_spike", w="default", wscale=[100.0, 30.0])}[cfg]
    T, Ts, sizes = spec["T"], 1.0, spec["sizes"]
    batch = batch_override or spec["batch"]
    seed = 1000 + cfg + (97 * rank if scaling == "weak" else 0)
    gen = torch.Generator().manual_seed(seed)
    srm, ref = srm_kernels(T, Ts, spec["tauSr"])
    if spec["inp"] == "bernoulli":
        x = bernoulli(gen, (batch, sizes[0], 1, 1, T), 0.05)
    else:                                 # one spike per input neuron at floor(U(0, 1000)) ms
        x = torch.zeros(batch, sizes[0], 1, 1, T)
        when = torch.randint(0, 1000, (batch, sizes[0]), generator=gen)
        x.view(batch, sizes[0], T).scatter_(2, when.unsqueeze(-1), 1.0 / Ts)
    weights = []
    for i, (cin, cout) in enumerate(zip(sizes[:-1], sizes[1:])):
        if spec["w"] == "normal":
            weights.append(torch.randn(cout, cin, 1, 1, 1, generator=gen))
        else:
            # Conv3d default init times weightScale (10 by default, src/slayer.py:187, :420).  With one
            # input spike per neuron the default scale leaves config 4 silent, so its layers use 100
            # and 30, which gives spike rates of about 1 % and 3 %.
            wscale = spec.get("wscale", [10.0] * len(sizes))[i]
            weights.append(torch.empty(cout, cin, 1, 1, 1).uniform_(-1, 1, generator=gen) * (wscale / cin ** 0.5))
    delays = [torch.rand(n, generator=gen) * spec["delay_max"] for n in sizes[1:]]
    label = torch.randint(0, sizes[-1], (batch,), generator=gen)
    target = bernoulli(gen, (batch, sizes[-1], 1, 1, T), 0.02)

    x, label, target = (shard(t, rank, world, scaling) for t in (x, label, target))
    x, target, srm, ref = (t.to(device) for t in (x, target, srm, ref))
    weights = [Weight("dense", w.to(device)) for w in weights]
    delays = [d.to(device) for d in delays]
    theta = float(SRM_NEURON["theta"])
    tau, scale = float(SRM_NEURON["tauRho"] * theta), float(SRM_NEURON["scaleRho"])

    # forward, keeping what the hot path consumes
    layers, s, rates = [], x, []
    for i, W in enumerate(weights):
        a = W(s).contiguous()
        u = ops.conv(a, srm, Ts)
        sp = ops.getSpikes(u, ref, theta, Ts)
        L = dict(kind="psp_spike", a=a, rows=a.numel() // T, s_in=s, u=u, W=W)
        rates.append(float(sp.mean()))
        if i in spec["delay_after"]:
            L.update(delay=delays[i], neg_delay=-delays[i], learn_delay=spec["learn"])
            s = ops.shift(sp, delays[i], Ts)
        else:
            s = sp
        L["out"] = s
        layers.append(L)
    # gradient arriving at the last layer's output
    if cfg == 4:                          # spikeTime loss: error = psp(out - target), sent back through psp
        g = ops.corr(ops.conv(s - target, srm, Ts), srm, Ts)
    else:
        g = count_loss_grad(ops, s, label, srm, Ts, T)
    param_grads = []
    for L in reversed(layers):
        L["g"] = g.contiguous()
        b = ops.shift(L["g"], L["neg_delay"], Ts) if "delay" in L else L["g"]
        ga = ops.corr(ops.spikeGrad(b, L["u"], theta, tau, scale), srm, Ts)
        g, gw = L["W"].vjp(L["s_in"], ga)
        param_grads.append(gw)
    for L in layers:                      # only the operands stay resident
        for k in ("u", "s_in", "out", "W"):
            L.pop(k, None)
    name = {1: "config 1: single SRM layer chain 2312->512, batch %d, T=300, fixed delays U(0,5), N(0,1) weights",
            2: "config 2: SRM MLP 2312-512-10 hot path, batch %d, T=300, Ts=1, input rate 5%%, learnable delays U(0,5) after the hidden layer",
            4: "config 4: long-sequence SRM 200-256-200, batch %d, T=2000, one input spike per neuron at U(0,1000) ms, "
               "learnable delays U(0,10) after both layers, weight scales 100 and 30"}[cfg] % batch
    name += ", psp K=%d, refractory %d taps" % (srm.numel(), ref.numel())
    return Workload(cfg, name, T, Ts, layers, (srm, ref), SRM_NEURON, param_grads, rates, x.shape[0])


def build_cnn(ops, device, rank, world, scaling, batch_override=None):
    """Config 3: every layer is spike(W(psp(s))); psp therefore runs on spike tensors."""
    T, Ts = 300, 1.0
    batch = batch_override or 128
    gen = torch.Generator().manual_seed(1003 + (97 * rank if scaling == "weak" else 0))
    srm, ref = srm_kernels(T, Ts)
    theta = float(SRM_NEURON["theta"])
    tau, scale = float(SRM_NEURON["tauRho"] * theta), float(SRM_NEURON["scaleRho"])
    x = bernoulli(gen, (batch, 2, 34, 34, T), 0.05)
    std = 0.5
    weights = [Weight("conv", conv_init(gen, 16, 2, 5, std), padding=1), Weight("pool", pool=2, pool_weight=1.1 * theta),
               Weight("conv", conv_init(gen, 32, 16, 3, std), padding=1), Weight("pool", pool=2, pool_weight=1.1 * theta),
               Weight("conv", conv_init(gen, 64, 32, 3, std), padding=1),
               Weight("dense", torch.randn(512, 8 * 8 * 64, 1, 1, 1, generator=gen) * std),
               Weight("dense", torch.randn(10, 512, 1, 1, 1, generator=gen) * std)]
    label = torch.randint(0, 10, (batch,), generator=gen)
    x, label = shard(x, rank, world, scaling), shard(label, rank, world, scaling)
    x, srm, ref = x.to(device), srm.to(device), ref.to(device)
    for W in weights:
        if W.weight is not None:
            W.weight = W.weight.to(device)
    layers, s, rates = [], x, []
    for W in weights:
        p = ops.conv(s, srm, Ts)
        u0 = W(p).contiguous()
        u = u0.clone()
        sp = ops.getSpikes(u, ref, theta, Ts)
        layers.append(dict(kind="spike_w", s_in=s, rows_in=s.numel() // T, u0=u0, u=u, rows=u.numel() // T, W=W, p=p))
        if getattr(ops, "packed_spikes", False):
            layers[-1]["s_bits"] = ops.packSpikes(s)
        rates.append(float(sp.mean()))
        s = sp
    g = count_loss_grad(ops, s, label, srm, Ts, T)
    param_grads = []
    for i in reversed(range(len(layers))):
        L = layers[i]
        L["g_s"] = g.contiguous()
        gu = ops.spikeGrad(L["g_s"], L["u"], theta, tau, scale)
        g_p, gw = L["W"].vjp(L["p"], gu)
        if gw is not None:
            param_grads.append(gw)
        L["g_p"] = g_p.contiguous() if i > 0 else None
        g = ops.corr(g_p.contiguous(), srm, Ts) if i > 0 else None
        del L["p"], L["W"]
    name = ("config 3: SRM CNN 34x34x2 -> 16c5 -> pool2 -> 32c3 -> pool2 -> 64c3 -> 512 -> 10, every layer spike(W(psp(.))), "
            "batch %d, T=300, N(0,0.5) weights, input rate 5%%, psp K=%d, refractory %d taps" % (x.shape[0], srm.numel(), ref.numel()))
    return Workload(3, name, T, Ts, layers, (srm, ref), SRM_NEURON, param_grads, rates, x.shape[0])


def build_loihi(ops, device, rank, world, scaling, batch_override=None):
    """Config 5: every layer is delayShift(spikeLoihi(W(x)), 1) with integer weights."""
    T, Ts = 1450, 1.0
    batch = batch_override or 64
    gen = torch.Generator().manual_seed(1005 + (97 * rank if scaling == "weak" else 0))
    neuron = dict(LOIHI_NEURON)
    neuron["theta"] = neuron["vThMant"] * 64
    k = loihi_kernel()
    neuron["scaleRho"] = 1.0 / float(k.max())            # as the layer constructor rescales it (src/slayerLoihi.py:53-56)
    theta = float(neuron["theta"])
    tau, scale = float(neuron["tauRho"] * theta), float(neuron["scaleRho"])
    x = bernoulli(gen, (batch, 2, 32, 32, T), 0.02)
    pool_w = float(2 * round(1.1 * theta / float(k.max()) / 2))      # quantised in steps of 2 (src/slayerLoihi.py:170)
    weights = [Weight("conv", conv_init(gen, 16, 2, 5, integer=True), padding=2), Weight("pool", pool=4, pool_weight=pool_w),
               Weight("conv", conv_init(gen, 32, 16, 3, integer=True), padding=1),
               Weight("dense", torch.randint(-128, 128, (512, 8 * 8 * 32, 1, 1, 1), generator=gen).float()),
               Weight("dense", torch.randint(-128, 128, (11, 512, 1, 1, 1), generator=gen).float())]
    label = torch.randint(0, 11, (batch,), generator=gen)
    x, label = shard(x, rank, world, scaling), shard(label, rank, world, scaling)
    x, k = x.to(device), k.to(device)
    for W in weights:
        if W.weight is not None:
            W.weight = W.weight.to(device)
    minus_one = torch.tensor([-1.0], device=device)
    layers, s, rates = [], x, []
    for W in weights:
        w = W(s).contiguous()
        sp, v, _ = ops.loihi(w, neuron["wgtExp"], neuron["theta"], neuron["iDecay"], neuron["vDecay"], neuron["refDelay"])
        layers.append(dict(kind="loihi", w=w, rows=w.numel() // T, s_in=s, v=v, W=W, minus_one=minus_one))
        rates.append(float(sp.mean()))
        s = ops.shift(sp, 1.0, Ts)
    g = count_loss_grad(ops, s, label, k, Ts, T)
    param_grads = []
    for L in reversed(layers):
        L["g"] = g.contiguous()
        gu = ops.spikeGrad(ops.shift(L["g"], -1.0, Ts), L["v"], theta, tau, scale)
        gw_in = ops.corr(gu, k, Ts)
        g, gw = L["W"].vjp(L["s_in"], gw_in)
        if gw is not None:
            param_grads.append(gw)
        del L["s_in"], L["v"], L["W"]
    name = ("config 5: Loihi CUBA CNN 32x32x2 -> 16c5 -> pool4 -> 32c3 -> 512 -> 11, every layer delayShift(spikeLoihi(W(x)), 1), "
            "batch %d, T=1450, integer weights U{-128..127}, vThMant=80, iDecay=1024, vDecay=128, input rate 2%%, "
            "backward corr K=%d" % (x.shape[0], k.numel()))
    return Workload(5, name, T, Ts, layers, (k,), neuron, param_grads, rates, x.shape[0])


def build_workload(cfg, ops, device, rank=0, world=1, scaling="strong", batch_override=None):
    with torch.no_grad():
        if cfg == 3:
            return build_cnn(ops, device, rank, world, scaling, batch_override)
        if cfg == 5:
            return build_loihi(ops, device, rank, world, scaling, batch_override)
        return build_mlp(cfg, ops, device, rank, world, scaling, batch_override)


FULL_BATCH = {1: 4, 2: 64, 3: 128, 4: 32, 5: 64}
CPU_SAMPLE_BATCH = {1: 4, 2: 64, 3: 4, 4: 32, 5: 2}        # batch subsample timed on the host cores


# ------------------------------------------------------------------------------ GPU clocks
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, device_index, period=0.002):
        super().__init__(daemon=True)
        self.period = period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.nv, self.h = pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception as e:          # clocks are reported as unavailable, never guessed
            self.err = repr(e)

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "sw_power_cap": 0x4, "hw_power_brake_slowdown": 0x80}
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                    nv.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = get(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        top = sorted(self.samples)[len(self.samples) // 2:]       # upper half = under load
        return {"sm_mhz": statistics.median(top), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def bind_near_gpu(device_index):
    """Run this process, and allocate its pinned buffers, on the CPUs next to its GPU (the
    affinity NVML reports), within the CPUs the process is allowed to use."""
    try:
        import pynvml
        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(device_index).uuid)
        if not uuid.startswith("GPU-"):
            uuid = "GPU-" + uuid
        h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        near = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        use = near & allowed
        if use and use != allowed:
            os.sched_setaffinity(0, use)
        return {"gpu_cpus": len(near), "allowed_cpus": len(allowed), "bound_to": len(use) if use else len(allowed)}
    except Exception as e:
        return {"error": repr(e)[:120]}


# --------------------------------------------------------------------------------- our arm
def flush_l2(buf):
    buf.zero_()


def time_resident(wl, ops, steps, warmup, device, world, flush, use_graph, allreduce):
    """Resident-input timing of one workload: (graph or eager total ms, eager total ms, per-op events,
    all-reduce ms per step, note)."""
    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def full_step():
        outs = wl.step(ops)
        if allreduce:
            from slayerpytorch_b200.sharding import allreduce_sum_
            allreduce_sum_(wl.param_grads + wl.delay_grads)
        return outs

    for _ in range(max(warmup, 3)):
        wl.prep()
        flush_l2(flush)
        full_step()
    barrier()

    graph, note = None, None
    if use_graph:
        try:
            wl.prep()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                keep = wl.step(ops)            # the collective stays outside the graph
            graph_keep = keep
            for _ in range(3):
                wl.prep()
                flush_l2(flush)
                graph.replay()
        except Exception as e:                 # reported, and the eager loop is timed instead
            graph, note = None, "capture failed: %r" % (e,)
        barrier()

    def graph_step():
        graph.replay()
        if allreduce:
            from slayerpytorch_b200.sharding import allreduce_sum_
            allreduce_sum_(wl.param_grads + graph_delay_grads)

    graph_delay_grads = list(wl.delay_grads)

    def timed(step):
        events = []
        for _ in range(steps):
            wl.prep()
            flush_l2(flush)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            events.append((e0, e1))
        barrier()
        return sum(a.elapsed_time(b) for a, b in events)

    eager_ms = timed(full_step)
    total_ms = timed(graph_step) if graph is not None else eager_ms

    # the collective alone (N > 1): same buffers, same size
    ar_ms = None
    if allreduce:
        from slayerpytorch_b200.sharding import allreduce_sum_
        bufs = wl.param_grads + (graph_delay_grads if graph is not None else wl.delay_grads)
        ev = []
        for _ in range(max(5, min(steps, 20))):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            allreduce_sum_(bufs)
            e1.record()
            ev.append((e0, e1))
        barrier()
        ar_ms = sum(a.elapsed_time(b) for a, b in ev) / len(ev)

    # per-operator breakdown: a separate eager pass with an event pair around every launch
    op_events = []

    def rec(op, layer, rows, fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        op_events.append((op, layer, rows, e0, e1))
        return out

    for _ in range(max(3, min(steps, 20))):
        wl.prep()
        flush_l2(flush)
        wl.step(ops, rec)
    barrier()
    per_op = {}
    for op, layer, rows, a, b in op_events:
        per_op.setdefault((op, layer, rows), []).append(a.elapsed_time(b))
    del graph
    return total_ms, eager_ms, per_op, ar_ms, note


def op_table_of(wl, per_op):
    total = sum(sum(v) for v in per_op.values())
    table = {}
    for (op, layer, rows), v in sorted(per_op.items(), key=lambda kv: (kv[0][1], kv[0][0])):
        us = 1e3 * sum(v) / len(v)
        el = rows * wl.T
        table["L%d/%s" % (layer, op)] = {"rows": rows, "us": round(us, 2),
                                         "GB/s": round(ALG_BYTES[op] * el / (us * 1e-6) / 1e9, 1),
                                         "share": round(sum(v) / total, 4)}
    return table


def time_plain_corr(wl, ops, layer, flush):
    """The corr launch that a corrSpikeGrad launch contains, on the same operand (average ms)."""
    L = wl.layers[layer]
    srm = wl.kernels[0]
    ev = []
    for _ in range(5):
        flush_l2(flush)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = ops.corr(L["g_p"], srm, wl.Ts)
        e1.record()
        ev.append((e0, e1))
        del out
    torch.cuda.synchronize()
    t = sorted(a.elapsed_time(b) for a, b in ev)[1:]          # the first call may set the kernel up
    return sum(t) / len(t)


def roofline_of(wl, per_op, peak, peak_kind, sm_mhz, ops=None, flush=None):
    """The kernel with the largest share of the step, described on its largest launch."""
    sparse = wl.sparse_convs(True)

    def k_of(op, layer):
        return "fir_sparse_kernel" if (op in SPARSE_DENSITY and layer in sparse) else kernel_of(op, wl.T)
    share = {}
    for (op, layer, rows), v in per_op.items():
        k = k_of(op, layer)
        share[k] = share.get(k, 0.0) + sum(v)
    total = sum(share.values())
    dominant = max(share, key=share.get)
    cands = [(rows, op, layer) for (op, layer, rows) in per_op if k_of(op, layer) == dominant]
    rows, op, layer = max(cands)
    times = per_op[(op, layer, rows)]
    avg_ms = sum(times) / len(times)
    el = rows * wl.T
    alg = ALG_BYTES[op] * el
    gbs = alg / (avg_ms * 1e-3) / 1e9
    tpe = NCU_TRAFFIC_PER_ELEMENT.get(dominant)
    taps = int(wl.kernels[0].numel()) if op in ("conv", "corr", "convPacked", "corrSpikeGrad") else 0
    fma_peak = FMA_LANES * (sm_mhz or 1965.0) * 1e6 / 1e12
    hbm = {"achieved": round(gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / peak, 4)}
    out = {"kernel": dominant, "kernel_share_of_step": round(share[dominant] / total, 4),
           "launch": "L%d/%s, %d x %d fp32" % (layer, op, rows, wl.T), "peak_kind": peak_kind,
           "traffic": (tpe * el if tpe else None), "algorithmic_bytes": alg, "avg_launch_us": round(avg_ms * 1e3, 2),
           "hbm": hbm}
    if dominant == "fir_sparse_kernel":
        taps = 0                         # the products with zeros are not owed: HBM bounds it
    fma_bound = taps and (2.0 * taps / (fma_peak * 1e12)) > (ALG_BYTES[op] / (peak * 1e9))
    if fma_bound:
        tfl = 2.0 * taps * el / (avg_ms * 1e-3) / 1e12
        out.update({"bound": "fp32_fma", "achieved": round(tfl, 2), "peak": round(fma_peak, 1), "unit": "TFLOP/s",
                    "frac": round(tfl / fma_peak, 4), "taps": taps,
                    "peak_how": "148 SMs x 128 fp32 lanes x 2 flop x the SM clock sampled during the run"})
    else:
        out.update({"bound": "hbm", **hbm})
    if op == "corrSpikeGrad":
        out["note"] = ("the launch also evaluates the surrogate gradient of its 16 outputs per thread (one exp, one division by "
                       "reciprocal + 4 FMAs each) and reads the potential; the 2K flop per element counted here leave that out")
        if ops is not None and flush is not None:
            ms = time_plain_corr(wl, ops, layer, flush)
            tfl = 2.0 * taps * el / (ms * 1e-3) / 1e12
            out["same_launch_without_epilogue"] = {"op": "corr", "avg_launch_us": round(ms * 1e3, 2), "achieved": round(tfl, 2),
                                                   "frac": round(tfl / fma_peak, 4)}
    return out


def time_ours(args, rank, world, device):
    from slayerpytorch_b200 import layer as L
    from slayerpytorch_b200.hoststream import HostPipeline, chunk_bounds
    ops = OurOps(fused=not args.unfused)
    peak, peak_kind = measured_peak_gbs()
    binding = bind_near_gpu(device.index)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    scaling = args.scaling if world > 1 else "weak"
    if args.config == 1 and world > 4 and scaling == "strong":
        scaling = "weak"                 # a batch of 4 does not split eight ways
    allreduce = world > 1 and args.config != 1

    wl = build_workload(args.config, ops, device, rank, world, scaling)
    sampler = ClockSampler(device.index)
    sampler.start()
    total_ms, eager_ms, per_op, ar_ms, graph_note = time_resident(
        wl, ops, args.steps, args.warmup, device, world, flush, not args.no_graph, allreduce)
    clocks = sampler.stop()

    # ---- end to end through the public layer API with host buffers
    if args.no_e2e:
        e2e = {"ms_total": float("nan"), "serial_ms_total": 0.0, "steps": 1, "h2d": 0, "d2h": 0, "how": "skipped (--no-e2e)"}
    else:
        e2e = time_e2e(args, wl, ops, device, world, flush, L, HostPipeline, chunk_bounds)

    units_all = torch.tensor([float(wl.units)], dtype=torch.float64, device=device)
    t = torch.tensor([total_ms, eager_ms, e2e["ms_total"], e2e["serial_ms_total"], ar_ms or 0.0], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        torch.distributed.all_reduce(units_all, op=torch.distributed.ReduceOp.SUM)
    total_ms, eager_ms, e2e_ms, e2e_serial_ms, ar_ms = (float(x) for x in t)
    units_all = float(units_all)
    if rank != 0:
        return None

    fused = not args.unfused
    sm_mhz = clocks["sm_mhz"] or 1965.0
    bound_ms = wl.chain_bound_ms(fused, peak, sm_mhz)
    nar = sum(g.numel() for g in wl.param_grads + wl.delay_grads)
    out = {
        "metric": METRIC, "value": units_all * args.steps / (total_ms * 1e-3), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl.name,
                   "fusion": ("none: the reference's sequence of launches" if args.unfused else
                              "getSpikes+delay as one launch (SRM: getSpikesDelayed; Loihi: getSpikesDelayed without the "
                              "current) and shift back + surrogate gradient as one launch (spikeGradShift) wherever a delay "
                              "follows the spikes; in spike(W(psp(.))) networks (config 3) the spikes of a layer cross to the "
                              "next layer's psp bit-packed (getSpikesPacked, convPacked), the output layer's as fp32, and the backward of "
                              "psp(spike(.)) - corr, then the surrogate gradient of the layer below - is one launch (corrSpikeGrad); same results"),
                   "neuron_timesteps_per_step_per_gpu": wl.units, "batch_per_gpu": wl.batch,
                   "l2": "flushed between steps (256 MiB write); in-place potentials restored between steps, untimed",
                   "spike_rates": [round(r, 4) for r in wl.rates],
                   "parallelism": "batch sharded over %d GPU(s), no collective between operators%s"
                                  % (world, "; one NCCL all-reduce(SUM) of parameter gradients per step" if allreduce else "")},
        "clocks": clocks,
        "e2e": {"value": units_all * e2e["steps"] / (e2e_ms * 1e-3), "unit": UNIT,
                "ms_per_step": e2e_ms / e2e["steps"], "steps": e2e["steps"],
                "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"], "how": e2e["how"],
                "single_call_ms_per_step": (e2e_serial_ms / e2e["steps"]) if e2e_serial_ms else None,
                "pcie_GB/s_per_direction": round(max(e2e["h2d"], e2e["d2h"]) / (e2e_ms / e2e["steps"] * 1e-3) / 1e9, 1),
                "host_binding": binding},
        "launch_mode": ("cuda graph replay of the step's %d launches" % wl.launches_per_step(fused))
                       if (not args.no_graph and graph_note is None) else ("eager" + (" (%s)" % graph_note if graph_note else "")),
        "eager_ms_per_step": eager_ms / args.steps,
        "gpu_launches": wl.launches_per_step(fused) * args.steps,
        "chain": {"bound_ms": round(bound_ms, 4), "frac_of_bound": round(bound_ms / (total_ms / args.steps), 4),
                  "how": "sum over the step's launches of max(algorithmic bytes / measured HBM peak, 2K flop / fp32 FMA peak at the "
                         "sampled clock); a conv that the event-driven kernel takes owes 2K flop x input density",
                  "event_driven_conv_layers": {("L%d" % k): round(v, 4) for k, v in wl.sparse_convs(fused).items()}},
        "roofline": roofline_of(wl, per_op, peak, peak_kind, sm_mhz, ops, flush),
        "per_op": op_table_of(wl, per_op),
    }
    if allreduce:
        out["allreduce"] = {"op": "SUM", "elements": nar, "bytes": 4 * nar, "ms": round(ar_ms, 4),
                            "share_of_step": round(ar_ms / (total_ms / args.steps), 4),
                            "what": "weight gradients of the rank's shard (computed in set-up by PyTorch) and the delay gradients of this step"}
    del wl
    torch.cuda.empty_cache()
    if world == 1:
        out["cpu_baseline"] = cpu_baseline_value(args.config, reps=3) if not args.no_e2e else None
        if not args.no_all_configs:
            out["configs"] = all_configs(args, ops, device, flush, peak, peak_kind, out)
        out["loss"] = loss_leg(ops, device)
    return out


def time_e2e(args, wl, ops, device, world, flush, L, HostPipeline, chunk_bounds):
    """The same step through slayerpytorch_b200.layer with autograd, operands in pinned host
    memory and every result copied back inside the timed region."""
    steps = min(args.steps, args.e2e_steps)
    n = wl.neuron
    if wl.cfg == 5:
        net = L.loihiLayer(dict(LOIHI_NEURON), {"Ts": wl.Ts, "tSample": wl.T}).to(device)
    else:
        net = L.spikeLayer(dict(n), {"Ts": wl.Ts, "tSample": wl.T}).to(device)
    in_keys = {"psp_spike": ("a", "g"), "spike_w": ("s_in", "u0", "g_s", "g_p"), "loihi": ("w", "g")}
    # Layers of the form spike(W(psp(.))) through the fused node spikePsp = psp of the next layer
    # applied to the spikes of this one: the spikes stay on the device as bits, and neither they
    # nor the gradient that reaches them cross PCIe; what crosses per layer is its potential, the
    # next layer's psp output and that output's gradient.
    chained = wl.layers[0]["kind"] == "spike_w" and not args.unfused
    last = len(wl.layers) - 1
    names = []
    for i, Lr in enumerate(wl.layers):
        for k in in_keys[Lr["kind"]]:
            if Lr.get(k) is None:
                continue
            if chained and ((k == "s_in" and i > 0) or (k == "g_s" and i < last)):
                continue
            names.append((i, k))
    dev_in = [wl.layers[i][k] for i, k in names]
    delays = {}
    for i, Lr in enumerate(wl.layers):
        if Lr.get("delay") is not None:
            if Lr["learn_delay"]:
                dl = net.delay(Lr["delay"].numel()).to(device)
                with torch.no_grad():
                    dl.delay.copy_(Lr["delay"].view(-1, 1, 1))
                delays[i] = dl
            else:
                delays[i] = Lr["delay"]

    def device_step(*tensors):
        by = {nk: t for nk, t in zip(names, tensors)}
        heads, grads, results = [], [], []          # results: callables evaluated after backward
        for i, Lr in enumerate(wl.layers):
            if Lr["kind"] == "psp_spike":
                a = by[(i, "a")].detach().requires_grad_(True)
                if i in delays:
                    if args.unfused:
                        dd = delays[i]
                        y = dd(net.spike(net.psp(a))) if Lr["learn_delay"] else net.delayShift(net.spike(net.psp(a)), dd, wl.Ts)
                    else:
                        y = net.spikeDelayed(net.psp(a), delays[i])
                else:
                    y = net.spike(net.psp(a))
                heads.append(y)
                grads.append(by[(i, "g")])
                results += [y.detach, lambda a=a: a.grad]
            elif Lr["kind"] == "spike_w" and chained:
                if i == 0:
                    results.append(net.psp(by[(0, "s_in")]).detach)            # psp of the network input
                u = by[(i, "u0")].detach().requires_grad_(True)
                if i < last:
                    p_next, packed = net.spikePsp(u)
                    heads.append(p_next)
                    grads.append(by[(i + 1, "g_p")])
                    results += [p_next.detach, (lambda packed=packed: packed.bits)]
                else:
                    y = net.spike(u)
                    heads.append(y)
                    grads.append(by[(i, "g_s")])
                    results.append(y.detach)
                results.append(lambda u=u: u.grad)
            elif Lr["kind"] == "spike_w":
                back = (i, "g_p") in by
                s_in = by[(i, "s_in")].detach().requires_grad_(back)
                u = by[(i, "u0")].detach().requires_grad_(True)
                p = net.psp(s_in)
                y = net.spike(u)
                heads.append(y)
                grads.append(by[(i, "g_s")])
                results += [p.detach, y.detach, lambda u=u: u.grad]
                if back:
                    heads.append(p)
                    grads.append(by[(i, "g_p")])
                    results.append(lambda s_in=s_in: s_in.grad)
            else:
                w = by[(i, "w")].detach().requires_grad_(True)
                y = net.delayShift(net.spikeLoihi(w), 1) if args.unfused else net.spikeLoihiDelayed(w, 1)
                heads.append(y)
                grads.append(by[(i, "g")])
                results += [y.detach, lambda w=w: w.grad]
        torch.autograd.backward(heads, grads)
        return tuple(r() for r in results)

    def pin(t):
        h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        h.copy_(t)
        return h

    h_in = [pin(t) for t in dev_in]
    probe = device_step(*[t[:1] for t in dev_in]) if dev_in[0].shape[0] > 1 else device_step(*dev_in)
    batch = dev_in[0].shape[0]
    h_out = [torch.empty((batch,) + tuple(o.shape[1:]), dtype=o.dtype, pin_memory=True) for o in probe]
    del probe
    h2d = sum(t.numel() * 4 for t in h_in)
    d2h = sum(t.numel() * 4 for t in h_out)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def timed(step):
        for _ in range(2):
            step()
        barrier()
        ev = []
        for _ in range(steps):
            flush_l2(flush)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            ev.append((e0, e1))
        barrier()
        return sum(a.elapsed_time(b) for a, b in ev)

    small = h2d < (1 << 30)
    serial_total = 0.0
    want = None
    if small:          # the single-call form: one copy-in, one step, one copy-out
        def e2e_serial():
            outs = device_step(*[h.to(device, non_blocking=True) for h in h_in])
            for h, o in zip(h_out, outs):
                h.copy_(o, non_blocking=True)
        serial_total = timed(e2e_serial)
        want = [h.clone() for h in h_out]
    chunks = min(args.e2e_chunks, batch)
    capture = False if (args.no_graph or not small) else args.e2e_capture
    pipe = HostPipeline(device, chunks=chunks, capture=capture)
    total = timed(lambda: pipe.run(device_step, h_in, h_out))
    if want is not None:                   # chunking must not change a single bit
        for a, b in zip(want, h_out):
            if not torch.equal(a.view(torch.int32), b.view(torch.int32)):
                raise RuntimeError("pipelined end-to-end result differs from the single-call result")
    how = "HostPipeline: %d batch chunks, copies and kernels overlapped on three streams%s; %d host tensors in, %d out%s" % (
        len(chunk_bounds(batch, chunks)), ", each chunk's step one CUDA-graph launch" if capture else "", len(h_in), len(h_out),
        "; spike -> psp of the next layer as one node (spikePsp): spikes cross as bits, their gradients not at all" if chained else "")
    del pipe, h_in, h_out
    return {"ms_total": total, "serial_ms_total": serial_total, "steps": steps, "h2d": h2d, "d2h": d2h, "how": how}


def all_configs(args, ops, device, flush, peak, peak_kind, main_out):
    """Resident-input numbers of every configuration (the main one is copied from the line itself)."""
    res = {}
    for cfg in (1, 2, 3, 4, 5):
        if cfg == args.config:
            res[str(cfg)] = {"value": main_out["value"], "ms_per_step": main_out["ms_per_step"],
                             "chain_frac_of_bound": main_out["chain"]["frac_of_bound"],
                             "units_per_step": main_out["config"]["neuron_timesteps_per_step_per_gpu"],
                             "dominant": main_out["roofline"]["kernel"], "dominant_frac": main_out["roofline"]["frac"],
                             "dominant_bound": main_out["roofline"]["bound"]}
            continue
        try:
            wl = build_workload(cfg, ops, device)
            steps = min(args.steps, 20)
            total_ms, eager_ms, per_op, _, note = time_resident(wl, ops, steps, 3, device, 1, flush, not args.no_graph, False)
            sm = main_out["clocks"]["sm_mhz"] or 1965.0
            roof = roofline_of(wl, per_op, peak, peak_kind, sm)
            ms = total_ms / steps
            res[str(cfg)] = {"workload": wl.name, "value": wl.units / (ms * 1e-3), "ms_per_step": ms,
                             "eager_ms_per_step": eager_ms / steps, "units_per_step": wl.units,
                             "chain_frac_of_bound": round(wl.chain_bound_ms(ops.fused, peak, sm) / ms, 4),
                             "dominant": roof["kernel"], "dominant_launch": roof["launch"], "dominant_bound": roof["bound"],
                             "dominant_frac": roof["frac"], "dominant_hbm_frac": roof["hbm"]["frac"],
                             "spike_rates": [round(r, 4) for r in wl.rates], "per_op": op_table_of(wl, per_op)}
            del wl
        except Exception as e:
            res[str(cfg)] = {"error": repr(e)[:300]}
        torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------ loss leg
LOSS_PARAMS = {"neuron": dict(SRM_NEURON), "simulation": {"Ts": 1.0, "tSample": 300},
               "training": {"error": {"type": "NumSpikes", "tgtSpikeRegion": {"start": 0, "stop": 300},
                                      "tgtSpikeCount": {True: TGT_TRUE, False: TGT_FALSE}}}}


def time_num_spikes_loss(loss_module, spikes, desired, iters=50):
    """Wall-clock time of numSpikes forward + backward on an output layer's spikes (host
    synchronised on both sides: what a training loop waits for)."""
    for _ in range(5):
        x = spikes.clone().requires_grad_(True)
        loss_module.numSpikes(x, desired).backward()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(iters):
        x = spikes.clone().requires_grad_(True)
        loss_module.numSpikes(x, desired).backward()
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) / iters * 1e3


def loss_inputs(device):
    gen = torch.Generator().manual_seed(5)
    s = bernoulli(gen, (64, 10, 1, 1, 300), 0.1).to(device)
    label = torch.randint(0, 10, (64,), generator=gen)
    desired = torch.zeros(64, 10, 1, 1, 1)
    desired[torch.arange(64), label] = 1
    return s, desired


def loss_leg(ops, device):
    from slayerpytorch_b200 import loss as device_loss
    s, desired = loss_inputs(device)
    return {"what": "spikeLoss.numSpikes forward + backward on 64 x 10 x 300 output spikes, wall clock, tensors on the device, "
                    "no host round trip", "ms": time_num_spikes_loss(device_loss.spikeLoss(LOSS_PARAMS).to(device), s, desired.to(device))}


# ------------------------------------------------------------------------------- CPU legs
def cpu_workload(cfg, ops):
    """The configuration on a batch subsample, built and run with the CPU oracle."""
    batch = CPU_SAMPLE_BATCH[cfg]
    wl = build_workload(cfg, ops, torch.device("cpu"), batch_override=batch)
    return wl, batch


def cpu_baseline_value(cfg, reps=3, ops=None):
    ops = ops or OracleOps()
    wl, batch = cpu_workload(cfg, ops)
    best = None
    for _ in range(reps):
        wl.prep()
        t0 = time.perf_counter()
        wl.step(ops)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": wl.units / best, "unit": UNIT, "cores": ops.threads, "kind": "port",
            "sample": "batch %d of %d of config %d (rows are independent: the rate does not depend on the batch), "
                      "the reference's sequence of operators, best of %d passes, C oracle with OpenMP"
                      % (batch, FULL_BATCH[cfg], cfg, reps),
            "ms_per_sample_step": best * 1e3}


def load_reference_cuda():
    """The reference's own CUDA operators, if they were built (oracle/_ref/)."""
    import importlib.machinery
    import importlib.util
    mods = []
    for name in ("slayerCuda_ref", "slayerLoihiCuda_ref"):
        path = os.path.join(ROOT, "oracle", "_ref", name + ".so")
        if not os.path.isfile(path):
            return None
        loader = importlib.machinery.ExtensionFileLoader(name, path)
        spec = importlib.util.spec_from_loader(name, loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
        mods.append(mod)
    return mods


def time_reference(args, rank, world):
    if rank != 0:
        return None
    ops = OracleOps()
    wl, batch = cpu_workload(args.config, ops)
    warm = max(args.warmup, 3)
    for _ in range(warm):
        wl.prep()
        wl.step(ops)
    dt = 0.0
    for _ in range(args.steps):
        wl.prep()
        t0 = time.perf_counter()
        wl.step(ops)
        dt += time.perf_counter() - t0
    value = wl.units * args.steps / dt
    sample = ("each step = batch %d of the configuration's %d (rows are independent: the rate does not depend on the batch)"
              % (batch, FULL_BATCH[args.config]))
    out = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
           "steps": args.steps, "warmup": warm, "ms_per_step": dt / args.steps * 1e3,
           "higher_is_better": True, "scaling": "weak" if world == 1 else args.scaling, "vs_baseline": None, "dtype": "f32",
           "data": "synthetic",
           "config": {"workload": wl.name,
                      "what": "explicit time-loop formulation of the reference operators (C restatement, OpenMP) on the host cores; " + sample},
           "cpu_baseline": {"value": value, "unit": UNIT, "cores": ops.threads, "kind": "port", "sample": sample},
           "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    del wl
    if torch.cuda.is_available() and not args.no_reference_cuda:
        try:
            mods = load_reference_cuda()
            if mods is not None:
                rops = RefCudaOps(*mods)
                cfgs = (1, 2, 3, 4, 5) if not args.no_all_configs else (args.config,)
                out["reference_cuda"] = {str(c): time_reference_cuda(rops, c, max(3, min(args.steps, 10))) for c in cfgs}
        except Exception as e:
            out["reference_cuda"] = {"unavailable": repr(e)[:200]}
        # the reference's own loss on this build's operators is timed in a process of its own, so
        # that this one loads nothing but the oracle and the reference
        try:
            r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference_loss"],
                               stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, timeout=300)
            out["reference_loss"] = json.loads(r.stdout.strip().splitlines()[-1])
        except Exception as e:
            out["reference_loss"] = {"unavailable": repr(e)[:200]}
    return out


def time_reference_loss():
    """The reference's own spikeLoss.py (installed under oracle/_ref by oracle/build_ref.py),
    unchanged: the NumPy round trip through the host is what is being timed."""
    import contextlib
    import importlib
    import io
    import types
    src = os.path.join(ROOT, "oracle", "_ref", "slayerSNN")
    if not os.path.isfile(os.path.join(src, "spikeLoss.py")):
        return {"unavailable": "reference Python package not installed under oracle/_ref"}
    import slayerpytorch_b200
    sc, lc = slayerpytorch_b200.load_ops()
    sys.modules.setdefault("slayerCuda", sc)
    sys.modules.setdefault("slayerLoihiCuda", lc)
    pkg = types.ModuleType("slayerSNN_bench")
    pkg.__path__ = [src]
    sys.modules["slayerSNN_bench"] = pkg
    with contextlib.redirect_stdout(io.StringIO()):
        ref_loss = importlib.import_module("slayerSNN_bench.spikeLoss")
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    s, desired = loss_inputs(device)
    return {"what": "the reference's spikeLoss.numSpikes forward + backward on the same 64 x 10 x 300 spikes, wall clock",
            "ms": time_num_spikes_loss(ref_loss.spikeLoss(LOSS_PARAMS).to(device), s, desired)}


def time_reference_cuda(rops, cfg, steps):
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    try:
        wl = build_workload(cfg, rops, device)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
        for _ in range(3):
            wl.prep()
            wl.step(rops)
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(steps):
            wl.prep()
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            wl.step(rops)
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        res = {"what": "the reference's CUDA kernels recompiled for sm_100, same chain (its own sequence of launches), same GPU, inputs resident",
               "value": wl.units * steps / (total * 1e-3), "unit": UNIT, "ms_per_step": total / steps, "steps": steps}
        del wl, flush
    except Exception as e:
        res = {"unavailable": repr(e)[:200]}
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_loss"])
    ap.add_argument("--config", type=int, default=3, choices=[1, 2, 3, 4, 5], help="workload (see the module docstring)")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N > 1: split the configuration's batch over the ranks (strong) or give every rank a full batch (weak)")
    ap.add_argument("--unfused", action="store_true",
                    help="the reference's sequence of launches instead of the fused getSpikesDelayed / spikeGradShift operators")
    ap.add_argument("--no-graph", action="store_true", help="time the eager launch loop instead of a CUDA-graph replay")
    ap.add_argument("--e2e-chunks", type=int, default=8, help="batch chunks of the end-to-end host pipeline")
    ap.add_argument("--e2e-steps", type=int, default=10, help="at most this many end-to-end steps are timed")
    ap.add_argument("--e2e-capture", default="chunk", choices=["pipeline", "chunk"],
                    help="CUDA-graph granularity of the end-to-end pipeline (small workloads only)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end (host buffers) measurement, e.g. under a profiler")
    ap.add_argument("--no-all-configs", action="store_true", help="skip the resident-input numbers of the other configurations")
    ap.add_argument("--no-reference-cuda", action="store_true", help="reference arm: skip the reference's CUDA kernels")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference_loss":
        print(json.dumps(time_reference_loss()), flush=True)
        return 0
    if args.impl == "reference":
        out = time_reference(args, rank, world)
        if out is not None:
            print(json.dumps(out), flush=True)
        return 0

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the GPU arm has no CPU fallback")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=device)
    try:
        out = time_ours(args, rank, world, device)
        if out is not None:
            print(json.dumps(out), flush=True)
    finally:
        if world > 1:
            torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
