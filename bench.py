#!/usr/bin/env python
"""Benchmark of the SLAYER spiking-neuron hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload ("step"): one forward+backward pass of the hot path over one batch of the SRM MLP
2312-512-10 (batch 64 per GPU, T = 300, Ts = 1 ms, 5 % input spike rate): for the hidden layer
psp -> getSpikes -> per-neuron delay shift, then shift^-1 -> surrogate gradient -> corr; for the
output layer the same without the delay.  Dense weighting stays in PyTorch and runs once, during
set-up, to produce the tensors the hot path consumes; the gradients that enter the backward pass
come from the spike-count loss of the same network.  Data is synthetic and seeded.

Metric: neuron-timesteps per second = batch * (512 + 10) * 300 per step / step time, summed over
all GPUs (weak scaling: every rank processes its own batch of 64; no collective on this path).

One JSON line is printed by rank 0.  ``value`` is measured with inputs resident in HBM, L2
flushed between steps, CUDA events around each step, the step's launches replayed from a
CUDA graph (``eager_ms_per_step`` is the same loop launched call by call); ``e2e`` is the same
chain through the package's public layer API with host (pinned) buffers, copies inside the
timed region, streamed in batch chunks by ``HostPipeline`` (``single_call_ms_per_step`` is one
copy-in, one step, one copy-out);
``roofline`` describes the kernel with the largest share of the step; ``cpu_baseline`` is the C
oracle on the host cores.  ``--impl reference`` times the explicit time-loop formulation (the C
oracle, all host threads) on the same workload and, when the reference's own CUDA operators
were built, adds their timing on this GPU as ``reference_cuda``.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np
import torch

METRIC = "neuron-timesteps/s, SRM getSpikes+psp+shift forward/backward"
UNIT = "neuron-timesteps/s"
NEURON = {"type": "SRMALPHA", "theta": 10, "tauSr": 10.0, "tauRef": 1.0, "scaleRef": 2,
          "tauRho": 1, "scaleRho": 1}
SIM = {"Ts": 1.0, "tSample": 300}
BATCH, N_IN, N_HID, N_OUT, T = 64, 2312, 512, 10, 300
TGT_TRUE, TGT_FALSE = 60, 10

# algorithmic bytes per neuron-timestep of each operator (read + write of fp32 tensors)
ALG_BYTES = {"conv": 8, "corr": 8, "getSpikes": 12, "shift": 8, "spikeGrad": 12, "spikeGradShift": 12,
             "getSpikesDelayed": 12}
KERNEL_OF = {"conv": "fir_kernel", "corr": "fir_kernel", "getSpikes": "srm_get_spikes_tma_kernel",
             "shift": "shift_vec4_kernel", "spikeGrad": "spike_grad_vec4_kernel",
             "spikeGradShift": "spike_grad_shift_rows_kernel", "getSpikesDelayed": "srm_get_spikes_tma_kernel"}
# DRAM bytes per element measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum of one
# launch over its element count); see the summaries under profiles/.  None = not captured yet.
NCU_TRAFFIC_PER_ELEMENT = {"fir_kernel": 7.33, "srm_get_spikes_tma_kernel": 11.62,
                           "shift_vec4_kernel": None, "spike_grad_vec4_kernel": None}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ------------------------------------------------------------------------ response kernels
def response_kernels():
    from slayerpytorch_b200.layer import alpha_kernel
    srm = torch.tensor(alpha_kernel(NEURON["tauSr"], SIM["Ts"], SIM["tSample"]), dtype=torch.float32)
    ref = torch.tensor(alpha_kernel(NEURON["tauRef"], SIM["Ts"], SIM["tSample"],
                                    mult=-NEURON["scaleRef"] * NEURON["theta"]), dtype=torch.float32)
    return srm, ref


class OracleOps:
    """The CPU oracle behind the operator names of slayerCuda (torch CPU tensors in and out).
    Used only by the cpu_baseline leg and the reference arm."""

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


# -------------------------------------------------------------------------------- workload
def make_workload(ops, device, seed, batch=BATCH):
    """Tensors the hot path consumes, produced by running the network once (untimed):
    a1, a2 = weighted input spikes of the two layers, g1 = gradient arriving at the delayed
    hidden spikes, g2 = gradient arriving at the output spikes, delay = per-neuron delays."""
    gen = torch.Generator().manual_seed(seed)
    srm, ref = response_kernels()
    x = (torch.rand(batch, N_IN, 1, 1, T, generator=gen) < 0.05).float()
    # dense layers: PyTorch Conv3d default init times weightScale = 10 (src/slayer.py:187, :420)
    w1 = torch.empty(N_HID, N_IN).uniform_(-1, 1, generator=gen) * (10.0 / N_IN ** 0.5)
    w2 = torch.empty(N_OUT, N_HID).uniform_(-1, 1, generator=gen) * (10.0 / N_HID ** 0.5)
    delay = (torch.rand(N_HID, generator=gen) * 5).float()
    label = torch.randint(0, N_OUT, (batch,), generator=gen)
    x, w1, w2, srm, ref, delay = (t.to(device) for t in (x, w1, w2, srm, ref, delay))
    Ts, theta = SIM["Ts"], float(NEURON["theta"])
    tau, scale = float(NEURON["tauRho"] * NEURON["theta"]), float(NEURON["scaleRho"])

    def dense(w, s):       # [N, Cin, 1, 1, T] -> [N, Cout, 1, 1, T]
        return torch.einsum("oc,nct->not", w, s[:, :, 0, 0, :]).reshape(s.shape[0], w.shape[0], 1, 1, T).contiguous()

    a1 = dense(w1, x)
    u1 = ops.conv(a1, srm, Ts)
    s1 = ops.getSpikes(u1, ref, theta, Ts)
    d1 = ops.shift(s1, delay, Ts)
    a2 = dense(w2, d1)
    u2 = ops.conv(a2, srm, Ts)
    s2 = ops.getSpikes(u2, ref, theta, Ts)
    # spike-count loss (src/spikeLoss.py:60-104, target region = whole sample): error signal
    # (count - target) / T at every step; its gradient w.r.t. the output spikes goes through psp
    count = s2.sum(-1, keepdim=True) * Ts
    target = torch.full((batch, N_OUT, 1, 1, 1), float(TGT_FALSE), device=count.device)
    target[torch.arange(batch), label.to(count.device)] = float(TGT_TRUE)
    err = ((count - target) / T).expand(-1, -1, -1, -1, T).contiguous()
    g2 = ops.corr(err * Ts, srm, Ts)
    gu2 = ops.spikeGrad(g2, u2, theta, tau, scale)
    ga2 = ops.corr(gu2, srm, Ts)
    g1 = torch.einsum("oc,not->nct", w2, ga2[:, :, 0, 0, :]).reshape(batch, N_HID, 1, 1, T).contiguous()
    rates = {"hidden": float(s1.mean()), "output": float(s2.mean())}
    return dict(a1=a1, a2=a2, g1=g1, g2=g2, delay=delay, neg_delay=-delay, srm=srm, ref=ref, rates=rates,
                theta=theta, tau=tau, scale=scale, Ts=Ts)


def workload_name(wl):
    return ("config 2: SRM MLP 2312-512-10 hot path, batch 64 per GPU, T=300, Ts=1, input rate 5%%, psp K=%d, "
            "refractory %d taps, delays U(0,5)" % (wl["srm"].numel(), wl["ref"].numel()))


def hot_path(ops, wl, record=None):
    """One step.  `record(name, rows, fn)` wraps an operator call for per-kernel timing."""
    Ts, theta, tau, scale = wl["Ts"], wl["theta"], wl["tau"], wl["scale"]
    srm, ref, delay = wl["srm"], wl["ref"], wl["delay"]
    run = record or (lambda name, big, fn: fn())
    # hidden layer: forward
    u1 = run("conv", True, lambda: ops.conv(wl["a1"], srm, Ts))
    if wl.get("unfused"):
        s1 = run("getSpikes", True, lambda: ops.getSpikes(u1, ref, theta, Ts))
        d1 = run("shift", True, lambda: ops.shift(s1, delay, Ts))
    else:       # the spikes are written once, already delayed (same bits as the two launches)
        d1 = run("getSpikesDelayed", True, lambda: ops.getSpikesDelayed(u1, ref, theta, Ts, delay))
    # hidden layer: backward
    if wl.get("unfused"):
        b1 = run("shift", True, lambda: ops.shift(wl["g1"], wl["neg_delay"], Ts))
        b2 = run("spikeGrad", True, lambda: ops.spikeGrad(b1, u1, theta, tau, scale))
    else:       # shift back and surrogate gradient in one pass (same bits, no intermediate tensor)
        b2 = run("spikeGradShift", True,
                 lambda: ops.spikeGradShift(wl["g1"], u1, wl["neg_delay"], theta, tau, scale, Ts))
    b3 = run("corr", True, lambda: ops.corr(b2, srm, Ts))
    # output layer: forward and backward
    u2 = run("conv", False, lambda: ops.conv(wl["a2"], srm, Ts))
    s2 = run("getSpikes", False, lambda: ops.getSpikes(u2, ref, theta, Ts))
    c2 = run("spikeGrad", False, lambda: ops.spikeGrad(wl["g2"], u2, theta, tau, scale))
    c3 = run("corr", False, lambda: ops.corr(c2, srm, Ts))
    return d1, b3, s2, c3


def launches_per_step(wl):
    return 10 if wl.get("unfused") else 8


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


# --------------------------------------------------------------------------------- our arm
def flush_l2(buf):
    buf.zero_()


def time_ours(args, rank, world, device):
    import slayerpytorch_b200
    from slayerpytorch_b200 import layer as L
    from slayerpytorch_b200.hoststream import HostPipeline, chunk_bounds
    slayerCuda, _ = slayerpytorch_b200.load_ops()
    peak, peak_kind = measured_peak_gbs()

    wl = make_workload(slayerCuda, device, seed=1002 + 97 * rank)
    wl["unfused"] = bool(args.unfused)
    units = BATCH * (N_HID + N_OUT) * T
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # ---- resident-input timing with per-operator events
    per_op = {}

    def recorder(events):
        def run(name, big, fn):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn()
            e1.record()
            events.append((name, big, e0, e1))
            return out
        return run

    for _ in range(max(args.warmup, 3)):
        flush_l2(flush)
        hot_path(slayerCuda, wl)
    barrier()

    # The launches of a step are short (7-50 us), so the step is replayed from a CUDA graph
    # captured once: the same kernels on the same buffers, without per-launch host overhead.
    graph, graph_note = None, None
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                hot_path(slayerCuda, wl)
            for _ in range(3):
                flush_l2(flush)
                graph.replay()
        except Exception as e:             # reported, and the eager loop below is timed instead
            graph, graph_note = None, "capture failed: %r" % (e,)
        barrier()

    def timed_steps(step):
        events = []
        for _ in range(args.steps):
            flush_l2(flush)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            events.append((e0, e1))
        barrier()
        return sum(a.elapsed_time(b) for a, b in events)

    sampler = ClockSampler(device.index)
    sampler.start()
    eager_ms = timed_steps(lambda: hot_path(slayerCuda, wl))
    total_ms = timed_steps(graph.replay) if graph is not None else eager_ms
    clocks = sampler.stop()

    # per-operator breakdown: a separate eager pass with an event pair around every launch
    op_events = []
    for _ in range(min(args.steps, 50)):
        flush_l2(flush)
        hot_path(slayerCuda, wl, recorder(op_events))
    barrier()
    for name, big, a, b in op_events:
        per_op.setdefault((name, big), []).append(a.elapsed_time(b))

    # ---- end to end through the public layer API with host buffers
    net = L.spikeLayer(dict(NEURON), dict(SIM)).to(device)
    pin = lambda t: t.detach().cpu().pin_memory()
    h_in = {k: pin(wl[k]) for k in ("a1", "a2", "g1", "g2")}
    h_out = {k: torch.empty_like(h_in[k]) .pin_memory() for k in ("a1", "a2", "g1", "g2")}
    delay_dev = wl["delay"]

    def device_step(a1, a2, g1, g2):
        a1 = a1.detach().requires_grad_(True)
        a2 = a2.detach().requires_grad_(True)
        if args.unfused:
            d1 = net.delayShift(net.spike(net.psp(a1)), delay_dev, SIM["Ts"])
        else:
            d1 = net.spikeDelayed(net.psp(a1), delay_dev)
        s2 = net.spike(net.psp(a2))
        torch.autograd.backward([d1, s2], [g1, g2])
        return d1.detach(), s2.detach(), a1.grad, a2.grad

    order = ("a1", "a2", "g1", "g2")

    def e2e_serial():
        outs = device_step(*[h_in[k].to(device, non_blocking=True) for k in order])
        for k, o in zip(order, outs):
            h_out[k].copy_(o, non_blocking=True)

    pipe = HostPipeline(device, chunks=args.e2e_chunks, capture=False if args.no_graph else args.e2e_capture)

    def e2e_pipelined():
        pipe.run(device_step, [h_in[k] for k in order], [h_out[k] for k in order])

    def time_e2e(step):
        for _ in range(3):
            step()
        barrier()
        return timed_steps(step)

    e2e_serial_ms = time_e2e(e2e_serial)
    want = {k: h_out[k].clone() for k in order}
    e2e_ms = time_e2e(e2e_pipelined)
    for k in order:                        # chunking must not change a single bit
        if not torch.equal(want[k].view(torch.int32), h_out[k].view(torch.int32)):
            raise RuntimeError("pipelined end-to-end result differs from the single-call result in " + k)
    bytes_io = sum(t.numel() * 4 for t in h_in.values())

    # ---- max over ranks
    t = torch.tensor([total_ms, e2e_ms, eager_ms, e2e_serial_ms], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    total_ms, e2e_ms, eager_ms, e2e_serial_ms = (float(x) for x in t)

    if rank != 0:
        return None

    # ---- roofline of the kernel with the largest share (hidden-layer launches)
    share = {}
    for (name, big), v in per_op.items():
        share[KERNEL_OF[name]] = share.get(KERNEL_OF[name], 0.0) + sum(v)
    dominant = max(share, key=share.get)
    dom_ops = [n for n in ALG_BYTES if KERNEL_OF[n] == dominant]
    dom_times = [x for n in dom_ops for x in per_op.get((n, True), [])]
    el_big = BATCH * N_HID * T
    avg_ms = sum(dom_times) / len(dom_times)
    alg_bytes = ALG_BYTES[dom_ops[0]] * el_big
    achieved = alg_bytes / (avg_ms * 1e-3) / 1e9
    tpe = NCU_TRAFFIC_PER_ELEMENT.get(dominant)
    roofline = {"bound": "hbm", "kernel": dominant, "launch": "hidden layer, %d x %d fp32" % (BATCH * N_HID, T),
                "achieved": round(achieved, 1), "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                "frac": round(achieved / peak, 4), "traffic": (tpe * el_big if tpe else None),
                "algorithmic_bytes": alg_bytes, "avg_launch_us": round(avg_ms * 1e3, 2)}
    if dominant == "fir_kernel":
        k = int(wl["srm"].numel())
        fma_peak = 148 * 128 * 2 * (clocks["sm_mhz"] or 1965.0) * 1e6 / 1e12
        roofline["fp32_fma"] = {"achieved_tflops": round(2 * k * el_big / (avg_ms * 1e-3) / 1e12, 2),
                                "peak_tflops_at_sampled_clock": round(fma_peak, 1), "taps": k}
    op_table = {}
    for (name, big), v in sorted(per_op.items()):
        el = el_big if big else BATCH * N_OUT * T
        us = 1e3 * sum(v) / len(v)
        op_table["%s/%s" % (name, "hidden" if big else "output")] = {
            "us": round(us, 2), "GB/s": round(ALG_BYTES[name] * el / (us * 1e-6) / 1e9, 1),
            "share": round(sum(v) / sum(sum(x) for x in per_op.values()), 3)}

    # ---- CPU baseline (C oracle, all host threads) on the full batch, best of 3
    cpu = cpu_baseline_value(reps=3)

    out = {
        "metric": METRIC, "value": world * units * args.steps / (total_ms * 1e-3), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(wl),
                   "fusion": "none: the reference's sequence of ten launches" if args.unfused else
                             "hidden layer: getSpikes+delay as one launch (getSpikesDelayed), shift back + surrogate "
                             "gradient as one launch (spikeGradShift); same results, eight launches",
                   "neuron_timesteps_per_step_per_gpu": units, "l2": "flushed between steps (256 MiB write)",
                   "spike_rates": wl["rates"], "parallelism": "batch sharded, no collective"},
        "clocks": clocks,
        "e2e": {"value": world * units * args.steps / (e2e_ms * 1e-3), "unit": UNIT,
                "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": bytes_io, "d2h_bytes_per_step": bytes_io,
                "how": "HostPipeline: %d batch chunks, copies and kernels overlapped on three streams%s"
                       % (len(chunk_bounds(BATCH, args.e2e_chunks)),
                          "" if args.no_graph else (", the whole step one CUDA-graph launch" if args.e2e_capture == "pipeline"
                                                    else ", each chunk's step one CUDA-graph launch")),
                "single_call_ms_per_step": e2e_serial_ms / args.steps,
                "pcie_GB/s_per_direction": round(bytes_io / (e2e_ms / args.steps * 1e-3) / 1e9, 1)},
        "launch_mode": ("cuda graph replay of the step's %d launches" % launches_per_step(wl)) if graph is not None
                       else ("eager" + (" (%s)" % graph_note if graph_note else "")),
        "eager_ms_per_step": eager_ms / args.steps,
        "gpu_launches": launches_per_step(wl) * args.steps,
        "roofline": roofline,
        "cpu_baseline": cpu,
        "per_op": op_table,
    }
    if world == 1:
        from slayerpytorch_b200 import loss as device_loss
        s2, desired = loss_inputs(slayerCuda, wl, device)
        out["loss"] = {"what": "spikeLoss.numSpikes forward + backward on the output spikes (%d x %d x %d), wall clock, "
                               "tensors on the device, no host round trip" % (BATCH, N_OUT, T),
                       "ms": time_num_spikes_loss(device_loss.spikeLoss(LOSS_PARAMS).to(device), s2, desired.to(device))}
    if world == 1 and not args.no_scaled:
        out["scaled"] = scaled_variant(slayerCuda, device, peak)
    return out


def scaled_variant(ops, device, peak):
    """Hidden-layer chain with the batch scaled until every tensor is >= 1 GiB (DRAM-resident)."""
    batch = 1792
    el = batch * N_HID * T
    gen = torch.Generator(device=device).manual_seed(7)
    srm, ref = (t.to(device) for t in response_kernels())
    a = (torch.randn(batch, N_HID, 1, 1, T, device=device, generator=gen).abs() * 1.2
         * (torch.rand(batch, N_HID, 1, 1, T, device=device, generator=gen) < 0.3)).float()
    g = torch.randn(batch, N_HID, 1, 1, T, device=device, generator=gen)
    delay = torch.rand(N_HID, device=device, generator=gen) * 5
    neg_delay = -delay
    Ts, theta, tau, scale = 1.0, 10.0, 10.0, 1.0
    times = {}

    def run(name, fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        times.setdefault(name, []).append((e0, e1))
        return out

    rate = None
    for it in range(5):
        u = run("conv", lambda: ops.conv(a, srm, Ts))
        s = run("getSpikes", lambda: ops.getSpikes(u, ref, theta, Ts))
        d = run("shift", lambda: ops.shift(s, delay, Ts))
        u_again = ops.conv(a, srm, Ts)
        df = run("getSpikesDelayed", lambda: ops.getSpikesDelayed(u_again, ref, theta, Ts, delay))
        del u_again, df
        b1 = run("shift", lambda: ops.shift(g, neg_delay, Ts))
        b2 = run("spikeGrad", lambda: ops.spikeGrad(b1, u, theta, tau, scale))
        b2f = run("spikeGradShift", lambda: ops.spikeGradShift(g, u, neg_delay, theta, tau, scale, Ts))
        b3 = run("corr", lambda: ops.corr(b2, srm, Ts))
        if rate is None:
            rate = float(s.mean())
        del u, s, d, b1, b2, b2f, b3
    torch.cuda.synchronize()
    res, t_of = {}, {}
    for name, evs in times.items():
        ms = [a_.elapsed_time(b_) for a_, b_ in evs[len(evs) // 5 * 2:]]     # drop 2 warm-up rounds
        t = sum(ms) / len(ms)
        t_of[name] = t
        gbs = ALG_BYTES[name] * el / (t * 1e-3) / 1e9
        res[name] = {"ms": round(t, 4), "GB/s": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak, 4)}
    # the chain as the benchmark step runs it: conv, getSpikesDelayed, spikeGradShift, corr (40 bytes
    # per element); the reference's sequence has two shifts and a separate spikeGrad (56 bytes)
    total = t_of["conv"] + t_of["getSpikesDelayed"] + t_of["spikeGradShift"] + t_of["corr"]
    total_ref_seq = t_of["conv"] + t_of["getSpikes"] + 2 * t_of["shift"] + t_of["spikeGrad"] + t_of["corr"]
    return {"workload": "hidden-layer chain, batch %d (%d x %d fp32 = %.2f GiB per tensor)"
                        % (batch, batch * N_HID, T, el * 4 / 2 ** 30),
            "value": el / (total * 1e-3), "unit": UNIT, "ms_per_step": total,
            "chain_GB/s": round(40 * el / (total * 1e-3) / 1e9, 1),
            "chain_frac_of_hbm_peak": round(40 * el / (total * 1e-3) / 1e9 / peak, 4),
            "reference_sequence_ms_per_step": total_ref_seq,
            "spike_rate": rate, "per_op": res}


# ------------------------------------------------------------------------------ loss leg
LOSS_PARAMS = {"neuron": dict(NEURON), "simulation": dict(SIM),
               "training": {"error": {"type": "NumSpikes", "tgtSpikeRegion": {"start": 0, "stop": T},
                                      "tgtSpikeCount": {True: TGT_TRUE, False: TGT_FALSE}}}}


def time_num_spikes_loss(loss_module, spikes, desired, iters=50):
    """Wall-clock time of numSpikes forward + backward on the output layer's spikes (host
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


def loss_inputs(ops, wl, device):
    u2 = ops.conv(wl["a2"], wl["srm"], wl["Ts"])
    s2 = ops.getSpikes(u2, wl["ref"], wl["theta"], wl["Ts"])
    gen = torch.Generator().manual_seed(5)
    label = torch.randint(0, N_OUT, (BATCH,), generator=gen)
    desired = torch.zeros(BATCH, N_OUT, 1, 1, 1)
    desired[torch.arange(BATCH), label] = 1
    return s2, desired


# ------------------------------------------------------------------------------- CPU legs
def cpu_baseline_value(reps=3, ops=None):
    ops = ops or OracleOps()
    wl = make_workload(ops, torch.device("cpu"), seed=1002)
    wl["unfused"] = True            # the reference's own sequence of operators
    units = BATCH * (N_HID + N_OUT) * T
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        hot_path(ops, wl)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": units / best, "unit": UNIT, "cores": ops.threads, "kind": "port",
            "sample": "full config-2 batch (64 samples), best of %d passes, C oracle with OpenMP" % reps,
            "ms_per_step": best * 1e3}


def load_reference_cuda():
    """The reference's own CUDA operators, if they were built (oracle/_ref/)."""
    import importlib.machinery
    import importlib.util
    path = os.path.join(ROOT, "oracle", "_ref", "slayerCuda_ref.so")
    if not os.path.isfile(path):
        return None
    loader = importlib.machinery.ExtensionFileLoader("slayerCuda_ref", path)
    spec = importlib.util.spec_from_loader("slayerCuda_ref", loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


class RefCudaOps:
    """Reference CUDA operators plus the tensor expression it uses for the surrogate gradient."""

    def __init__(self, mod):
        self.m = mod
        self.conv, self.corr, self.getSpikes, self.shift = mod.conv, mod.corr, mod.getSpikes, mod.shift

    def spikeGrad(self, g, u, theta, tau, scale):
        th, ta, sc = (torch.tensor(v, device=g.device, dtype=g.dtype) for v in (theta, tau, scale))
        return g * (sc / ta * torch.exp(-torch.abs(u - th) / ta))


def time_reference(args, rank, world):
    if rank != 0:
        return None
    ops = OracleOps()
    wl = make_workload(ops, torch.device("cpu"), seed=1002)
    wl["unfused"] = True            # the reference's own sequence of operators
    units = BATCH * (N_HID + N_OUT) * T
    for _ in range(max(1, min(args.warmup, 3))):
        hot_path(ops, wl)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        hot_path(ops, wl)
    dt = time.perf_counter() - t0
    value = units * args.steps / dt
    out = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
           "steps": args.steps, "warmup": max(1, min(args.warmup, 3)), "ms_per_step": dt / args.steps * 1e3,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
           "data": "synthetic",
           "config": {"workload": workload_name(wl),
                      "what": "explicit time-loop formulation of the reference operators (C restatement, OpenMP) on the host cores"},
           "cpu_baseline": {"value": value, "unit": UNIT, "cores": ops.threads, "kind": "port",
                            "sample": "full config-2 batch per step"},
           "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    if torch.cuda.is_available():
        try:
            mod = load_reference_cuda()
            if mod is not None:
                out["reference_cuda"] = time_reference_cuda(RefCudaOps(mod), max(5, min(args.steps, 20)))
        except Exception as e:
            out["reference_cuda"] = {"unavailable": repr(e)[:200]}
        try:
            out["reference_loss"] = time_reference_loss()
        except Exception as e:
            out["reference_loss"] = {"unavailable": repr(e)[:200]}
    return out


def time_reference_loss():
    """The reference's own spikeLoss.py (installed under oracle/_ref by oracle/build_ref.py),
    unchanged, on this build's operator modules: the NumPy round trip is what is being timed."""
    import importlib
    import types
    src = os.path.join(ROOT, "oracle", "_ref", "slayerSNN")
    if not os.path.isfile(os.path.join(src, "spikeLoss.py")):
        return {"unavailable": "reference Python package not installed under oracle/_ref"}
    import slayerpytorch_b200
    ops, loihi_ops = slayerpytorch_b200.load_ops()
    sys.modules.setdefault("slayerCuda", ops)
    sys.modules.setdefault("slayerLoihiCuda", loihi_ops)
    pkg = types.ModuleType("slayerSNN_bench")
    pkg.__path__ = [src]
    sys.modules["slayerSNN_bench"] = pkg
    import contextlib
    import io
    with contextlib.redirect_stdout(io.StringIO()):
        ref_loss = importlib.import_module("slayerSNN_bench.spikeLoss")
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    wl = make_workload(ops, device, seed=1002)
    s2, desired = loss_inputs(ops, wl, device)
    return {"what": "the reference's spikeLoss.numSpikes forward + backward on the same spikes, wall clock",
            "ms": time_num_spikes_loss(ref_loss.spikeLoss(LOSS_PARAMS).to(device), s2, desired)}


def time_reference_cuda(ops, steps):
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    wl = make_workload(ops, device, seed=1002)
    wl["unfused"] = True
    units = BATCH * (N_HID + N_OUT) * T
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    for _ in range(3):
        hot_path(ops, wl)
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        hot_path(ops, wl)
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return {"what": "the reference's CUDA kernels recompiled for sm_100, same chain, same GPU, inputs resident",
            "value": units * steps / (total * 1e-3), "unit": UNIT, "ms_per_step": total / steps}


# ------------------------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--unfused", action="store_true",
                    help="the reference's sequence of ten launches per step instead of the fused "
                         "getSpikesDelayed / spikeGradShift operators")
    ap.add_argument("--no-graph", action="store_true", help="time the eager launch loop instead of a CUDA-graph replay")
    ap.add_argument("--e2e-chunks", type=int, default=8, help="batch chunks of the end-to-end host pipeline")
    ap.add_argument("--e2e-capture", default="chunk", choices=["pipeline", "chunk"],
                    help="CUDA-graph granularity of the end-to-end pipeline: one graph per chunk (faster: 2.1 ms "
                         "against 2.3 ms per step), or the whole step as one graph (least host work)")
    ap.add_argument("--no-scaled", action="store_true", help="skip the batch-scaled (>= 1 GiB tensors) variant")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

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
