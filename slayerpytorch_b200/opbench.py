"""Time one operator on synthetic data of a given shape (CUDA events, inputs resident in HBM).

    python -m slayerpytorch_b200.opbench --op getSpikes --rows 262144 --T 300 --iters 5

Operators: conv, corr, convPacked, getSpikes, getSpikesPacked, getSpikesDelayed, shift, shiftScalar,
spikeGrad, spikeGradShift, corrSpikeGrad, delayGrad, loihi, loihiDelayed.  Prints one JSON line with
the average launch time, algorithmic GB/s (8 bytes per element for conv/corr/shift, 12 for
getSpikes/spikeGrad, 16 for loihi) and elements per second.  Small enough to run under a
profiler: every iteration is exactly one kernel launch of the operator (getSpikes works in
place, so its potential is restored by a device copy between launches).
"""
import argparse
import json
import sys

import torch

import slayerpytorch_b200
from slayerpytorch_b200.layer import alpha_kernel, loihi_psp_kernel

ALG_BYTES = {"conv": 8, "corr": 8, "getSpikes": 12, "shift": 8, "shiftScalar": 8, "spikeGrad": 12, "spikeGradShift": 12, "delayGrad": 8,
             "getSpikesDelayed": 12, "getSpikesPacked": 8.125, "convPacked": 4.125,
             "loihi": 16, "loihiDelayed": 12, "corrSpikeGrad": 12}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=sorted(ALG_BYTES))
    ap.add_argument("--rows", type=int, default=262144)
    ap.add_argument("--T", type=int, default=300)
    ap.add_argument("--K", type=int, default=0, help="filter taps for conv/corr (0 = SRM alpha kernel, 77 taps)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--density", type=float, default=0.3, help="fraction of non-zero input samples")
    ap.add_argument("--neurons", type=int, default=512, help="rows per batch sample (length of the shift table)")
    ap.add_argument("--packed-fir", type=int, default=None, metavar="MODE",
                    help="conv/corr: kernel selection as slayer_b200_set_fir_packed takes it (0 scalar, 1 packed, 2 / 3 tile size)")
    ap.add_argument("--fir-flow", type=int, default=None, metavar="MODE",
                    help="conv/corr: form of the scalar kernel as slayer_b200_set_fir_flow takes it (0, 1, 2, 3)")
    ap.add_argument("--srm-stages", type=int, default=None, metavar="N",
                    help="getSpikes*: stages per warp as slayer_b200_set_srm_stages takes it (2 .. 8)")
    ap.add_argument("--no-skip-zeros", action="store_true", help="conv/corr: no zero skipping (the dense kernels only)")
    ap.add_argument("--skip-zeros", type=int, default=None, metavar="MODE",
                    help="conv/corr/convPacked: zero skipping as slayer_b200_set_fir_skip_zeros takes it (0 never, 1 probe, 2 always event-driven)")
    ap.add_argument("--spikes", action="store_true", help="conv/corr: the input is a 0/1 spike tensor of the given density")
    args = ap.parse_args(argv)

    sc, lc = slayerpytorch_b200.load_ops()
    if args.packed_fir is not None:
        from slayerpytorch_b200 import capi
        capi.set_fir_packed(args.packed_fir)
    if args.fir_flow is not None:
        from slayerpytorch_b200 import capi
        capi.set_fir_flow(args.fir_flow)
    if args.srm_stages is not None:
        from slayerpytorch_b200 import capi
        capi.set_srm_stages(args.srm_stages)
    if args.no_skip_zeros:
        from slayerpytorch_b200 import capi
        capi.set_fir_skip_zeros(0)
    if args.skip_zeros is not None:
        from slayerpytorch_b200 import capi
        capi.set_fir_skip_zeros(args.skip_zeros)
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(1)
    neurons = min(args.neurons, args.rows)
    batch = max(1, args.rows // neurons)
    shape = (batch, neurons, 1, 1, args.T)
    el = batch * neurons * args.T

    srm = torch.tensor(alpha_kernel(10.0, 1.0, 300), dtype=torch.float32, device=dev)
    ref = torch.tensor(alpha_kernel(1.0, 1.0, 300, mult=-20.0), dtype=torch.float32, device=dev)
    if args.K:
        filt = torch.randn(args.K, device=dev, generator=gen)
    elif args.op == "corr" and args.T > 1000:
        filt = torch.tensor(loihi_psp_kernel({"iDecay": 1024, "vDecay": 128, "wgtExp": 0}), dtype=torch.float32, device=dev)
    else:
        filt = srm
    a = (torch.randn(shape, device=dev, generator=gen).abs() * 1.2
         * (torch.rand(shape, device=dev, generator=gen) < args.density)).float()
    extra = {}
    restore = None
    if args.spikes:
        a = (torch.rand(shape, device=dev, generator=gen) < args.density).float()
    if args.op in ("conv", "corr"):
        fn = (lambda: sc.conv(a, filt, 1.0)) if args.op == "conv" else (lambda: sc.corr(a, filt, 1.0))
        extra["taps"] = int(filt.numel())
    elif args.op == "getSpikes":
        u0 = sc.conv(a, srm, 1.0)
        u = torch.empty_like(u0)
        restore = lambda: u.copy_(u0)
        fn = lambda: sc.getSpikes(u, ref, 10.0, 1.0)
    elif args.op == "getSpikesPacked":
        u0 = sc.conv(a, srm, 1.0)
        u = torch.empty_like(u0)
        restore = lambda: u.copy_(u0)
        fn = lambda: sc.getSpikesPacked(u, ref, 10.0, 1.0)
    elif args.op == "convPacked":
        bits = sc.packSpikes(a)
        fn = lambda: sc.convPacked(bits, args.T, filt, 1.0, 1.0)
        extra["taps"] = int(filt.numel())
    elif args.op == "getSpikesDelayed":
        u0 = sc.conv(a, srm, 1.0)
        u = torch.empty_like(u0)
        restore = lambda: u.copy_(u0)
        dl = torch.rand(neurons, device=dev, generator=gen) * 5
        fn = lambda: sc.getSpikesDelayed(u, ref, 10.0, 1.0, dl)
    elif args.op == "shift":
        d = torch.rand(neurons, device=dev, generator=gen) * 5
        fn = lambda: sc.shift(a, d, 1.0)
    elif args.op == "shiftScalar":
        fn = lambda: sc.shift(a, 1.0, 1.0)
    elif args.op == "spikeGrad":
        g = torch.randn(shape, device=dev, generator=gen)
        fn = lambda: sc.spikeGrad(g, a, 10.0, 10.0, 1.0)
    elif args.op == "corrSpikeGrad":
        g = torch.randn(shape, device=dev, generator=gen)
        fn = lambda: sc.corrSpikeGrad(g, filt, a, 10.0, 10.0, 1.0, 1.0)
        extra["taps"] = int(filt.numel())
    elif args.op == "spikeGradShift":
        g = torch.randn(shape, device=dev, generator=gen)
        d = -(torch.rand(neurons, device=dev, generator=gen) * 5)
        fn = lambda: sc.spikeGradShift(g, a, d, 10.0, 10.0, 1.0, 1.0)
    elif args.op == "delayGrad":
        g = torch.randn(shape, device=dev, generator=gen)
        fn = lambda: sc.delayGrad(g, a, 1.0)
    else:
        w = (torch.randint(-128, 128, shape, device=dev, generator=gen)
             * (torch.rand(shape, device=dev, generator=gen) < 0.05)).float()
        if args.op == "loihi":
            fn = lambda: lc.getSpikes(w, 0, 5120, 1024, 128, 1)
        else:           # spikes written already delayed by one step, current not written
            fn = lambda: lc.getSpikesDelayed(w, 0, 5120, 1024, 128, 1, 1)

    times = []
    out = None
    for it in range(args.warmup + args.iters):
        if restore:
            restore()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        torch.cuda.synchronize()
        if it >= args.warmup:
            times.append(e0.elapsed_time(e1))
    if args.op in ("getSpikes", "getSpikesDelayed"):
        extra["spike_rate"] = float(out.mean())
    if args.op in ("conv", "corr", "convPacked"):
        extra["input_density"] = float((a != 0).float().mean())
    if args.op in ("loihi", "loihiDelayed"):
        extra["spike_rate"] = float(out[0].mean())
    ms = sum(times) / len(times)
    print(json.dumps({"op": args.op, "rows": batch * neurons, "T": args.T, "elements": el,
                      "tensor_GiB": round(el * 4 / 2 ** 30, 3), "avg_ms": round(ms, 4), "min_ms": round(min(times), 4),
                      "GB/s": round(ALG_BYTES[args.op] * el / ms / 1e6, 1),
                      "Gelements/s": round(el / ms / 1e6, 2), **extra}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
