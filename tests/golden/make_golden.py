"""Generate the golden fixtures in this directory from a reference checkout.

Run once, where the reference is available:

    python tests/golden/make_golden.py <path-to-reference-checkout>

It writes four small ``.npz`` files next to itself:

``srm_kat.npz``
    The reference's MATLAB-derived known-answer data for the 250-25-1 SRM network
    (test/test_files/snnData/*, used by test/test_slayer002.py, test_slayer003.py and
    test_slayer004.py): input spike events, initial and learned weights, desired output
    spikes, the expected weight gradients, the membrane-potential / spike trace of one hidden
    and the output neuron, and the tabulated response kernels.
``loihi_kat.npz``
    The Loihi-chip recordings of the same network (test/test_files/Loihi/*, used by
    test/test_slayerLoihi001.py): input events, learned weights, recorded hidden and output
    spikes and voltages.
``ref_python.npz``
    Outputs of the reference's own Python code run here on the CPU with seeded inputs:
    the alpha / Loihi response kernels built by ``spikeLayer`` (src/slayer.py:114-123,
    src/slayerLoihi.py:66-89), the pure-PyTorch psp layer (src/slayer.py:760-791) and the
    NumPy Loihi neuron model ``Neuron.run`` (test/test_slayerLoihi002.py:30-82, extracted
    from the test file by name so that nothing else in that file is executed).

``events_ref.npz``
    Seeded synthetic address events and the spike tensors the reference's own
    ``event.toSpikeTensor`` (src/spikeFileIO.py:66-144; the class is extracted from the file by
    name, because the module imports matplotlib) makes of them: one- and two-dimensional
    events, events outside the tensor, both binning modes, sampling times 1 and 0.5 ms.

Only data is stored; no reference source code is copied.
"""
import ast
import importlib
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference_modules(root):
    """Import src/slayer.py and src/slayerLoihi.py as ``slayerSNN.*`` without running the
    package ``__init__`` (which needs matplotlib / an old NumPy) and without CUDA operators
    (stub modules stand in; nothing here calls them)."""
    for name in ("slayerCuda", "slayerLoihiCuda"):
        sys.modules.setdefault(name, types.ModuleType(name))
    pkg = types.ModuleType("slayerSNN")
    pkg.__path__ = [os.path.join(root, "src")]
    sys.modules["slayerSNN"] = pkg
    slayer = importlib.import_module("slayerSNN.slayer")
    loihi = importlib.import_module("slayerSNN.slayerLoihi")
    return slayer, loihi


def aer_to_index(path, Ts, id_offset, time_first=True, t_offset=0):
    """Event list -> integer (neuron, time-bin) pairs, as the reference tests bin them."""
    ev = np.loadtxt(path).reshape(-1, 2)
    if time_first:
        t = np.rint(ev[:, 0] / Ts + t_offset).astype(np.int64)
        n = np.rint(ev[:, 1] + id_offset).astype(np.int64)
    else:
        n = np.rint(ev[:, 0]).astype(np.int64)
        t = np.rint(ev[:, 1]).astype(np.int64)
    return np.stack([n, t], axis=1)


def srm_kat(root):
    d = os.path.join(root, "test", "test_files", "snnData")
    Ts = 0.1
    out = dict(
        Ts=np.float32(Ts), Ns=np.int64(500), theta=np.float32(10),
        tauSr=np.float32(1), tauRef=np.float32(1), scaleRef=np.float32(2),
        spikeIn=aer_to_index(os.path.join(d, "spikeIn.txt"), Ts, -1),
        spikeHid=aer_to_index(os.path.join(d, "spikeHid.txt"), Ts, -1),
        spikeOut=aer_to_index(os.path.join(d, "spikeOut.txt"), Ts, -1),
        w1Initial=np.loadtxt(os.path.join(d, "w1Initial.txt")).astype(np.float32),
        w2Initial=np.loadtxt(os.path.join(d, "w2Initial.txt")).astype(np.float32).reshape(1, -1),
        w1learned=np.loadtxt(os.path.join(d, "w1learned.txt")).astype(np.float32),
        w2learned=np.loadtxt(os.path.join(d, "w2learned.txt")).astype(np.float32).reshape(1, -1),
        gradW1Initial=np.loadtxt(os.path.join(d, "gradW1Initial.txt")).astype(np.float64),
        gradW2Initial=np.loadtxt(os.path.join(d, "gradW2Initial.txt")).astype(np.float64).reshape(1, -1),
        spikeFuncHid=np.loadtxt(os.path.join(d, "spikeFuncHid.txt")).astype(np.float64),
        spikeFuncOut=np.loadtxt(os.path.join(d, "spikeFuncOut.txt")).astype(np.float64),
        h_sr=np.loadtxt(os.path.join(d, "h_sr.txt")).astype(np.float64),
        h_ref=np.loadtxt(os.path.join(d, "h_ref.txt")).astype(np.float64),
    )
    np.savez_compressed(os.path.join(HERE, "srm_kat.npz"), **out)
    return out


def loihi_kat(root):
    d = os.path.join(root, "test", "test_files", "Loihi")
    Ts = 0.1
    out = dict(
        Ts=np.float32(Ts), Ns=np.int64(500),
        vThMant=np.int64(80), vDecay=np.int64(128), iDecay=np.int64(1024),
        refDelay=np.int64(1), wgtExp=np.int64(0),
        # test_slayerLoihi001.py:42-46 delays the input events by 49 bins
        spikeIn=aer_to_index(os.path.join(d, "snnData", "spikeIn.txt"), Ts, -1, t_offset=49),
        w1learned=np.loadtxt(os.path.join(d, "snnData", "w1learned.txt")).astype(np.float64),
        w2learned=np.loadtxt(os.path.join(d, "snnData", "w2learned.txt")).astype(np.float64).reshape(1, -1),
        hiddenSpikes=aer_to_index(os.path.join(d, "LoihiData", "loihiHiddenSpikes.txt"), Ts, 0, time_first=False),
        outputSpikes=aer_to_index(os.path.join(d, "LoihiData", "loihiOutputSpikes.txt"), Ts, 0, time_first=False),
        hiddenVoltage24=np.loadtxt(os.path.join(d, "LoihiData", "loihiHiddenVoltage24.txt")).astype(np.float64),
        outputVoltage=np.loadtxt(os.path.join(d, "LoihiData", "loihiOutputVoltage.txt")).astype(np.float64),
    )
    np.savez_compressed(os.path.join(HERE, "loihi_kat.npz"), **out)
    return out


def extract_class(path, name):
    """Compile one top-level class of a Python file without executing the rest of it."""
    with open(path) as f:
        tree = ast.parse(f.read())
    node = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == name)
    ns = {"np": np}
    exec(compile(ast.Module(body=[node], type_ignores=[]), path, "exec"), ns)
    return ns[name]


def ref_python(root):
    import torch
    slayer, loihi = load_reference_modules(root)
    out = {}

    # response kernels of the SRM configurations used by the benchmark configs and the KAT
    sim1 = {"Ts": 1.0, "tSample": 300}
    nrn1 = {"type": "SRMALPHA", "theta": 10, "tauSr": 10.0, "tauRef": 1.0, "scaleRef": 2,
            "tauRho": 1, "scaleRho": 1}
    L = slayer.spikeLayer(nrn1, sim1)
    out["srm_Ts1_srmKernel"] = L.srmKernel.numpy()
    out["srm_Ts1_refKernel"] = L.refKernel.numpy()
    sim2 = {"Ts": 0.1, "tSample": 50}
    nrn2 = dict(nrn1, tauSr=1.0)
    L2 = slayer.spikeLayer(nrn2, sim2, fullRefKernel=True)
    out["srm_kat_srmKernel"] = L2.srmKernel.numpy()
    out["srm_kat_refKernel"] = L2.refKernel.numpy()
    L3 = slayer.spikeLayer(nrn2, sim2)
    out["srm_kat_refKernel_short"] = L3.refKernel.numpy()

    # Loihi response kernels (config-5 parameters and a second set)
    for tag, nrn in (("loihi_a", {"type": "LOIHI", "vThMant": 80, "vDecay": 128, "iDecay": 1024,
                                  "refDelay": 1, "wgtExp": 0, "tauRho": 1, "scaleRho": 1}),
                     ("loihi_b", {"type": "LOIHI", "vThMant": 40, "vDecay": 256, "iDecay": 2048,
                                  "refDelay": 3, "wgtExp": 1, "tauRho": 1, "scaleRho": 1})):
        LL = loihi.spikeLayer(dict(nrn), {"Ts": 1, "tSample": 1450})
        out[tag + "_srmKernel"] = LL.srmKernel.numpy().astype(np.float32)
        out[tag + "_refKernel"] = LL.refKernel.numpy().astype(np.float32)
        out[tag + "_theta"] = np.int64(LL.neuron["theta"])

    # the reference's pure-PyTorch psp layer against which its CUDA conv is pinned
    # (test/test_slayer011.py:35-43), run on the CPU
    g = torch.Generator().manual_seed(1234)
    for tag, layer, Ts, shape in (("psp_Ts1", L, 1.0, (2, 3, 2, 1, 150)),
                                  ("psp_kat", L2, 0.1, (2, 5, 1, 1, 500))):
        x = (torch.rand(shape, generator=g) > 0.8).float() / Ts
        with torch.no_grad():
            y = slayer._pspLayer(layer.srmKernel, Ts)(x)
        out[tag + "_in"] = x.numpy()
        out[tag + "_out"] = y.numpy()
        out[tag + "_Ts"] = np.float32(Ts)

    # the NumPy Loihi neuron model of test/test_slayerLoihi002.py on that test's input recipe
    Neuron = extract_class(os.path.join(root, "test", "test_slayerLoihi002.py"), "Neuron")
    rng = np.random.RandomState(4321)
    for k, (refDelay, wgtExp, vThMant, vDecay, iDecay) in enumerate(
            [(1, 0, 80, 128, 1024), (2, 0, 80, 128, 1024), (5, 0, 80, 128, 1024),
             (17, 0, 80, 128, 1024), (3, 1, 40, 256, 2048), (1, 0, 5, 0, 4095)]):
        weight = np.round((rng.random_sample((64, 128)) - 0.5) * 10) * 2
        spikes = rng.random_sample((128, 200)) > 0.8
        wS = weight.dot(spikes)
        s, c, v = Neuron(vThMant, vDecay, iDecay, refDelay, wgtExp).run(wS)
        out["nrn%d_params" % k] = np.array([wgtExp, vThMant * 64, iDecay, vDecay, refDelay], np.int64)
        out["nrn%d_w" % k] = wS.astype(np.float32)
        out["nrn%d_spike" % k] = s.astype(np.int32)
        out["nrn%d_current" % k] = c.astype(np.int32)
        out["nrn%d_voltage" % k] = v.astype(np.int32)
    out["nrn_count"] = np.int64(6)

    np.savez_compressed(os.path.join(HERE, "ref_python.npz"), **out)
    return out


def events_ref(root):
    event = extract_class(os.path.join(root, "src", "spikeFileIO.py"), "event")
    rng = np.random.RandomState(77)
    out = {}
    cases = [("2d_or", 2, (2, 9, 11, 40), 1.0, "OR"), ("2d_sum", 2, (2, 9, 11, 40), 1.0, "SUM"),
             ("2d_half", 2, (3, 6, 5, 64), 0.5, "OR"), ("1d_or", 1, (4, 1, 20, 33), 1.0, "OR"),
             ("1d_sum_half", 1, (2, 1, 7, 50), 0.5, "SUM")]
    for tag, dim, shape, Ts, mode in cases:
        C, H, W, T = shape
        n = 400
        # some events fall outside the tensor in every coordinate; many share a bin
        x = rng.randint(-1, W + 2, n)
        y = rng.randint(-1, H + 2, n) if dim == 2 else None
        p = rng.randint(0, C + 1, n)
        p[0] = 0                                       # the class subtracts min(p): keep it 0
        t = rng.rand(n) * (T + 4) * Ts - Ts
        t[:8] = (np.arange(8) + 0.5) * Ts              # exact half bins: rounding to even
        start = (rng.rand(*shape) < 0.1).astype(np.float32) * 3.0 if mode == "SUM" else np.zeros(shape, np.float32)
        got = event(x.copy(), None if y is None else y.copy(), p.copy(), t.copy()).toSpikeTensor(
            start.copy(), samplingTime=Ts, randomShift=False, binningMode=mode)
        out[tag + "_x"], out[tag + "_p"], out[tag + "_t"] = x.astype(np.int32), p.astype(np.int32), t
        if y is not None:
            out[tag + "_y"] = y.astype(np.int32)
        out[tag + "_start"], out[tag + "_out"] = start, np.asarray(got, np.float32)
        out[tag + "_Ts"] = np.float64(Ts)
    out["cases"] = np.array([c[0] + ":" + c[4] for c in cases])
    np.savez_compressed(os.path.join(HERE, "events_ref.npz"), **out)
    return out


def main(argv):
    if len(argv) < 2:
        print(__doc__)
        return 2
    root = argv[1]
    a = srm_kat(root)
    b = loihi_kat(root)
    c = ref_python(root)
    d = events_ref(root)
    for name, d in (("srm_kat", a), ("loihi_kat", b), ("ref_python", c), ("events_ref", d)):
        size = os.path.getsize(os.path.join(HERE, name + ".npz"))
        print("%s.npz: %d arrays, %d bytes" % (name, len(d), size))
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
