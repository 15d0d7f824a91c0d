"""CPU: host-side logic of the package (kernel construction, module loading)."""
import numpy as np
import pytest

import slayerpytorch_b200


def test_extension_modules_import_and_identify_themselves():
    sc, lc = slayerpytorch_b200.load_ops()
    assert sc.backend == "slayer_b200" and lc.backend == "slayer_b200"
    for name in ("getSpikes", "conv", "corr", "shift", "spikeGrad"):
        assert hasattr(sc, name)
    assert hasattr(lc, "getSpikes")


def test_operators_refuse_cpu_tensors():
    """No CPU fallback: a host tensor is an error, as in the reference (CHECK_INPUT)."""
    import torch
    sc, lc = slayerpytorch_b200.load_ops()
    x = torch.zeros(1, 2, 1, 1, 8)
    with pytest.raises(RuntimeError):
        sc.conv(x, torch.zeros(3), 1.0)
    with pytest.raises(RuntimeError):
        sc.getSpikes(x, torch.zeros(3), 10.0, 1.0)
    with pytest.raises(RuntimeError):
        sc.shift(x, 1.0, 1.0)
    with pytest.raises(RuntimeError):
        lc.getSpikes(x, 0, 80, 1, 1, 1)


def test_mirror_srm_kernels_match_reference_python(golden_dir):
    from slayerpytorch_b200 import layer as L
    g = np.load(golden_dir + "/ref_python.npz")
    nrn = {"type": "SRMALPHA", "theta": 10, "tauSr": 10.0, "tauRef": 1.0, "scaleRef": 2, "tauRho": 1, "scaleRho": 1}
    net = L.spikeLayer(nrn, {"Ts": 1.0, "tSample": 300})
    np.testing.assert_array_equal(net.srmKernel.numpy(), g["srm_Ts1_srmKernel"])
    np.testing.assert_array_equal(net.refKernel.numpy(), g["srm_Ts1_refKernel"])
    net = L.spikeLayer(dict(nrn, tauSr=1.0), {"Ts": 0.1, "tSample": 50}, fullRefKernel=True)
    np.testing.assert_array_equal(net.srmKernel.numpy(), g["srm_kat_srmKernel"])
    np.testing.assert_array_equal(net.refKernel.numpy(), g["srm_kat_refKernel"])


def test_mirror_loihi_layer_kernels_match_reference_python(golden_dir):
    from slayerpytorch_b200 import layer as L
    g = np.load(golden_dir + "/ref_python.npz")
    for tag, nrn in (("loihi_a", {"type": "LOIHI", "vThMant": 80, "vDecay": 128, "iDecay": 1024, "refDelay": 1,
                                  "wgtExp": 0, "tauRho": 1, "scaleRho": 1}),
                     ("loihi_b", {"type": "LOIHI", "vThMant": 40, "vDecay": 256, "iDecay": 2048, "refDelay": 3,
                                  "wgtExp": 1, "tauRho": 1, "scaleRho": 1})):
        net = L.loihiLayer(dict(nrn), {"Ts": 1, "tSample": 1450})
        np.testing.assert_array_equal(net.srmKernel.numpy(), g[tag + "_srmKernel"])
        np.testing.assert_array_equal(net.refKernel.numpy(), g[tag + "_refKernel"])
        assert net.neuron["theta"] == int(g[tag + "_theta"])


def test_host_pipeline_chunk_bounds():
    from slayerpytorch_b200.hoststream import chunk_bounds
    assert chunk_bounds(64, 8) == [(8 * i, 8 * i + 8) for i in range(8)]
    assert chunk_bounds(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert chunk_bounds(3, 8) == [(0, 1), (1, 2), (2, 3)]
    assert chunk_bounds(0, 4) == [(0, 0)]
    assert chunk_bounds(5, 1) == [(0, 5)]
    for batch in range(1, 40):
        for chunks in range(1, 12):
            b = chunk_bounds(batch, chunks)
            assert b[0][0] == 0 and b[-1][1] == batch
            assert all(x[1] == y[0] for x, y in zip(b, b[1:]))
            sizes = [y - x for x, y in b]
            assert min(sizes) >= 1 and max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        chunk_bounds(4, 0)
