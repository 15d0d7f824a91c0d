"""GPU: the new operators against the reference's own CUDA binary, and the reference's own
autograd code running unchanged on the new operator modules.

Needs the optional artefacts of oracle/build_ref.py; skipped where they are absent.
"""
import io
import contextlib

import numpy as np
import pytest
import torch

import slayerpytorch_b200
from tests import refshim

pytestmark = pytest.mark.gpu

REL = 1e-5


@pytest.fixture(scope="module")
def ours():
    return slayerpytorch_b200.load_ops()


@pytest.fixture(scope="module")
def ref_ops():
    a, b = refshim.load_ref_extension("slayerCuda_ref"), refshim.load_ref_extension("slayerLoihiCuda_ref")
    if a is None or b is None:
        pytest.skip("reference CUDA operators not built (oracle/build_ref.py)")
    return a, b


def rnd(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).cuda()


@pytest.mark.parametrize("T,K", [(300, 77), (300, 2), (500, 110), (1450, 110), (64, 160), (2000, 77)])
def test_conv_corr_equal_reference_binary(ours, ref_ops, T, K):
    x = rnd((3, 7, 2, 1, T), T + K) * (rnd((3, 7, 2, 1, T), 1) > 0.5)
    f = rnd((K,), K)
    for Ts in (1.0, 0.1):
        for name in ("conv", "corr"):
            got = getattr(ours[0], name)(x, f, Ts)
            want = getattr(ref_ops[0], name)(x, f, Ts)
            if not torch.equal(got, want):
                torch.testing.assert_close(got, want, rtol=REL, atol=1e-6)
                pytest.fail("%s within tolerance of the reference binary but not bit-exact" % name)


@pytest.mark.parametrize("shape,nus,Ts", [((2, 5, 3, 2, 300), 11, 1.0), ((1, 25, 1, 1, 500), 110, 0.1),
                                          ((2, 3, 1, 1, 2000), 11, 1.0), ((3, 4, 2, 2, 97), 160, 1.0)])
def test_srm_get_spikes_equal_reference_binary(ours, ref_ops, shape, nus, Ts):
    u = rnd(shape, sum(shape), 8.0)
    nu = -rnd((nus,), nus, 5.0).abs()
    ua, ub = u.clone(), u.clone()
    sa = ours[0].getSpikes(ua, nu, 10.0, Ts)
    sb = ref_ops[0].getSpikes(ub, nu, 10.0, Ts)
    assert torch.equal(sa != 0, sb != 0)
    torch.testing.assert_close(sa, sb, rtol=1e-6, atol=0)     # 1/Ts: exact vs fast-math division
    assert torch.equal(ua, ub)
    assert sa.sum() > 0


def test_shift_equal_reference_binary(ours, ref_ops):
    x = rnd((5, 10, 6, 3, 500), 9)
    lut = (torch.rand(10, 6, 3, generator=torch.Generator().manual_seed(1)) * 2 - 1).cuda()
    # Ts = 1: identical division; Ts = 0.1: the reference divides approximately (-use_fast_math),
    # so a delay within an ulp of a bin edge may land one bin off; none does for this seed, and
    # the exact-division result is what the reference's own test expects (test_slayer009.py:57)
    for Ts in (1.0, 0.1):
        a, b = ours[0].shift(x, lut, Ts), ref_ops[0].shift(x, lut, Ts)
        assert torch.equal(a, b)
    for d in (4, -3, 0, 499, 500, 2.7):
        assert torch.equal(ours[0].shift(x, d, 1), ref_ops[0].shift(x, d, 1))
        assert torch.equal(ours[0].shift(x, d), ref_ops[0].shift(x, d))
    one = torch.tensor([3.0]).cuda()
    assert torch.equal(ours[0].shift(x, one, 1.0), ref_ops[0].shift(x, one, 1.0))
    assert torch.equal(ours[0].shift(x, one), ref_ops[0].shift(x, one))
    assert torch.equal(ours[0].shift(x, lut, torch.tensor(1.0).cuda()), ref_ops[0].shift(x, lut, 1.0))
    with pytest.raises(RuntimeError):
        ours[0].shift(x, lut[:5], 1.0)


@pytest.mark.parametrize("params", [(0, 5120, 1024, 128, 1), (0, 5120, 1024, 128, 7), (1, 2560, 2048, 256, 3)])
def test_loihi_equal_reference_binary(ours, ref_ops, params):
    g = torch.Generator().manual_seed(sum(params))
    w = (torch.randint(-60, 60, (2, 6, 4, 4, 1450), generator=g) * (torch.rand(2, 6, 4, 4, 1450, generator=g) < 0.3)).float().cuda()
    got = ours[1].getSpikes(w, *params)
    want = ref_ops[1].getSpikes(w, *params)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    assert got[0].sum() > 0


# ------------------------------------------- the reference's Python on the new operators
@pytest.fixture(scope="module")
def ref_py_on_ours(ours):
    with contextlib.redirect_stdout(io.StringIO()):
        m = refshim.load_reference_python(ours[0], ours[1], "slayerSNN_on_b200")
    if m is None:
        pytest.skip("reference Python package not installed (oracle/build_ref.py)")
    return m


def test_reference_modules_are_bound_to_the_new_operators(ref_py_on_ours, ours):
    assert ref_py_on_ours.slayer.slayerCuda is ours[0]
    assert ref_py_on_ours.loihi.slayerLoihiCuda is ours[1]
    assert ours[0].backend == "slayer_b200"


def srm_net(slayer_mod, params, dev):
    neuron, sim = dict(params["neuron"]), dict(params["simulation"])
    L = slayer_mod.spikeLayer(neuron, sim).to(dev)
    return L


PARAMS = {"neuron": {"type": "SRMALPHA", "theta": 10, "tauSr": 10.0, "tauRef": 1.0, "scaleRef": 2,
                     "tauRho": 1, "scaleRho": 1},
          "simulation": {"Ts": 1.0, "tSample": 300}}


def test_reference_autograd_chain_runs_unchanged_and_matches_mirror(ref_py_on_ours):
    """_pspFunction, _spikeFunction, _delayLayer/_delayFunction, delayShift of the reference
    (src/slayer.py) on the new operators vs this package's mirror layer: same forward bits,
    gradients within 1e-5 (the mirror fuses the surrogate gradient)."""
    from slayerpytorch_b200 import layer as mirror
    dev = torch.device("cuda")
    R = srm_net(ref_py_on_ours.slayer, PARAMS, dev)
    M = mirror.spikeLayer(dict(PARAMS["neuron"]), dict(PARAMS["simulation"])).to(dev)
    assert torch.equal(R.srmKernel, M.srmKernel) and torch.equal(R.refKernel, M.refKernel)
    g = torch.Generator().manual_seed(3)
    a = (torch.randn(4, 32, 1, 1, 300, generator=g).abs() * 2 * (torch.rand(4, 32, 1, 1, 300, generator=g) < 0.3)).cuda()
    gout = torch.randn(4, 32, 1, 1, 300, generator=g).cuda()
    dR, dM = R.delay(32).to(dev), M.delay(32).to(dev)
    with torch.no_grad():
        dR.delay.copy_(torch.rand(32, 1, 1, generator=g) * 5)
        dM.delay.copy_(dR.delay)
    outs = []
    for net, dl in ((R, dR), (M, dM)):
        x = a.clone().requires_grad_(True)
        y = net.delayShift(dl(net.spike(net.psp(x))), 1)
        y.backward(gout)
        outs.append((y.detach(), x.grad, dl.delay.grad))
    assert torch.equal(outs[0][0], outs[1][0])
    assert outs[0][0].sum() > 0
    torch.testing.assert_close(outs[0][1], outs[1][1], rtol=REL, atol=1e-6)
    torch.testing.assert_close(outs[0][2], outs[1][2], rtol=1e-4, atol=1e-4)


def test_reference_gradient_kat_on_the_new_operators(ref_py_on_ours, golden_dir):
    """test/test_slayer003.py replayed with the reference's own slayer.py + spikeLoss.py running
    on the new operators: weight gradients vs the MATLAB values, ||delta|| / size < 1e-4."""
    srm = np.load(golden_dir + "/srm_kat.npz")
    dev = torch.device("cuda")
    params = {"neuron": {"type": "SRMALPHA", "theta": 10, "tauSr": 1.0, "tauRef": 1.0, "scaleRef": 2,
                         "tauRho": 0.1, "scaleRho": 1},
              "simulation": {"Ts": 0.1, "tSample": 50, "nSample": 1},
              "training": {"error": {"type": "SpikeTime"}}}
    S = ref_py_on_ours.slayer
    L = S.spikeLayer(params["neuron"], params["simulation"], fullRefKernel=True).to(dev)
    fc1, fc2 = L.dense(250, 25).to(dev), L.dense(25, 1).to(dev)
    fc1.weight = torch.nn.Parameter(torch.from_numpy(srm["w1Initial"]).reshape(25, 250, 1, 1, 1).to(dev))
    fc2.weight = torch.nn.Parameter(torch.from_numpy(srm["w2Initial"]).reshape(1, 25, 1, 1, 1).to(dev))

    def events(idx, n):
        x = np.zeros((n, 500), np.float32)
        for nid, tid in idx:
            if tid < 500:
                x[nid, tid] = 10.0
        return torch.from_numpy(x).reshape(1, n, 1, 1, 500).to(dev)

    out = L.spike(L.psp(fc2(L.spike(L.psp(fc1(events(srm["spikeIn"], 250)))))))
    error = ref_py_on_ours.loss.spikeLoss(params).to(dev)
    loss = error.spikeTime(out, events(srm["spikeOut"], 1))
    loss.backward()
    g1 = fc1.weight.grad.reshape(25, 250).cpu().numpy()
    g2 = fc2.weight.grad.reshape(1, 25).cpu().numpy()
    assert np.linalg.norm(srm["gradW2Initial"] - g2) / g2.size < 1e-4
    assert np.linalg.norm(srm["gradW1Initial"] - g1) / g1.size < 1e-4


def test_reference_loihi_layer_on_the_new_operators(ref_py_on_ours, golden_dir):
    """test/test_slayerLoihi001.py replayed with the reference's slayerLoihi.py on the new
    operators: chip-recorded spikes and voltages; plus spikeLoihi backward runs."""
    kat = np.load(golden_dir + "/loihi_kat.npz")
    dev = torch.device("cuda")
    neuron = {"type": "LOIHI", "vThMant": 80, "vDecay": 128, "iDecay": 1024, "refDelay": 1, "wgtExp": 0,
              "tauRho": 1, "scaleRho": 1}
    sim = {"Ts": 0.1, "tSample": 50}
    with contextlib.redirect_stdout(io.StringIO()):
        L = ref_py_on_ours.loihi.spikeLayer(neuron, sim).to(dev)
    x = np.zeros((250, 500), np.float32)
    for nid, tid in kat["spikeIn"]:
        if 0 <= tid < 500:
            x[nid, tid] = 10.0
    w1 = torch.from_numpy((np.round(kat["w1learned"] * 2) * 2).astype(np.float32)).to(dev)
    w2 = torch.from_numpy((np.round(kat["w2learned"] * 2) * 2).astype(np.float32)).to(dev)
    xin = torch.from_numpy(x).to(dev)
    a1 = (w1 @ xin).reshape(1, 25, 1, 1, 500)
    s1, v1 = L.spikeLoihiFull(a1)[0:2]
    s1 = L.delayShift(s1, 1)
    a2 = (w2 @ s1.reshape(25, 500)).reshape(1, 1, 1, 1, 500)
    s2, v2 = L.spikeLoihiFull(a2)[0:2]
    s2 = L.delayShift(s2, 1)
    hid = np.zeros((25, 500), bool)
    for nid, tid in kat["hiddenSpikes"]:
        hid[nid, tid] = True
    outp = np.zeros((1, 500), bool)
    for nid, tid in kat["outputSpikes"]:
        outp[nid, tid] = True
    assert np.array_equal(s1.reshape(25, 500).cpu().numpy() > 0, hid)
    assert np.array_equal(s2.reshape(1, 500).cpu().numpy() > 0, outp)
    assert np.abs(v1[0, 24, 0, 0, :-1].cpu().numpy() - kat["hiddenVoltage24"]).max() < 1e-3
    assert np.abs(v2.reshape(-1)[:-1].cpu().numpy() - kat["outputVoltage"]).max() < 1e-3
    a = a1.clone().requires_grad_(True)
    y = L.spikeLoihi(a)
    y.backward(torch.ones_like(y))
    assert torch.isfinite(a.grad).all() and a.grad.abs().sum() > 0


@pytest.mark.parametrize("Ts,region", [(1.0, (0, 300)), (1.0, (50, 250)), (0.5, (10, 120))])
def test_device_resident_losses_equal_the_reference_losses(ref_py_on_ours, Ts, region):
    """slayerpytorch_b200.loss (no host round trip) against the reference's spikeLoss.py and
    spikeClassifier: loss values and the gradients that reach the spikes."""
    from slayerpytorch_b200 import loss as ours_loss
    dev = torch.device("cuda")
    T = int(round(300 / Ts)) if Ts == 1.0 else 300
    params = {"neuron": {"type": "SRMALPHA", "theta": 10, "tauSr": 10.0, "tauRef": 1.0, "scaleRef": 2,
                         "tauRho": 1, "scaleRho": 1},
              "simulation": {"Ts": Ts, "tSample": int(T * Ts), "nSample": 12},
              "training": {"error": {"type": "NumSpikes", "tgtSpikeRegion": {"start": region[0], "stop": region[1]},
                                     "tgtSpikeCount": {True: 60, False: 10}}}}
    g = torch.Generator().manual_seed(int(Ts * 10) + region[0])
    spikes = ((torch.rand(6, 10, 1, 1, T, generator=g) < 0.08).float() / Ts).to(dev)
    label = torch.randint(0, 10, (6,), generator=g)
    desired = torch.zeros(6, 10, 1, 1, 1)
    desired[torch.arange(6), label] = 1

    ref = ref_py_on_ours.loss.spikeLoss(params).to(dev)
    mine = ours_loss.spikeLoss(params).to(dev)
    for scale in (1, 0.5):
        a = spikes.clone().requires_grad_(True)
        la = ref.numSpikes(a, desired, scale)
        la.backward()
        b = spikes.clone().requires_grad_(True)
        lb = mine.numSpikes(b, desired.to(dev), scale)
        lb.backward()
        assert la.item() > 0
        torch.testing.assert_close(lb, la, rtol=1e-6, atol=0)
        torch.testing.assert_close(b.grad, a.grad, rtol=1e-5, atol=1e-7)
        # a CPU one-hot works too (the reference only takes that form)
        torch.testing.assert_close(mine.numSpikes(spikes, desired, scale), la, rtol=1e-6, atol=0)

    params["training"]["error"] = {"type": "SpikeTime"}
    ref, mine = ref_py_on_ours.loss.spikeLoss(params).to(dev), ours_loss.spikeLoss(params).to(dev)
    target = ((torch.rand(6, 10, 1, 1, T, generator=g) < 0.05).float() / Ts).to(dev)
    a = spikes.clone().requires_grad_(True)
    la = ref.spikeTime(a, target)
    la.backward()
    b = spikes.clone().requires_grad_(True)
    lb = mine.spikeTime(b, target)
    lb.backward()
    torch.testing.assert_close(lb, la, rtol=1e-6, atol=0)
    torch.testing.assert_close(b.grad, a.grad, rtol=1e-5, atol=1e-7)

    import importlib
    ref_cls = importlib.import_module(ref_py_on_ours.loss.__name__.rsplit(".", 1)[0] + ".spikeClassifier").spikeClassifier
    got = ours_loss.spikeClassifier.getClass(spikes)
    want = ref_cls.getClass(spikes)
    assert not got.is_cuda and torch.equal(got, want)
    # the accuracy line of the reference's training scripts (example/02_NMNIST_MLP/nmnistMLP.py:120)
    assert int(torch.sum(got == label)) == int(torch.sum(want == label))
    on_dev = ours_loss.spikeClassifier.getClass(spikes, host=False)
    assert on_dev.is_cuda and torch.equal(on_dev.cpu(), want)


def test_long_sequence_delay_network_through_the_reference_delay_layer(ours, ref_ops):
    """The long-sequence network 200-256-200 (T = 2000, Ts = 1, learnable delays U(0, 10) ms
    after both layers, one input spike per neuron at a random time, spikeTime loss against 2 %
    target trains; topology of example/01_Oxford/oxfordTrain.py:33-49) run twice through the
    reference's UNCHANGED slayer.py / spikeLoss.py - _pspFunction, _spikeFunction, _delayLayer
    and _delayFunction (src/slayer.py:817-957) - once bound to the new operators and once bound
    to the reference's own CUDA binary.  Spikes must be identical, every gradient within 1e-5."""
    with contextlib.redirect_stdout(io.StringIO()):
        on_new = refshim.load_reference_python(ours[0], ours[1], "slayerSNN_cfg4_new")
        on_ref = refshim.load_reference_python(ref_ops[0], ref_ops[1], "slayerSNN_cfg4_ref")
    if on_new is None or on_ref is None:
        pytest.skip("reference Python package not installed (oracle/build_ref.py)")
    assert on_new.slayer.slayerCuda is ours[0] and on_ref.slayer.slayerCuda is ref_ops[0]
    dev = torch.device("cuda")
    params = {"neuron": {"type": "SRMALPHA", "theta": 10, "tauSr": 1.0, "tauRef": 1.0, "scaleRef": 2,
                         "tauRho": 1, "scaleRho": 1},
              "simulation": {"Ts": 1.0, "tSample": 2000, "nSample": 1},
              "training": {"error": {"type": "SpikeTime"}}}
    N, T = 8, 2000
    g = torch.Generator().manual_seed(1004)
    x = torch.zeros(N, 200, 1, 1, T)
    when = torch.randint(0, 1000, (N, 200), generator=g)
    x.view(N, 200, T).scatter_(2, when.unsqueeze(-1), 1.0)
    target = (torch.rand(N, 200, 1, 1, T, generator=g) < 0.02).float()
    w1 = torch.randn(256, 200, 1, 1, 1, generator=g) * 4
    w2 = torch.randn(200, 256, 1, 1, 1, generator=g) * 1.5
    d1 = torch.rand(256, 1, 1, generator=g) * 10
    d2 = torch.rand(200, 1, 1, generator=g) * 10

    results = []
    for mods in (on_new, on_ref):
        S = mods.slayer
        L = S.spikeLayer(dict(params["neuron"]), dict(params["simulation"])).to(dev)
        fc1, fc2 = L.dense(200, 256).to(dev), L.dense(256, 200).to(dev)
        dl1, dl2 = L.delay(256).to(dev), L.delay(200).to(dev)
        with torch.no_grad():
            fc1.weight.copy_(w1)
            fc2.weight.copy_(w2)
            dl1.delay.copy_(d1)
            dl2.delay.copy_(d2)
        h = dl1(L.spike(L.psp(fc1(x.to(dev)))))
        out = dl2(L.spike(L.psp(fc2(h))))
        loss = mods.loss.spikeLoss(params).to(dev).spikeTime(out, target.to(dev))
        loss.backward()
        results.append(dict(h=h.detach(), out=out.detach(), loss=loss.detach(),
                            gw1=fc1.weight.grad, gw2=fc2.weight.grad, gd1=dl1.delay.grad, gd2=dl2.delay.grad))
    new, ref = results
    assert torch.equal(new["h"], ref["h"]) and torch.equal(new["out"], ref["out"])
    assert 0.001 < new["h"].mean() < 0.5 and new["out"].sum() > 0
    for k in ("loss", "gw1", "gw2", "gd1", "gd2"):
        scale = ref[k].abs().max().item()
        assert scale > 0, k
        torch.testing.assert_close(new[k], ref[k], rtol=REL, atol=REL * scale, msg=lambda m, k=k: k + ": " + m)
