"""Pin the CPU oracle against the reference's golden data (no GPU needed).

Fixtures come from tests/golden/make_golden.py.  Each test names the reference test it
replays.
"""
import os

import numpy as np
import pytest

from oracle import cpu_oracle as co
from oracle import numpy_loops as nl

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def srm():
    return dict(np.load(os.path.join(GOLDEN, "srm_kat.npz")))


@pytest.fixture(scope="module")
def loihi():
    return dict(np.load(os.path.join(GOLDEN, "loihi_kat.npz")))


@pytest.fixture(scope="module")
def refpy():
    return dict(np.load(os.path.join(GOLDEN, "ref_python.npz")))


def alpha_kernel(tau, Ts, tSample, mult=1.0, eps=0.01):
    """Alpha response kernel, truncated where it falls below eps after its peak
    (restates spikeLayer._calculateAlphaKernel, src/slayer.py:114-123)."""
    out = []
    for t in np.arange(0, tSample, Ts):
        v = mult * t / tau * np.exp(1 - t / tau)
        if abs(v) < eps and t > tau:
            break
        out.append(v)
    return np.asarray(out, np.float32)


def dense_events(idx, n, T, value):
    x = np.zeros((n, T), np.float32)
    for nid, tid in idx:
        if 0 <= tid < T:
            x[nid, tid] = value
    return x


def test_alpha_kernels_match_reference_python(refpy, srm):
    np.testing.assert_array_equal(alpha_kernel(10.0, 1.0, 300), refpy["srm_Ts1_srmKernel"])
    np.testing.assert_array_equal(alpha_kernel(1.0, 1.0, 300, mult=-20.0), refpy["srm_Ts1_refKernel"])
    assert refpy["srm_Ts1_srmKernel"].size == 77 and refpy["srm_Ts1_refKernel"].size == 11
    k = alpha_kernel(1.0, 0.1, 50)
    np.testing.assert_array_equal(k, refpy["srm_kat_srmKernel"])
    kr = alpha_kernel(1.0, 0.1, 50, mult=-20.0, eps=0.0001)
    np.testing.assert_array_equal(kr, refpy["srm_kat_refKernel"])
    # the MATLAB tables hold the same kernels to 4 decimals
    n = min(k.size, srm["h_sr"].shape[0])
    np.testing.assert_allclose(k[:n], srm["h_sr"][:n, 1], atol=6e-5)
    n = min(kr.size, srm["h_ref"].shape[0])
    np.testing.assert_allclose(kr[:n], srm["h_ref"][:n, 1], atol=6e-4)


def test_conv_matches_reference_psp_layer(refpy):
    """test/test_slayer011.py: CUDA conv == pure-PyTorch psp layer, norm/numel < 1e-6."""
    for tag, kern in (("psp_Ts1", "srm_Ts1_srmKernel"), ("psp_kat", "srm_kat_srmKernel")):
        x, y, Ts = refpy[tag + "_in"], refpy[tag + "_out"], float(refpy[tag + "_Ts"])
        got = co.conv(x, refpy[kern], Ts)
        assert np.linalg.norm(got - y) / y.size < 1e-6
        np.testing.assert_allclose(got, y, rtol=2e-5, atol=1e-5)
        np.testing.assert_allclose(nl.conv(x, refpy[kern], Ts), got, rtol=2e-5, atol=1e-5)


def test_conv_corr_are_adjoint():
    rng = np.random.RandomState(0)
    x = rng.randn(7, 93).astype(np.float32)
    g = rng.randn(7, 93).astype(np.float32)
    f = rng.randn(20).astype(np.float32)
    lhs = np.sum(co.conv(x, f, 0.5).astype(np.float64) * g)
    rhs = np.sum(x * co.corr(g, f, 0.5).astype(np.float64))
    assert abs(lhs - rhs) < 1e-3 * max(1.0, abs(lhs))
    np.testing.assert_allclose(nl.corr(g, f, 0.5), co.corr(g, f, 0.5), rtol=1e-4, atol=1e-5)


def test_srm_spike_trace_of_hidden_and_output_neuron(srm, refpy):
    """test/test_slayer002.py:153-167 recipe on the MATLAB trace: column 0 is u before the
    refractory response, column 1 after it, column 2 the spike train."""
    nu = refpy["srm_kat_refKernel"]
    for key in ("spikeFuncHid", "spikeFuncOut"):
        data = srm[key][:500]
        s, u = co.srm_get_spikes(data[:, 0].reshape(1, 1, 1, 1, -1), nu, 10.0, 0.1)
        s, u = s.ravel(), u.ravel()
        np.testing.assert_array_equal(s > 0, data[:, 2] > 0)
        np.testing.assert_allclose(u, data[:, 1], atol=2e-3)
        s2, u2 = nl.srm_get_spikes(data[:, 0].reshape(1, -1), nu, 10.0, 0.1)
        np.testing.assert_array_equal(s2.ravel(), s)
        np.testing.assert_array_equal(u2.ravel(), u)


def srm_forward(x, w1, w2, k_srm, k_ref, Ts, order):
    """250-25-1 network forward on the oracle ops.  order 'psp_first' is test_slayer002/004,
    'fc_first' is test_slayer003."""
    if order == "psp_first":
        u1 = w1 @ co.conv(x, k_srm, Ts)
    else:
        u1 = co.conv(w1 @ x, k_srm, Ts)
    s1, u1p = co.srm_get_spikes(u1.reshape(1, -1, 1, 1, x.shape[-1]), k_ref, 10.0, Ts)
    s1, u1p = s1.reshape(u1.shape), u1p.reshape(u1.shape)
    if order == "psp_first":
        u2 = w2 @ co.conv(s1, k_srm, Ts)
    else:
        u2 = co.conv(w2 @ s1, k_srm, Ts)
    s2, u2p = co.srm_get_spikes(u2.reshape(1, -1, 1, 1, x.shape[-1]), k_ref, 10.0, Ts)
    return s1, u1p, s2.reshape(u2.shape), u2p.reshape(u2.shape)


def test_srm_network_spikes_match_matlab(srm, refpy):
    """test/test_slayer002.py: learned weights; MATLAB spike lists for hidden/output layer."""
    T, Ts = 500, 0.1
    x = dense_events(srm["spikeIn"], 250, T, 1 / Ts)
    s1, _, s2, _ = srm_forward(x, srm["w1learned"], srm["w2learned"],
                               refpy["srm_kat_srmKernel"], refpy["srm_kat_refKernel"], Ts, "psp_first")
    hid = dense_events(srm["spikeHid"], 25, T, 1 / Ts)
    out = dense_events(srm["spikeOut"], 1, T, 1 / Ts)
    np.testing.assert_array_equal(s1 > 0, hid > 0)
    np.testing.assert_array_equal(s2 > 0, out > 0)


def test_srm_class_of_initial_network(srm, refpy):
    """test/test_slayer004.py:70-72: the 250->25 layer's most active neuron is 21."""
    T, Ts = 500, 0.1
    x = dense_events(srm["spikeIn"], 250, T, 1 / Ts)
    u1 = srm["w1Initial"] @ co.conv(x, refpy["srm_kat_srmKernel"], Ts)
    s1, _ = co.srm_get_spikes(u1.reshape(1, 25, 1, 1, T), refpy["srm_kat_refKernel"], 10.0, Ts)
    assert int(np.argmax(s1.reshape(25, T).sum(-1))) == 21


def test_srm_weight_gradients_match_matlab(srm, refpy):
    """test/test_slayer003.py:89-101: conv -> getSpikes -> corr -> surrogate end to end,
    tauRho = 0.1, full refractory kernel; ||delta|| / size < 1e-4 for both layers."""
    T, Ts, theta = 500, 0.1, 10.0
    tau, scale = 0.1 * theta, 1.0
    k, kr = refpy["srm_kat_srmKernel"], refpy["srm_kat_refKernel"]
    w1, w2 = srm["w1Initial"], srm["w2Initial"]
    x = dense_events(srm["spikeIn"], 250, T, 1 / Ts)
    des = dense_events(srm["spikeOut"], 1, T, 1 / Ts)
    s1, u1p, s2, u2p = srm_forward(x, w1, w2, k, kr, Ts, "fc_first")
    # loss = 1/2 * sum(psp(out - des)^2) * Ts   (src/spikeLoss.py:57-58)
    e = co.conv(s2 - des, k, Ts)
    d_s2 = co.corr(e * np.float32(Ts), k, Ts)
    d_a2 = co.corr(co.spike_grad(d_s2, u2p, theta, tau, scale), k, Ts)
    g2 = d_a2 @ s1.T
    d_s1 = w2.T @ d_a2
    d_a1 = co.corr(co.spike_grad(d_s1, u1p, theta, tau, scale), k, Ts)
    g1 = d_a1 @ x.T
    assert np.linalg.norm(srm["gradW2Initial"] - g2) / g2.size < 1e-4
    assert np.linalg.norm(srm["gradW1Initial"] - g1) / g1.size < 1e-4


def test_loihi_network_matches_chip_recordings(loihi):
    """test/test_slayerLoihi001.py:96-133: hidden/output spikes and voltages recorded from a
    Loihi chip; weights round(w*4/2)*2, input delayed 49 bins, 1-bin axonal delay per layer."""
    T = 500
    w1 = np.round(loihi["w1learned"] * 4 / 2) * 2
    w2 = np.round(loihi["w2learned"] * 4 / 2) * 2
    x = dense_events(loihi["spikeIn"], 250, T, 1 / 0.1)
    args = (0, 80 * 64, 1024, 128, 1)
    # spikeLoihiFull multiplies by Ts before the op and divides spikes by Ts after it
    s1, v1, _ = co.loihi_get_spikes(((w1 @ x) * 0.1).astype(np.float32), *args)
    s1 = co.shift(s1 / np.float32(0.1), 1.0, 1.0)
    s2, v2, _ = co.loihi_get_spikes(((w2 @ s1) * 0.1).astype(np.float32), *args)
    s2 = co.shift(s2 / np.float32(0.1), 1.0, 1.0)
    np.testing.assert_array_equal(s1 > 0, dense_events(loihi["hiddenSpikes"], 25, T, 1) > 0)
    np.testing.assert_array_equal(s2 > 0, dense_events(loihi["outputSpikes"], 1, T, 1) > 0)
    np.testing.assert_allclose(v1[24, :-1], loihi["hiddenVoltage24"], atol=1e-3)
    np.testing.assert_allclose(v2[0, :-1], loihi["outputVoltage"], atol=1e-3)


def test_loihi_matches_reference_numpy_model(refpy):
    """test/test_slayerLoihi002.py:112-126 on stored outputs of its Neuron.run model."""
    for k in range(int(refpy["nrn_count"])):
        p = [int(v) for v in refpy["nrn%d_params" % k]]
        w = refpy["nrn%d_w" % k]
        for impl in (co, nl):
            s, v, u = impl.loihi_get_spikes(w, *p)
            np.testing.assert_array_equal(s, refpy["nrn%d_spike" % k])
            np.testing.assert_array_equal(u, refpy["nrn%d_current" % k])
            np.testing.assert_array_equal(v, refpy["nrn%d_voltage" % k])


def test_loihi_uint32_wraparound_c_vs_numpy():
    rng = np.random.RandomState(5)
    w = np.round(rng.randn(16, 300) * 3e5).astype(np.float32)   # drives |state|*4096 past 2^32
    a = co.loihi_get_spikes(w, 1, 5120, 10, 3, 2)
    b = nl.loihi_get_spikes(w, 1, 5120, 10, 3, 2)
    for x, y in zip(a, b):
        np.testing.assert_array_equal(x, y)


def test_shift_recipe_of_reference_test(refpy):
    """test/test_slayer009.py:46-81: Ts = 0.1, delays in (-1, 1) per neuron; scalar delay 4."""
    rng = np.random.RandomState(9)
    x = rng.randn(3, 4, 5, 2, 50).astype(np.float32)
    lut = (rng.rand(4, 5, 2) * 2 - 1).astype(np.float32)
    y = co.shift(x, lut, 0.1)
    np.testing.assert_array_equal(y, nl.shift(x, lut, 0.1))
    for c in range(4):
        for h in range(5):
            for w in range(2):
                d = int((lut[c, h, w] / np.float32(0.1)).item())
                a, b = x[:, c, h, w], y[:, c, h, w]
                if d > 0:
                    assert np.array_equal(a[:, :-d], b[:, d:]) and not b[:, :d].any()
                elif d == 0:
                    assert np.array_equal(a, b)
                else:
                    assert np.array_equal(a[:, -d:], b[:, :d]) and not b[:, d:].any()
    y4 = co.shift(x, 4, 1)
    assert np.array_equal(x[..., :-4], y4[..., 4:]) and not y4[..., :4].any()
    for d in (0, 1, -1, 49, -49, 50, -50, 150, 2.7, -2.7):
        np.testing.assert_array_equal(co.shift(x, d, 1.0), nl.shift(x, d, 1.0))


def test_spike_grad_c_vs_numpy():
    rng = np.random.RandomState(3)
    g = rng.randn(5, 64).astype(np.float32)
    u = (rng.randn(5, 64) * 20).astype(np.float32)
    np.testing.assert_allclose(co.spike_grad(g, u, 10, 10, 1), nl.spike_grad(g, u, 10, 10, 1), rtol=1e-6, atol=1e-12)


def test_delay_grad_c_vs_composition():
    """oracle delay_grad = Ts * sum(g * conv(out, [-1, 1]/Ts, 1)) (src/slayer.py:950-954)."""
    rng = np.random.RandomState(8)
    for Ts in (1.0, 0.5):
        g = rng.randn(4, 3, 2, 1, 50).astype(np.float32)
        out = rng.randn(4, 3, 2, 1, 50).astype(np.float32)
        diff = co.conv(out, np.array([-1.0, 1.0], np.float32) / Ts, 1.0)
        want = (g.astype(np.float64) * diff).sum(axis=(0, -1)) * Ts
        got = co.delay_grad(g, out, Ts)
        assert got.shape == (3, 2, 1)
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)


def test_srm_c_vs_numpy_random():
    rng = np.random.RandomState(11)
    for T, nus in ((1, 3), (7, 11), (64, 1), (300, 11), (97, 160)):
        u = (rng.randn(2, 3, 1, 2, T) * 8).astype(np.float32)
        nu = -np.abs(rng.randn(nus)).astype(np.float32) * 5
        a = co.srm_get_spikes(u, nu, 10.0, 1.0)
        b = nl.srm_get_spikes(u, nu, 10.0, 1.0)
        np.testing.assert_array_equal(a[0], b[0])
        np.testing.assert_array_equal(a[1], b[1])


def test_event_binning_oracle_equals_the_reference_function(golden_dir):
    """oracle.numpy_loops.bin_events against spike tensors made by the reference's own
    event.toSpikeTensor (src/spikeFileIO.py:66-144) from seeded synthetic events."""
    from oracle import numpy_loops as nl
    g = np.load(golden_dir + "/events_ref.npz")
    assert len(g["cases"]) >= 5
    for case in g["cases"]:
        tag, mode = str(case).split(":")
        y = g[tag + "_y"] if tag + "_y" in g else None
        got = nl.bin_events(g[tag + "_start"], g[tag + "_x"], y, g[tag + "_p"], g[tag + "_t"], float(g[tag + "_Ts"]), 0, mode)
        np.testing.assert_array_equal(got, g[tag + "_out"], err_msg=tag)
