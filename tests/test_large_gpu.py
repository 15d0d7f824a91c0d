"""GPU: every operator on tensors with more than 2^31 elements (64-bit indexing), checked on
sampled rows against the oracle.  Rows are independent, so a sample of rows - the first and
last ones, the ones around element 2^31, and a random handful - covers the index arithmetic.
Needs about 45 GB of device memory; skipped on smaller devices."""
import numpy as np
import pytest
import torch

import slayerpytorch_b200
from oracle import cpu_oracle as co
from slayerpytorch_b200.layer import alpha_kernel

pytestmark = pytest.mark.gpu

T, BATCH, NEURONS = 300, 14500, 512            # 7,424,000 rows x 300 = 2.227e9 elements
ROWS = BATCH * NEURONS


@pytest.fixture(scope="module")
def big():
    free, _ = torch.cuda.mem_get_info()
    if free < 60e9:
        pytest.skip("needs about 45 GB of free device memory")
    assert ROWS * T > 2 ** 31
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.empty(BATCH, NEURONS, 1, 1, T, device=dev)
    x.normal_(generator=g).abs_().mul_(2.5)
    m = torch.empty_like(x).uniform_(generator=g)
    x.mul_((m < 0.3).float())
    del m
    boundary = (2 ** 31) // T
    sample = sorted(set([0, 1, 31, 32, ROWS - 1, ROWS - 32, ROWS - 33, boundary - 1, boundary, boundary + 1,
                         ROWS // 2 + 7] + list(np.random.RandomState(0).randint(0, ROWS, 40))))
    co.set_ftz(True)
    yield {"x": x, "sample": sample, "idx": torch.tensor(sample, device=dev), "gen": g,
           "srm": torch.tensor(alpha_kernel(10.0, 1.0, 300), dtype=torch.float32, device=dev),
           "ref": torch.tensor(alpha_kernel(1.0, 1.0, 300, mult=-20.0), dtype=torch.float32, device=dev),
           "delay": torch.rand(NEURONS, device=dev, generator=g) * 5}
    co.set_ftz(False)
    torch.cuda.empty_cache()


def pick(t, big):
    return t.view(ROWS, T)[big["idx"]].cpu().numpy()


def test_srm_chain_beyond_2_to_31_elements(big):
    sc, _ = slayerpytorch_b200.load_ops()
    x, sample = big["x"], big["sample"]
    xs = pick(x, big)
    k, r, dl = big["srm"].cpu().numpy(), big["ref"].cpu().numpy(), big["delay"].cpu().numpy()
    lut_of = lambda i: dl[[sample[i] % NEURONS]]

    u = sc.conv(x, big["srm"], 1.0)
    np.testing.assert_array_equal(pick(u, big), co.conv(xs, k, 1.0))
    c = sc.corr(x, big["srm"], 1.0)
    np.testing.assert_array_equal(pick(c, big), co.corr(xs, k, 1.0))
    del c
    u0s = pick(u, big)
    s = sc.getSpikes(u, big["ref"], 10.0, 1.0)
    s_w, u_w = co.srm_get_spikes(u0s, r, 10.0, 1.0)
    assert 0.01 < s_w.mean() < 0.5
    np.testing.assert_array_equal(pick(s, big), s_w)
    np.testing.assert_array_equal(pick(u, big), u_w)

    d = sc.shift(s, big["delay"], 1.0)
    want_d = np.stack([co.shift(s_w[i].reshape(1, 1, T), lut_of(i), 1.0).reshape(T) for i in range(len(sample))])
    np.testing.assert_array_equal(pick(d, big), want_d)
    del d
    u2 = sc.conv(x, big["srm"], 1.0)
    dd = sc.getSpikesDelayed(u2, big["ref"], 10.0, 1.0, big["delay"])
    np.testing.assert_array_equal(pick(dd, big), want_d)
    np.testing.assert_array_equal(pick(u2, big), u_w)
    del dd, u2

    gs = sc.spikeGradShift(x, u, -big["delay"], 10.0, 10.0, 1.0, 1.0)
    want = np.stack([co.spike_grad(co.shift(xs[i].reshape(1, 1, T), -lut_of(i), 1.0).reshape(T), u_w[i], 10.0, 10.0, 1.0)
                     for i in range(len(sample))])
    np.testing.assert_allclose(pick(gs, big), want, rtol=1e-5, atol=1e-37)
    del gs
    sg = sc.spikeGrad(x, u, 10.0, 10.0, 1.0)
    np.testing.assert_allclose(pick(sg, big), co.spike_grad(xs, u_w, 10.0, 10.0, 1.0), rtol=1e-5, atol=1e-37)
    del sg

    dg = sc.delayGrad(x, s, 1.0)
    assert dg.shape == (NEURONS, 1, 1) and bool(torch.isfinite(dg).all())
    for n in (0, NEURONS - 1):
        gx = x.view(BATCH, NEURONS, T)[:, n].double()
        so = s.view(BATCH, NEURONS, T)[:, n].double()
        prev = torch.zeros_like(so)
        prev[:, 1:] = so[:, :-1]
        want_n = (gx * (prev - so)).sum().item()
        assert abs(dg.view(-1)[n].item() - want_n) <= 1e-4 * max(1.0, abs(want_n))


def test_loihi_beyond_2_to_31_elements(big):
    _, lc = slayerpytorch_b200.load_ops()
    dev = big["x"].device
    w = torch.randint(-128, 128, (BATCH, NEURONS, 1, 1, T), device=dev, generator=big["gen"]).float()
    m = torch.empty_like(w).uniform_(generator=big["gen"])
    w.mul_((m < 0.05).float())
    del m
    outs = lc.getSpikes(w, 0, 5120, 1024, 128, 1)
    for got, want in zip(outs, co.loihi_get_spikes(pick(w, big), 0, 5120, 1024, 128, 1)):
        np.testing.assert_array_equal(pick(got, big), want)


# ------------------------------------------ the largest layers of the CNN and Loihi workloads
def sampled(t, rows, T, idx):
    return t.view(rows, T)[idx].cpu().numpy()


def test_cnn_first_layer_shape_rows_match_oracle():
    """The first spiking layer of the SRM CNN workload at full size (128 x 16 x 32 x 32 neurons =
    2,097,152 rows x 300 steps, 2.5 GB per tensor): getSpikes, then psp on the spike tensor,
    the surrogate gradient and corr, checked on 1200 random rows against the oracle."""
    free, _ = torch.cuda.mem_get_info()
    if free < 30e9:
        pytest.skip("needs about 20 GB of free device memory")
    sc, _ = slayerpytorch_b200.load_ops()
    dev = torch.device("cuda")
    N, C, H, W, T = 128, 16, 32, 32, 300
    rows = N * C * H * W
    g = torch.Generator(device=dev).manual_seed(1003)
    srm = torch.tensor(alpha_kernel(10.0, 1.0, 300), dtype=torch.float32, device=dev)
    ref = torch.tensor(alpha_kernel(1.0, 1.0, 300, mult=-20.0), dtype=torch.float32, device=dev)
    # membrane potential of a convolution layer fed with psp of 5 % input spikes: smooth, a few
    # percent of the samples above threshold
    a = torch.empty(N, C, H, W, T, device=dev).normal_(generator=g).mul_(2.5)
    m = torch.empty_like(a).uniform_(generator=g)
    a.mul_((m < 0.25).float())
    del m
    u = sc.conv(a, srm, 1.0)
    idx_np = np.sort(np.random.RandomState(3).choice(rows, 1200, replace=False))
    idx_np[:3], idx_np[-3:] = (0, 1, 31), (rows - 33, rows - 32, rows - 1)
    idx = torch.from_numpy(idx_np).to(dev)
    k, r = srm.cpu().numpy(), ref.cpu().numpy()
    co.set_ftz(True)
    try:
        u0 = sampled(u, rows, T, idx)
        np.testing.assert_array_equal(u0, co.conv(sampled(a, rows, T, idx), k, 1.0))
        del a
        s = sc.getSpikes(u, ref, 10.0, 1.0)
        s_w, u_w = co.srm_get_spikes(u0, r, 10.0, 1.0)
        assert 0.002 < s_w.mean() < 0.3
        np.testing.assert_array_equal(sampled(s, rows, T, idx), s_w)
        np.testing.assert_array_equal(sampled(u, rows, T, idx), u_w)
        assert torch.all((s == 0) | (s == 1.0))
        p = sc.conv(s, srm, 1.0)                          # psp of a spike tensor (mostly zeros)
        np.testing.assert_array_equal(sampled(p, rows, T, idx), co.conv(s_w, k, 1.0))
        del p
        gout = torch.empty(N, C, H, W, T, device=dev).normal_(generator=g)
        gu = sc.spikeGrad(gout, u, 10.0, 10.0, 1.0)
        want = co.spike_grad(sampled(gout, rows, T, idx), u_w, 10.0, 10.0, 1.0)
        np.testing.assert_allclose(sampled(gu, rows, T, idx), want, rtol=1e-5, atol=1e-37)
        del gout
        c = sc.corr(gu, srm, 1.0)
        np.testing.assert_array_equal(sampled(c, rows, T, idx), co.corr(sampled(gu, rows, T, idx), k, 1.0))
    finally:
        co.set_ftz(False)
        torch.cuda.empty_cache()


def test_loihi_first_layer_shape_rows_match_oracle():
    """The first layer of the Loihi workload at full size (64 x 16 x 32 x 32 neurons = 1,048,576
    rows x 1450 steps, 6.1 GB per tensor, rows not 16-byte aligned): all three outputs exact on
    1000 random rows, then the unit delay, the surrogate gradient on the voltage and corr with
    the 110-tap Loihi response."""
    free, _ = torch.cuda.mem_get_info()
    if free < 60e9:
        pytest.skip("needs about 45 GB of free device memory")
    sc, lc = slayerpytorch_b200.load_ops()
    from slayerpytorch_b200.layer import loihi_psp_kernel
    dev = torch.device("cuda")
    N, C, H, W, T = 64, 16, 32, 32, 1450
    rows = N * C * H * W
    g = torch.Generator(device=dev).manual_seed(1005)
    # weighted input of a 5x5x2 convolution with integer weights over 2 % input spikes
    w = torch.randint(-128, 128, (N, C, H, W, T), device=dev, generator=g).float()
    m = torch.empty_like(w).uniform_(generator=g)
    w.mul_((m < 0.1).float())
    del m
    idx_np = np.sort(np.random.RandomState(5).choice(rows, 1000, replace=False))
    idx_np[:3], idx_np[-3:] = (0, 1, 31), (rows - 33, rows - 32, rows - 1)
    idx = torch.from_numpy(idx_np).to(dev)
    s, v, u = lc.getSpikes(w, 0, 5120, 1024, 128, 1)
    want = co.loihi_get_spikes(sampled(w, rows, T, idx), 0, 5120, 1024, 128, 1)
    del w
    for got, b, name in zip((s, v, u), want, ("spike", "voltage", "current")):
        np.testing.assert_array_equal(sampled(got, rows, T, idx), b, err_msg=name)
    assert 0.001 < want[0].mean() < 0.6
    del u
    d = sc.shift(s, 1.0, 1.0)
    assert torch.equal(d[..., 1:], s[..., :-1]) and not d[..., 0].any()
    del d, s
    k = torch.tensor(loihi_psp_kernel({"iDecay": 1024, "vDecay": 128, "wgtExp": 0}), dtype=torch.float32, device=dev)
    assert k.numel() == 110
    gout = torch.empty(N, C, H, W, T, device=dev).normal_(generator=g)
    gu = sc.spikeGrad(gout, v, 5120.0, 5120.0, 1.0 / 195.0)
    np.testing.assert_allclose(sampled(gu, rows, T, idx),
                               co.spike_grad(sampled(gout, rows, T, idx), want[1], 5120.0, 5120.0, 1.0 / 195.0),
                               rtol=1e-5, atol=1e-37)
    del gout, v
    co.set_ftz(True)
    try:
        c = sc.corr(gu, k, 1.0)
        np.testing.assert_array_equal(sampled(c, rows, T, idx), co.corr(sampled(gu, rows, T, idx), k.cpu().numpy(), 1.0))
    finally:
        co.set_ftz(False)
        torch.cuda.empty_cache()
