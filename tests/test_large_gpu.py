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
