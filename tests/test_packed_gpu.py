"""GPU: bit-packed spike tensors (32 time steps per word) against the fp32 operators and the oracle.

The packed operators must give exactly what the fp32 ones give: pack / unpack are each other's
inverse, getSpikes writes the same spike positions and the same updated potential whether the
spikes leave as bits or as samples, and the psp filter of a packed tensor has the bits of the
filter of its fp32 view.
"""
import numpy as np
import pytest
import torch

import slayerpytorch_b200
from oracle import cpu_oracle as co
from slayerpytorch_b200.capi import SlayerB200Error
from tests import gpu_util as G

pytestmark = pytest.mark.gpu


def setup_module(module):
    co.set_ftz(True)


def teardown_module(module):
    co.set_ftz(False)


def np_pack(s):
    """Reference packing on the host: little-endian bit order inside 32-bit words."""
    T = s.shape[-1]
    pad = (-T) % 32
    b = np.concatenate([s != 0, np.zeros(s.shape[:-1] + (pad,), bool)], axis=-1)
    return np.packbits(b, axis=-1, bitorder="little").view(np.uint32).reshape(s.shape[:-1] + ((T + pad) // 32,))


@pytest.mark.parametrize("T", [1, 31, 32, 33, 64, 300, 301, 1450, 2000])
def test_pack_unpack_round_trip(T):
    rng = np.random.RandomState(T)
    s = ((rng.rand(3, 5, 2, 1, T) < 0.2) * 10.0).astype(np.float32)
    s[0, 0, 0, 0, -1] = 10.0
    bits = G.c_pack(G.dev(s))
    np.testing.assert_array_equal(G.host(bits).view(np.uint32), np_pack(s))
    np.testing.assert_array_equal(G.host(G.c_unpack(bits, T, 10.0)), s)
    np.testing.assert_array_equal(G.host(G.c_unpack(bits, T, 0.25)), (s != 0) * np.float32(0.25))


@pytest.mark.parametrize("T", [4, 32, 36, 64, 100, 128, 300, 500, 2000])
@pytest.mark.parametrize("nus", [1, 11, 34, 110])
def test_get_spikes_packed_equals_get_spikes(T, nus):
    rng = np.random.RandomState(T * 3 + nus)
    u0 = (rng.randn(3, 7, 1, 5, T) * 8).astype(np.float32)          # 105 rows: a partial block of 32
    nu = (-np.abs(rng.randn(nus)) * 6).astype(np.float32)
    for theta in (10.0, -1.0):                    # theta < 0: the zero padding past the row end would spike
        ua, ub = G.dev(u0), G.dev(u0)
        s = G.c_srm(ua, G.dev(nu), theta, 1.0)
        bits = G.c_srm_packed(ub, G.dev(nu), theta)
        np.testing.assert_array_equal(G.host(bits).view(np.uint32), np_pack(G.host(s)))
        np.testing.assert_array_equal(G.host(ub), G.host(ua))
        s_o, u_o = co.srm_get_spikes(u0, nu, theta, 1.0)
        np.testing.assert_array_equal(G.host(bits).view(np.uint32), np_pack(s_o))
        np.testing.assert_array_equal(G.host(ub), u_o)
    assert s.sum() > 0 or T < 8


def test_get_spikes_packed_sizes_the_kernel_does_not_take():
    """T % 4 != 0: the C entry point says so; the Python operator runs getSpikes + packSpikes."""
    sc, _ = slayerpytorch_b200.load_ops()
    rng = np.random.RandomState(9)
    u0 = (rng.randn(2, 6, 1, 1, 301) * 8).astype(np.float32)
    nu = (-np.abs(rng.randn(11)) * 6).astype(np.float32)
    with pytest.raises(SlayerB200Error):
        G.c_srm_packed(G.dev(u0), G.dev(nu), 10.0)
    ua, ub = G.dev(u0), G.dev(u0)
    bits = sc.getSpikesPacked(ua, G.dev(nu), 10.0, 1.0)
    s = sc.getSpikes(ub, G.dev(nu), 10.0, 1.0)
    np.testing.assert_array_equal(G.host(bits).view(np.uint32), np_pack(G.host(s)))
    np.testing.assert_array_equal(G.host(ua), G.host(ub))
    assert torch.equal(sc.unpackSpikes(bits, 301, 1.0), s) and torch.equal(sc.packSpikes(s), bits)


@pytest.mark.parametrize("zeros", [0, 1, 2])
@pytest.mark.parametrize("density", [0.002, 0.05, 0.5])
@pytest.mark.parametrize("T,K", [(300, 77), (301, 77), (64, 8), (1450, 110), (33, 40), (2000, 2)])
def test_conv_packed_equals_conv_of_the_fp32_view(density, T, K, zeros):
    """zeros: the zero-skipping setting - dense tiled kernel only, probe (these inputs have 2^25
    samples and more where T allows the event-driven kernel), event-driven kernel forced."""
    from slayerpytorch_b200 import capi
    rng = np.random.RandomState(int(density * 1000) + T + K)
    rows = (1 << 25) // T + 5 if T >= 64 else 9000
    gen = torch.Generator(device="cuda").manual_seed(int(density * 1000) + T + K)
    s = (torch.rand(rows, T, device="cuda", generator=gen) < density).float()
    f = rng.randn(K).astype(np.float32)
    bits = G.c_pack(s)
    before = capi.set_fir_skip_zeros(zeros)
    try:
        for Ts in (1.0, 0.1):
            value = np.float32(1.0) / np.float32(Ts)
            got = G.c_conv_packed(bits, T, G.dev(f), value, Ts)
            capi.set_fir_skip_zeros(0)
            assert torch.equal(got, G.c_conv(s * float(value), G.dev(f), Ts))
            capi.set_fir_skip_zeros(zeros)
            np.testing.assert_array_equal(G.host(got[:300]), co.conv(G.host(s[:300]) * value, f, Ts))
    finally:
        capi.set_fir_skip_zeros(before)
    assert capi.device_status() == 0


@pytest.mark.parametrize("density", [0.05, 0.5])
@pytest.mark.parametrize("T,K", [(300, 77), (301, 77), (1450, 110)])
def test_conv_packed_two_row_kernel(density, T, K):
    """Dense packed input goes to the scalar kernel, which expands the bits while it fills its
    tiles; slayer_b200_set_fir_packed(1) sends it to the two-row kernel instead.  Same bits."""
    from slayerpytorch_b200 import capi
    rng = np.random.RandomState(int(density * 1000) + T + K + 1)
    s = (rng.rand(3000, T) < density).astype(np.float32)
    f = rng.randn(K).astype(np.float32)
    bits = G.c_pack(G.dev(s))
    want = co.conv(s * np.float32(2.0), f, 0.5)
    before = capi.set_fir_skip_zeros(0), capi.set_fir_packed(0)
    try:
        for two_row in (0, 1):
            capi.set_fir_packed(two_row)
            np.testing.assert_array_equal(G.host(G.c_conv_packed(bits, T, G.dev(f), 2.0, 0.5)), want)
    finally:
        capi.set_fir_skip_zeros(before[0])
        capi.set_fir_packed(before[1])
    assert capi.device_status() == 0


def test_conv_packed_very_long_filter():
    sc, _ = slayerpytorch_b200.load_ops()
    rng = np.random.RandomState(4)
    s = (rng.rand(3, 2500) < 0.05).astype(np.float32)
    f = (rng.randn(2300) * 0.05).astype(np.float32)
    bits = G.c_pack(G.dev(s))
    with pytest.raises(SlayerB200Error):
        G.c_conv_packed(bits, 2500, G.dev(f), 1.0, 1.0)
    got = sc.convPacked(bits, 2500, G.dev(f), 1.0, 1.0)          # the operator unpacks and filters
    np.testing.assert_array_equal(G.host(got), co.conv(s, f, 1.0))


def test_spike_then_psp_layer_function_equals_the_two_steps():
    """layer.spikePsp = psp(spike(u)) as one autograd node that keeps the spikes packed."""
    from slayerpytorch_b200 import layer as L
    neuron = {"type": "SRMALPHA", "theta": 10, "tauSr": 10.0, "tauRef": 1.0, "scaleRef": 2, "tauRho": 1, "scaleRho": 1}
    net = L.spikeLayer(neuron, {"Ts": 1.0, "tSample": 300}).cuda()
    g = torch.Generator().manual_seed(8)
    u0 = (torch.randn(4, 6, 3, 3, 300, generator=g) * 7).cuda()
    gout = torch.randn(4, 6, 3, 3, 300, generator=g).cuda()
    a = u0.clone().requires_grad_(True)
    pa = net.psp(net.spike(a * 1.0))
    pa.backward(gout)
    b = u0.clone().requires_grad_(True)
    pb, packed = net.spikePsp(b * 1.0)
    pb.backward(gout)
    assert torch.equal(pa, pb) and pa.abs().sum() > 0
    assert torch.equal(a.grad, b.grad)
    s = net.spike(u0.clone())
    assert torch.equal(packed.dense(), s) and packed.T == 300 and packed.bits.dtype == torch.int32
    assert torch.equal(net.psp(packed), net.psp(s))                 # psp accepts the packed form
