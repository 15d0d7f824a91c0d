"""GPU parity: the CUDA kernels, called through the C ABI, against the CPU oracle.

Integer / index / copy work (shift, spike positions, the updated SRM potential, all Loihi
outputs) must be bit-exact.  conv / corr reproduce the oracle's fused-multiply-add chain and
are also compared bit for bit; the stated tolerance of the task (1e-5 relative) is the
fallback assertion should a platform differ.  spike_grad is held to 1e-5 relative.
"""
import numpy as np
import pytest
import torch

from oracle import cpu_oracle as co
from tests import gpu_util as G

pytestmark = pytest.mark.gpu

REL = 1e-5   # tolerance for floating-point values (conv, corr, shift values, gradients)


def setup_module(module):
    co.set_ftz(True)       # the FIR and SRM kernels flush denormals like the reference build


def teardown_module(module):
    co.set_ftz(False)


def assert_same_floats(got, want):
    """Bit-exact up to NaN payloads: equal values, equal signs (so -0.0 stays -0.0), NaN where NaN."""
    np.testing.assert_array_equal(got, want)
    np.testing.assert_array_equal(np.signbit(got), np.signbit(want))


def assert_close_or_equal(got, want):
    if np.array_equal(got, want):
        return
    scale = np.maximum(np.abs(want), 1e-30)
    worst = np.max(np.abs(got - want) / scale)
    np.testing.assert_allclose(got, want, rtol=REL, atol=1e-30)
    pytest.fail("within %g relative but not bit-exact (worst %.3g)" % (REL, worst))


# ------------------------------------------------------------------------------- shift
@pytest.mark.parametrize("shape", [(1, 1, 1, 1, 1), (2, 3, 1, 1, 7), (3, 5, 2, 1, 300),
                                   (2, 7, 1, 3, 1450), (1, 33, 1, 1, 2000), (4, 9, 1, 1, 64)])
def test_shift_scalar(shape):
    rng = np.random.RandomState(sum(shape))
    x = rng.randn(*shape).astype(np.float32)
    xd = G.dev(x)
    T = shape[-1]
    for d in sorted({0, 1, -1, 2, 3, -3, 4, 5, T - 1, -(T - 1), T, -T, 3 * T, -3 * T, 2.7, -2.7}):
        for Ts in (1.0, 0.1):
            got = G.host(G.c_shift_scalar(xd, d, Ts))
            np.testing.assert_array_equal(got, co.shift(x, d, Ts), err_msg="d=%s Ts=%s" % (d, Ts))


@pytest.mark.parametrize("shape,Ts", [((5, 10, 4, 3, 500), 0.1), ((3, 16, 1, 1, 300), 1.0),
                                      ((2, 6, 2, 2, 1450), 1.0), ((4, 130, 1, 1, 30), 1.0),
                                      ((2, 3, 1, 1, 5), 0.5)])
def test_shift_per_neuron(shape, Ts):
    """Recipe of test/test_slayer009.py: delays in (-1, 1) at Ts = 0.1, plus wider ranges."""
    rng = np.random.RandomState(42 + shape[-1])
    x = rng.randn(*shape).astype(np.float32)
    for span in (1.0, 5.0, 2.0 * shape[-1] * Ts):
        lut = ((rng.rand(*shape[1:4]) * 2 - 1) * span).astype(np.float32)
        got = G.host(G.c_shift_lut(G.dev(x), G.dev(lut), Ts))
        np.testing.assert_array_equal(got, co.shift(x, lut, Ts))


def test_shift_unaligned_buffers_take_the_scalar_path():
    rng = np.random.RandomState(7)
    flat = rng.randn(4 * 300 + 3).astype(np.float32)
    base = G.dev(flat)
    for off in (1, 2, 3):
        xd = base[off:off + 1200].view(1, 4, 1, 1, 300)
        x = flat[off:off + 1200].reshape(1, 4, 1, 1, 300)
        np.testing.assert_array_equal(G.host(G.c_shift_scalar(xd, 3, 1.0)), co.shift(x, 3, 1.0))


# --------------------------------------------------------------------------- conv / corr
@pytest.fixture(params=["scalar-lean", "scalar", "scalar-no-row-offsets", "scalar-run-exit", "scalar-tile-barrier", "packed",
                        "packed-half-tiles", "packed-full-tiles", "event-driven"])
def fir_variant(request):
    """conv / corr have several kernels that must give the same bits: the scalar one in its three
    forms (segments dealt out across tiles with split-phase barriers, the same with more
    registers - the default, which also keeps 16-byte accesses for rows that are off the 16-byte
    grid by giving each row an offset inside the tile -, that without the row offsets, that with
    the loop over the tap groups always left where the groups end, one CTA-wide barrier per tile),
    the packed one (two rows per lane,
    two-wide FMAs) with either of its tile sizes, and the event-driven one (a list of non-zero
    samples per row; here forced on whatever the input holds)."""
    from slayerpytorch_b200 import capi
    packed, flow, zeros = {"scalar-lean": (0, 1, 1), "scalar": (0, 2, 1), "scalar-no-row-offsets": (0, 3, 1),
                           "scalar-run-exit": (0, 4, 1),
                           "scalar-tile-barrier": (0, 0, 1), "packed": (1, 2, 1),
                           "packed-half-tiles": (2, 2, 1), "packed-full-tiles": (3, 2, 1),
                           "event-driven": (0, 2, 2)}[request.param]
    before = capi.set_fir_packed(packed), capi.set_fir_flow(flow), capi.set_fir_skip_zeros(zeros)
    yield request.param
    capi.set_fir_packed(before[0])
    capi.set_fir_flow(before[1])
    capi.set_fir_skip_zeros(before[2])
    assert capi.device_status() == 0


@pytest.mark.parametrize("T", [1, 5, 64, 300, 301, 500, 1450, 2000])
@pytest.mark.parametrize("K", [1, 2, 3, 4, 5, 11, 12, 13, 77, 110, 160])
def test_conv_corr_bit_exact(T, K, fir_variant):
    rng = np.random.RandomState(1000 * T + K)
    rows = 37 if T < 1000 else 33
    x = (rng.rand(rows, T) < 0.2).astype(np.float32) * rng.randn(rows, T).astype(np.float32)
    f = rng.randn(K).astype(np.float32)
    xd, fd = G.dev(x), G.dev(f)
    for Ts in (1.0, 0.1):
        assert_close_or_equal(G.host(G.c_conv(xd, fd, Ts)), co.conv(x, f, Ts))
        assert_close_or_equal(G.host(G.c_conv(xd, fd, Ts, corr=True)), co.corr(x, f, Ts))


def test_conv_delay_gradient_filter(fir_variant):
    """K = 2 difference filter of the delay gradient (src/slayer.py:950-953): (x[t-1]-x[t])/Ts."""
    rng = np.random.RandomState(3)
    x = rng.randn(2, 5, 1, 1, 300).astype(np.float32)
    f = (np.array([-1, 1], np.float32) / np.float32(0.1))
    got = G.host(G.c_conv(G.dev(x), G.dev(f), 1))
    assert_close_or_equal(got, co.conv(x, f, 1))
    want = np.zeros_like(x)
    want[..., 0] = -x[..., 0] * 10
    want[..., 1:] = (x[..., :-1] - x[..., 1:]) * 10
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-4)


def test_conv_spike_input_and_psp_kernel(golden_dir, fir_variant):
    g = np.load(golden_dir + "/ref_python.npz")
    for tag, kern in (("psp_Ts1", "srm_Ts1_srmKernel"), ("psp_kat", "srm_kat_srmKernel")):
        x, y, Ts = g[tag + "_in"], g[tag + "_out"], float(g[tag + "_Ts"])
        got = G.host(G.c_conv(G.dev(x), G.dev(g[kern]), Ts))
        assert np.linalg.norm(got - y) / y.size < 1e-6      # test/test_slayer011.py:39-43
        assert_close_or_equal(got, co.conv(x, g[kern], Ts))


def test_conv_many_rows_and_row_remainders(fir_variant):
    rng = np.random.RandomState(5)
    f = rng.randn(77).astype(np.float32)
    fd = G.dev(f)
    for rows in (1, 2, 31, 32, 33, 63, 64, 65, 127, 1000):
        x = rng.randn(rows, 300).astype(np.float32)
        assert_close_or_equal(G.host(G.c_conv(G.dev(x), fd, 1.0)), co.conv(x, f, 1.0))
        assert_close_or_equal(G.host(G.c_conv(G.dev(x), fd, 1.0, corr=True)), co.corr(x, f, 1.0))


def test_conv_unaligned_buffer(fir_variant):
    rng = np.random.RandomState(8)
    f = rng.randn(11).astype(np.float32)
    for rows, T in ((9, 300), (70, 302), (5, 77)):
        flat = rng.randn(rows * T + 3).astype(np.float32)
        base = G.dev(flat)
        for off in (1, 2, 3):
            xd = base[off:off + rows * T].view(rows, T)
            want = co.conv(flat[off:off + rows * T].reshape(rows, T), f, 1.0)
            assert_close_or_equal(G.host(G.c_conv(xd, G.dev(f), 1.0)), want)
            # input aligned, output not
            out = torch.full((rows * T + 3,), float("nan"), device="cuda")
            ov = out[off:off + rows * T].view(rows, T)
            xa = G.dev(flat[off:off + rows * T].reshape(rows, T))
            from slayerpytorch_b200 import capi
            capi.call("slayer_b200_conv", G.ptr(ov), G.ptr(xa), G.ptr(G.dev(f)), rows, T, f.size, 1.0, G.stream())
            assert_close_or_equal(G.host(ov), want)
            assert torch.isnan(out[:off]).all() and torch.isnan(out[off + rows * T:]).all()


@pytest.mark.parametrize("density", [0.0, 0.002, 0.01, 0.05])
@pytest.mark.parametrize("T,K", [(300, 77), (304, 8), (1450, 110), (40, 77)])
def test_conv_corr_on_spike_tensors_skip_zeros(density, T, K):
    """Mostly-zero inputs take the zero-skipping path of the packed kernel (one CTA walks several
    tiles here, so the per-tile switch between the two paths is exercised too); with the path
    switched off the dense path runs.  Both must give the oracle's bits."""
    from slayerpytorch_b200 import capi
    rng = np.random.RandomState(int(density * 1e4) + T + K)
    rows = 20000 if T <= 304 else 4200
    x = (rng.rand(rows, T) < density).astype(np.float32)
    x[rows // 3:rows // 3 + 700] = rng.randn(700, T).astype(np.float32)      # a dense stretch in the middle
    x[5, 7 % T] = -0.0
    f = rng.randn(K).astype(np.float32)
    xd, fd = G.dev(x), G.dev(f)
    want_conv, want_corr = co.conv(x, f, 1.0), co.corr(x, f, 1.0)
    before = capi.set_fir_packed(1)
    try:
        for mode, skip in ((2, True), (3, True), (1, False)):
            capi.set_fir_packed(mode)
            capi.set_fir_skip_zeros(skip)
            assert_close_or_equal(G.host(G.c_conv(xd, fd, 1.0)), want_conv)
            assert_close_or_equal(G.host(G.c_conv(xd, fd, 1.0, corr=True)), want_corr)
    finally:
        capi.set_fir_skip_zeros(True)
        capi.set_fir_packed(before)


@pytest.mark.parametrize("density", [0.0, 0.01, 0.04, 0.3])
@pytest.mark.parametrize("T,K", [(300, 77), (301, 2), (1450, 110), (64, 64), (4096, 33)])
def test_conv_corr_probe_picks_a_kernel_and_the_bits_do_not_change(density, T, K):
    """conv inputs of 2^25 samples and more are sampled on the device and go to the event-driven
    kernel or to the dense one; forced either way the bits are the same (corr too, which only takes
    the event-driven kernel when forced), and the oracle's on sampled rows.  Some rows are dense,
    one holds non-finite samples, a -0.0 counts as zero."""
    from slayerpytorch_b200 import capi
    rng = np.random.RandomState(int(density * 1e3) + T + K)
    rows = (1 << 25) // T + 37
    gen = torch.Generator(device="cuda").manual_seed(int(density * 1e3) + T + K)
    xd = torch.randn(rows, T, device="cuda", generator=gen)
    xd.mul_((torch.rand(rows, T, device="cuda", generator=gen) < density).float())
    special = {11: rng.randn(T), rows - 1: rng.randn(T), 17: np.zeros(T), 5: np.zeros(T)}
    special[5][7 % T] = -0.0
    special[17][T // 2], special[17][T - 1], special[17][0] = np.inf, np.nan, -np.inf
    for r, v in special.items():
        xd[r] = torch.from_numpy(v.astype(np.float32)).cuda()
    f = rng.randn(K).astype(np.float32)
    fd = G.dev(f)
    got = {}
    before = capi.set_fir_skip_zeros(1)
    try:
        for mode in (0, 1, 2):
            capi.set_fir_skip_zeros(mode)
            got[mode] = (G.c_conv(xd, fd, 0.5), G.c_conv(xd, fd, 0.5, corr=True))
    finally:
        capi.set_fir_skip_zeros(before)
    for mode in (1, 2):
        for a, b in zip(got[mode], got[0]):
            assert torch.equal(torch.nan_to_num(a, nan=12345.0), torch.nan_to_num(b, nan=12345.0))
            assert torch.equal(torch.isnan(a), torch.isnan(b))
    pick = torch.tensor([0, 1, 5, 11, 12, 16, 18, rows // 2, rows - 2, rows - 1], device="cuda")
    x = G.host(xd[pick])
    assert_close_or_equal(G.host(got[1][0][pick]), co.conv(x, f, 0.5))
    assert_close_or_equal(G.host(got[1][1][pick]), co.corr(x, f, 0.5))


def test_conv_probe_with_a_non_finite_tap_takes_the_dense_kernel():
    """0 x Inf is NaN: with a non-finite tap a zero sample does change the sums it enters, so the
    probe rules the event-driven kernel out and the dense result stands."""
    from slayerpytorch_b200 import capi
    rng = np.random.RandomState(21)
    rows, T = (1 << 25) // 300 + 1, 300
    xd = (torch.rand(rows, T, device="cuda") < 0.01).float()
    f = rng.randn(20).astype(np.float32)
    f[7] = -np.inf
    fd = G.dev(f)
    before = capi.set_fir_skip_zeros(0)
    try:
        dense = G.c_conv(xd, fd, 1.0)
        capi.set_fir_skip_zeros(1)
        auto = G.c_conv(xd, fd, 1.0)
    finally:
        capi.set_fir_skip_zeros(before)
    assert not torch.isfinite(dense[:, 7:]).any()
    assert torch.equal(torch.isnan(auto), torch.isnan(dense))
    assert torch.equal(torch.nan_to_num(auto, nan=1.0), torch.nan_to_num(dense, nan=1.0))


def test_conv_skip_zeros_with_non_finite_samples():
    """An Inf or NaN sample only reaches the outputs within K taps of it, on both paths."""
    from slayerpytorch_b200 import capi
    rng = np.random.RandomState(11)
    x = (rng.rand(256, 300) < 0.004).astype(np.float32)
    x[3, 100], x[70, 5], x[200, 299], x[201, 0] = np.inf, np.nan, -np.inf, np.inf
    f = rng.randn(77).astype(np.float32)
    xd, fd = G.dev(x), G.dev(f)
    got = {}
    before = capi.set_fir_packed(True)
    try:
        for skip in (True, False):
            capi.set_fir_skip_zeros(skip)
            got[skip] = (G.host(G.c_conv(xd, fd, 1.0)), G.host(G.c_conv(xd, fd, 1.0, corr=True)))
    finally:
        capi.set_fir_skip_zeros(True)
        capi.set_fir_packed(before)
    for a, b in zip(got[True], got[False]):
        np.testing.assert_array_equal(a, b)                  # NaN == NaN in this comparison
    conv = got[True][0]
    assert np.isfinite(conv[3, :100]).all() and not np.isfinite(conv[3, 100:177]).any() and np.isfinite(conv[3, 177:]).all()
    np.testing.assert_array_equal(conv[4], co.conv(x[4:5], f, 1.0)[0])


def test_conv_very_long_filter_fallback(fir_variant):
    rng = np.random.RandomState(9)
    x = rng.randn(3, 2500).astype(np.float32)
    f = (rng.randn(2300) * 0.05).astype(np.float32)
    assert_close_or_equal(G.host(G.c_conv(G.dev(x), G.dev(f), 1.0)), co.conv(x, f, 1.0))
    assert_close_or_equal(G.host(G.c_conv(G.dev(x), G.dev(f), 1.0, corr=True)), co.corr(x, f, 1.0))


# ------------------------------------------------------------------------- SRM getSpikes
def srm_case(rng, shape, nus, scale=8.0):
    u = (rng.randn(*shape) * scale).astype(np.float32)
    nu = (-np.abs(rng.randn(nus)) * 6).astype(np.float32)
    return u, nu


@pytest.mark.parametrize("T", [1, 2, 31, 32, 33, 64, 68, 100, 128, 132, 300, 500, 2000])
@pytest.mark.parametrize("nus", [1, 2, 11, 33, 34, 65, 110, 160, 257])
def test_srm_get_spikes_bit_exact(T, nus):
    rng = np.random.RandomState(T * 1000 + nus)
    u, nu = srm_case(rng, (2, 3, 1, 7, T), nus)
    ud = G.dev(u)
    s = G.host(G.c_srm(ud, G.dev(nu), 10.0, 1.0))
    s_want, u_want = co.srm_get_spikes(u, nu, 10.0, 1.0)
    np.testing.assert_array_equal(s, s_want)
    assert_same_floats(G.host(ud), u_want)
    assert T < 4 or s.sum() > 0


def test_srm_long_refractory_kernel_fallback():
    rng = np.random.RandomState(77)
    u, nu = srm_case(rng, (1, 5, 1, 1, 700), 400)
    ud = G.dev(u)
    s = G.host(G.c_srm(ud, G.dev(nu), 10.0, 1.0))
    s_want, u_want = co.srm_get_spikes(u, nu, 10.0, 1.0)
    np.testing.assert_array_equal(s, s_want)
    np.testing.assert_array_equal(G.host(ud), u_want)


def test_srm_edge_values():
    """theta hit exactly, nu[0] != 0, dense bursts (positive kernel), NaN / Inf rows, Ts != 1."""
    rng = np.random.RandomState(123)
    T = 100
    u = (rng.randn(1, 6, 1, 1, T) * 5).astype(np.float32)
    u[0, 0, 0, 0, ::7] = 10.0                      # exactly theta -> spike (>=)
    u[0, 1, 0, 0, :] = 11.0                        # spikes everywhere unless suppressed
    u[0, 2, 0, 0, 10] = np.nan
    u[0, 3, 0, 0, 20] = np.inf
    u[0, 4, 0, 0, 30] = -np.inf
    u[0, 5, 0, 0, :] = -0.0
    for nu in (np.array([0.5, -3, -2, -1], np.float32), np.array([1.0, 2.0, 0.5], np.float32),
               np.array([-20.0], np.float32)):
        for Ts in (1.0, 0.1, 2.0):
            ud = G.dev(u)
            s = G.host(G.c_srm(ud, G.dev(nu), 10.0, Ts))
            s_want, u_want = co.srm_get_spikes(u, nu, 10.0, Ts)
            np.testing.assert_array_equal(s > 0, s_want > 0)
            np.testing.assert_allclose(s, s_want, rtol=1e-6)
            assert_same_floats(G.host(ud), u_want)


def test_srm_minus_infinity_tap_is_an_absolute_refractory_period():
    """A tap of -inf (or a NaN tap) must only act after a spike (src/cuda/spikeKernels.h:22-33):
    rows that never spike keep their potential bit for bit, rows that spike read -inf (resp.
    NaN) for exactly the steps the tap covers."""
    rng = np.random.RandomState(321)
    for T in (100, 300, 301):
        u = (rng.randn(2, 20, 1, 1, T) * 6).astype(np.float32)
        u[0, 0] = -5.0                                           # never spikes
        u[0, 1, 0, 0, :] = 11.0                                  # would spike at every step
        for nu in (np.array([0.0, -np.inf, -np.inf, -20.0, -3.0], np.float32),
                   np.array([-0.0, -30.0, -np.inf], np.float32),
                   np.array([0.0, -5.0, np.nan, -1.0], np.float32)):
            ud = G.dev(u)
            s = G.host(G.c_srm(ud, G.dev(nu), 10.0, 1.0))
            s_want, u_want = co.srm_get_spikes(u, nu, 10.0, 1.0)
            np.testing.assert_array_equal(s, s_want)
            assert_same_floats(G.host(ud), u_want)
            assert np.array_equal(G.host(ud)[0, 0], u[0, 0]) and s.sum() > 0


@pytest.mark.parametrize("off", [1, 2, 3])
@pytest.mark.parametrize("T,nus", [(300, 11), (64, 2), (301, 11), (1450, 34), (130, 110)])
def test_srm_get_spikes_unaligned_buffers(off, T, nus):
    """Bases 4, 8 and 12 bytes off a 16-byte boundary: the 8- and 4-byte cp.async kernels."""
    rng = np.random.RandomState(off * 100 + T + nus)
    rows = 70
    flat_u = (rng.randn(rows * T + 3) * 8).astype(np.float32)
    nu = (-np.abs(rng.randn(nus)) * 6).astype(np.float32)
    base_u = G.dev(flat_u)
    base_s = torch.full((rows * T + 3,), float("nan"), device="cuda")
    ud = base_u[off:off + rows * T].view(2, 35, 1, 1, T)
    sd = base_s[off:off + rows * T].view(2, 35, 1, 1, T)
    assert ud.data_ptr() % 16 == 4 * off
    from slayerpytorch_b200 import capi
    capi.call("slayer_b200_srm_get_spikes", G.ptr(sd), G.ptr(ud), G.ptr(G.dev(nu)), rows, nus, T, 10.0, 1.0, G.stream())
    u = flat_u[off:off + rows * T].reshape(2, 35, 1, 1, T)
    s_want, u_want = co.srm_get_spikes(u, nu, 10.0, 1.0)
    np.testing.assert_array_equal(G.host(sd), s_want)
    assert_same_floats(G.host(ud), u_want)
    assert s_want.sum() > 0
    # nothing outside the views was touched
    assert torch.isnan(base_s[:off]).all() and torch.isnan(base_s[off + rows * T:]).all()
    np.testing.assert_array_equal(G.host(base_u)[:off], flat_u[:off])
    np.testing.assert_array_equal(G.host(base_u)[off + rows * T:], flat_u[off + rows * T:])


def test_srm_trace_of_reference_fixture(golden_dir):
    """test/test_slayer002.py:153-167 on the MATLAB trace, now on the GPU."""
    srm = np.load(golden_dir + "/srm_kat.npz")
    nu = np.load(golden_dir + "/ref_python.npz")["srm_kat_refKernel"]
    for key in ("spikeFuncHid", "spikeFuncOut"):
        data = srm[key][:500]
        ud = G.dev(data[:, 0].reshape(1, 1, 1, 1, -1))
        s = G.host(G.c_srm(ud, G.dev(nu), 10.0, 0.1)).ravel()
        np.testing.assert_array_equal(s > 0, data[:, 2] > 0)
        np.testing.assert_allclose(G.host(ud).ravel(), data[:, 1], atol=2e-3)


# ----------------------------------------------------------------------- Loihi getSpikes
@pytest.mark.parametrize("T", [1, 2, 33, 200, 1450])
@pytest.mark.parametrize("params", [(0, 5120, 1024, 128, 1), (0, 5120, 1024, 128, 2),
                                    (0, 5120, 1024, 128, 17), (1, 2560, 2048, 256, 3),
                                    (0, 320, 4095, 0, 63), (2, 100, 0, 4096, 5)])
def test_loihi_get_spikes_bit_exact(T, params):
    rng = np.random.RandomState(T + sum(params))
    w = (np.round((rng.rand(3, 11, 1, 2, T) - 0.5) * 60) * (rng.rand(3, 11, 1, 2, T) < 0.3)).astype(np.float32)
    got = G.c_loihi(G.dev(w), *params)
    want = co.loihi_get_spikes(w, *params)
    for a, b, name in zip(got, want, ("spike", "voltage", "current")):
        np.testing.assert_array_equal(G.host(a), b, err_msg=name)


def test_loihi_wraparound_negative_currents_and_fractions():
    rng = np.random.RandomState(55)
    w = np.round(rng.randn(40, 300) * 3e5).astype(np.float32)
    w[::3] *= -1
    w[1] = (rng.randn(300) * 3.7).astype(np.float32)          # int() truncates toward zero
    got = G.c_loihi(G.dev(w), 1, 5120, 10, 3, 2)
    want = co.loihi_get_spikes(w, 1, 5120, 10, 3, 2)
    for a, b in zip(got, want):
        np.testing.assert_array_equal(G.host(a), b)


@pytest.mark.parametrize("off", [1, 2, 3])
@pytest.mark.parametrize("T", [300, 1450, 33])
def test_loihi_get_spikes_unaligned_buffers(off, T):
    """Bases off a 16-byte boundary: the 8- and 4-byte tile kernels (T even/odd, offsets 4/8/12)."""
    rng = np.random.RandomState(off * 10 + T)
    rows = 45
    w = (np.round((rng.rand(rows * T + 3) - 0.5) * 90) * (rng.rand(rows * T + 3) < 0.3)).astype(np.float32)
    base_w = G.dev(w)
    outs = [torch.full((rows * T + 3,), float("nan"), device="cuda") for _ in range(3)]
    wd = base_w[off:off + rows * T].view(rows, T)
    views = [o[off:off + rows * T].view(rows, T) for o in outs]
    from slayerpytorch_b200 import capi
    capi.call("slayer_b200_loihi_get_spikes", G.ptr(views[0]), G.ptr(views[1]), G.ptr(views[2]), G.ptr(wd),
              rows, T, 0, 5120, 1024, 128, 2, G.stream())
    want = co.loihi_get_spikes(w[off:off + rows * T].reshape(rows, T), 0, 5120, 1024, 128, 2)
    for got, b, o in zip(views, want, outs):
        np.testing.assert_array_equal(G.host(got), b)
        assert torch.isnan(o[:off]).all() and torch.isnan(o[off + rows * T:]).all()
    assert want[0].sum() > 0


@pytest.mark.parametrize("theta", [0x7fffffff, 0x80000000, 0xffffff00])
def test_loihi_threshold_at_and_above_2_to_31(theta):
    """theta is unsigned in the signature and compared as a signed int (spikeLoihiKernels.h:64):
    from 2^31 on it is negative, so a voltage of zero is above threshold."""
    rng = np.random.RandomState(theta % 1000)
    for T in (64, 301):
        w = (np.round((rng.rand(40, T) - 0.5) * 60) * (rng.rand(40, T) < 0.3)).astype(np.float32)
        got = G.c_loihi(G.dev(w), 0, theta, 1024, 128, 2)
        want = co.loihi_get_spikes(w, 0, theta, 1024, 128, 2)
        for a, b, name in zip(got, want, ("spike", "voltage", "current")):
            np.testing.assert_array_equal(G.host(a), b, err_msg=name)
        assert (want[0].sum() > 0) == (theta >= 0x80000000)


@pytest.mark.parametrize("T", [1, 2, 33, 64, 65, 200, 1450])
@pytest.mark.parametrize("delay", [0, 1, 2, 31, 32, 63])
def test_loihi_get_spikes_delayed_equals_get_spikes_then_shift(T, delay):
    """Spikes written once, already delayed, with and without the current: the bits of getSpikes
    followed by a scalar shift, and of the oracle."""
    rng = np.random.RandomState(T * 64 + delay)
    params = (0, 5120, 1024, 128, 2)
    w = (np.round((rng.rand(3, 13, 1, 2, T) - 0.5) * 90) * (rng.rand(3, 13, 1, 2, T) < 0.3)).astype(np.float32)
    wd = G.dev(w)
    s_o, v_o, u_o = co.loihi_get_spikes(w, *params)
    want_d = co.shift(s_o, float(delay), 1.0)
    for current in (True, False):
        d, v, u = G.c_loihi_delayed(wd, *params, delay, current=current)
        np.testing.assert_array_equal(G.host(d), want_d)
        np.testing.assert_array_equal(G.host(v), v_o)
        if current:
            np.testing.assert_array_equal(G.host(u), u_o)
    s, _, _ = G.c_loihi(wd, *params)
    np.testing.assert_array_equal(G.host(d), G.host(G.c_shift_scalar(s, delay, 1.0)))
    assert T < 30 or s_o.sum() > 0


def test_loihi_get_spikes_delayed_sizes_outside_the_fused_path():
    import slayerpytorch_b200
    from slayerpytorch_b200.capi import SlayerB200Error
    _, lc = slayerpytorch_b200.load_ops()
    rng = np.random.RandomState(4)
    w = (np.round((rng.rand(40, 300) - 0.5) * 90) * (rng.rand(40, 300) < 0.3)).astype(np.float32)
    wd = G.dev(w).view(1, 40, 1, 1, 300)
    with pytest.raises(SlayerB200Error):
        G.c_loihi_delayed(wd, 0, 5120, 1024, 128, 1, 64)
    s_o, v_o, u_o = co.loihi_get_spikes(w, 0, 5120, 1024, 128, 1)
    for delay in (64, 100, 400):                       # the operator runs getSpikes + shift
        d, v, u = lc.getSpikesDelayed(wd, 0, 5120, 1024, 128, 1, delay, True)
        np.testing.assert_array_equal(G.host(d).reshape(40, 300), co.shift(s_o, float(delay), 1.0))
        np.testing.assert_array_equal(G.host(v).reshape(40, 300), v_o)
        np.testing.assert_array_equal(G.host(u).reshape(40, 300), u_o)
    assert len(lc.getSpikesDelayed(wd, 0, 5120, 1024, 128, 1, 1)) == 2


def test_loihi_reference_numpy_model_fixture(golden_dir):
    g = np.load(golden_dir + "/ref_python.npz")
    for k in range(int(g["nrn_count"])):
        p = [int(v) for v in g["nrn%d_params" % k]]
        s, v, u = G.c_loihi(G.dev(g["nrn%d_w" % k]), *p)
        np.testing.assert_array_equal(G.host(s), g["nrn%d_spike" % k])
        np.testing.assert_array_equal(G.host(u), g["nrn%d_current" % k])
        np.testing.assert_array_equal(G.host(v), g["nrn%d_voltage" % k])


# ---------------------------------------------------------------------------- spike_grad
@pytest.mark.parametrize("n", [1, 3, 4, 1023, 4096 + 5])
def test_spike_grad(n):
    rng = np.random.RandomState(n)
    g = rng.randn(n).astype(np.float32)
    u = (rng.randn(n) * 30).astype(np.float32)
    for theta, tau, scale in ((10.0, 10.0, 1.0), (10.0, 1.0, 1.0), (5120.0, 5120.0, 1 / 195.0)):
        got = G.host(G.c_spike_grad(G.dev(g), G.dev(u), theta, tau, scale))
        want = co.spike_grad(g, u, theta, tau, scale)
        np.testing.assert_allclose(got, want, rtol=REL, atol=1e-37)
        # and against the tensor expression it replaces (src/slayer.py:862)
        ut, gt = torch.from_numpy(u).cuda(), torch.from_numpy(g).cuda()
        th, ta, sc = (torch.tensor(v, device="cuda", dtype=torch.float32) for v in (theta, tau, scale))
        ref = gt * (sc / ta * torch.exp(-torch.abs(ut - th) / ta))
        np.testing.assert_allclose(got, ref.cpu().numpy(), rtol=REL, atol=1e-37)


# ------------------------------------------------------------------- srm_get_spikes_delayed
@pytest.mark.parametrize("T", [4, 32, 36, 64, 100, 128, 300, 500, 2000, 2048])
@pytest.mark.parametrize("nus", [1, 11, 34, 110])
def test_srm_delayed_equals_get_spikes_then_shift(T, nus):
    """Spikes written once, already delayed: the bits of getSpikes followed by shift."""
    rng = np.random.RandomState(T * 7 + nus)
    shape = (3, 5, 2, 1, T)
    u0, nu = srm_case(rng, shape, nus)
    n_neurons = 10
    Ts = 0.5
    lut = ((rng.rand(n_neurons) * 2 - 1) * min(T + 3, 70) * Ts).astype(np.float32)
    lut[0], lut[1], lut[2], lut[3] = 0.0, 3.0 * Ts, -2.0 * Ts, 1e6
    nud, ld = G.dev(nu), G.dev(lut)
    ua = G.dev(u0)
    want_s = G.c_srm(ua, nud, 10.0, Ts)
    want_d = G.host(G.c_shift_lut(want_s, ld, Ts))
    assert want_d.any() or T < 8
    ub = G.dev(u0)
    got_d = G.host(G.c_srm_delayed(ub, nud, ld, 10.0, Ts))
    np.testing.assert_array_equal(got_d, want_d)
    assert_same_floats(G.host(ub), G.host(ua))
    # oracle
    s_o, u_o = co.srm_get_spikes(u0, nu, 10.0, Ts)
    np.testing.assert_array_equal(got_d, co.shift(s_o, lut, Ts))
    # one delay for every row
    for sv in (0.0, 2.0 * Ts, -5.0 * Ts, -1e9):
        uc = G.dev(u0)
        got = G.host(G.c_srm_delayed(uc, nud, None, 10.0, Ts, scalar=sv))
        np.testing.assert_array_equal(got, G.host(G.c_shift_scalar(want_s, sv, Ts)))


def test_srm_delayed_rows_not_a_multiple_of_32_and_positive_theta_padding():
    rng = np.random.RandomState(99)
    shape = (7, 9, 1, 1, 300)                     # 63 rows
    u0, nu = srm_case(rng, shape, 11)
    lut = (rng.rand(9) * 8 - 2).astype(np.float32)
    for theta in (10.0, -1.0):                    # theta < 0: the zero padding past the row end would spike
        ua, ub = G.dev(u0), G.dev(u0)
        want = G.host(G.c_shift_lut(G.c_srm(ua, G.dev(nu), theta, 1.0), G.dev(lut), 1.0))
        got = G.host(G.c_srm_delayed(ub, G.dev(nu), G.dev(lut), theta, 1.0))
        np.testing.assert_array_equal(got, want)
        assert_same_floats(G.host(ub), G.host(ua))


@pytest.mark.parametrize("T", [1, 7, 301, 1450, 2052])
def test_srm_delayed_sizes_outside_the_fused_path(T):
    """T % 4 != 0 or T > 2048: needs the scratch buffer, then runs as the two operators."""
    from slayerpytorch_b200.capi import SlayerB200Error
    rng = np.random.RandomState(T)
    shape = (2, 6, 1, 1, T)
    u0, nu = srm_case(rng, shape, 11)
    lut = (rng.rand(6) * 8 - 2).astype(np.float32)
    ua, ub = G.dev(u0), G.dev(u0)
    want = G.host(G.c_shift_lut(G.c_srm(ua, G.dev(nu), 10.0, 1.0), G.dev(lut), 1.0))
    got = G.host(G.c_srm_delayed(ub, G.dev(nu), G.dev(lut), 10.0, 1.0, scratch=True))
    np.testing.assert_array_equal(got, want)
    with pytest.raises(SlayerB200Error):
        G.c_srm_delayed(G.dev(u0), G.dev(nu), G.dev(lut), 10.0, 1.0, scratch=False)


# ----------------------------------------------------------------------- corr_spike_grad
@pytest.mark.parametrize("shape,K,Ts", [((1, 1, 1, 1, 1), 1, 1.0), ((2, 3, 1, 1, 7), 3, 1.0), ((5, 10, 4, 3, 500), 77, 0.1),
                                        ((3, 16, 1, 1, 300), 77, 1.0), ((4, 8, 2, 1, 301), 12, 0.5), ((2, 6, 1, 1, 1450), 110, 1.0),
                                        ((3, 5, 1, 1, 33), 40, 2.0), ((70, 37, 1, 1, 302), 77, 1.0), ((1, 3, 1, 1, 5001), 2, 1.0),
                                        ((2, 2, 1, 1, 2500), 2300, 1.0), ((2, 2, 1, 1, 64), 0, 1.0)])
def test_corr_spike_grad_equals_corr_then_spike_grad(shape, K, Ts):
    """The backward step of "spike, then psp" in one launch: corr of the gradient times the
    surrogate gradient at the potential.  Equal to the two operators it replaces (the product is
    taken of the filtered value rounded to fp32 either way; only denormal intermediates of the
    surrogate differ: 1e-37 absolute) and to the oracle within 1e-5."""
    rng = np.random.RandomState(sum(shape) + K)
    g = rng.randn(*shape).astype(np.float32)
    u = (rng.randn(*shape) * 30).astype(np.float32)
    f = rng.randn(K).astype(np.float32)
    gd, ud, fd = G.dev(g), G.dev(u), G.dev(f)
    for theta, tau, scale in ((10.0, 10.0, 1.0), (5120.0, 5120.0, 1 / 195.0)):
        got = G.host(G.c_corr_spike_grad(gd, fd, ud, theta, tau, scale, Ts))
        two = G.host(G.c_spike_grad(G.c_conv(gd, fd, Ts, corr=True), ud, theta, tau, scale))
        np.testing.assert_allclose(got, two, rtol=0, atol=1e-37)
        want = co.spike_grad(co.corr(g, f, Ts), u, theta, tau, scale)
        np.testing.assert_allclose(got, want, rtol=REL, atol=1e-37)


def test_corr_spike_grad_divides_like_the_separate_pass_for_any_tau():
    """The epilogue divides by tau through its reciprocal and two fused corrections; the quotient
    must be the correctly rounded one for every tau it accepts (a significand of all ones, thirds,
    tiny and huge values), and tau outside its range takes the two passes."""
    rng = np.random.RandomState(5)
    g = rng.randn(64, 300).astype(np.float32)
    u = (rng.randn(64, 300) * np.logspace(-3, 3, 300, dtype=np.float32)).astype(np.float32)
    u[3, 7], u[4, 8], u[5, 9] = np.inf, -np.inf, np.nan
    f = rng.randn(20).astype(np.float32)
    gd, ud, fd = G.dev(g), G.dev(u), G.dev(f)
    c = G.c_conv(gd, fd, 1.0, corr=True)
    taus = [np.nextafter(np.float32(2), np.float32(1)), np.nextafter(np.float32(1), np.float32(2)), np.float32(1 / 3), np.float32(0.1),
            np.float32(7.3), np.float32(1e-3), np.float32(123456.7), np.float32(2.0 ** -60), np.float32(2.0 ** 60),
            np.float32(1e-30), np.float32(1e30)] + list(rng.uniform(0.5, 64, 8).astype(np.float32))
    cmax = float(c.abs().max())
    for tau in taus:
        for theta in (0.0, 10.0):
            got = G.host(G.c_corr_spike_grad(gd, fd, ud, theta, float(tau), 1.0, 1.0))
            two = G.host(G.c_spike_grad(c, ud, theta, float(tau), 1.0))
            # an exponential below 1.18e-38 is flushed to zero in the filter's translation unit and kept
            # as a denormal by the separate pass; scale / tau and the filtered value multiply that
            flush = 1.2e-38 * (1.0 / float(tau)) * cmax
            np.testing.assert_allclose(got, two, rtol=0, atol=1e-37 + flush, err_msg="tau = %r" % tau)


def test_corr_spike_grad_unaligned_buffers_and_many_rows():
    rng = np.random.RandomState(78)
    f = rng.randn(77).astype(np.float32)
    for rows, T, off in ((9, 300, 1), (70, 302, 2), (1000, 300, 0), (33, 2000, 3)):
        n = rows * T
        g, u = rng.randn(n + 3).astype(np.float32), (rng.randn(n + 3) * 20).astype(np.float32)
        gd, ud = G.dev(g)[off:off + n].view(rows, T), G.dev(u)[off:off + n].view(rows, T)
        got = G.host(G.c_corr_spike_grad(gd, G.dev(f), ud, 10.0, 10.0, 1.0, 1.0))
        two = G.host(G.c_spike_grad(G.c_conv(gd, G.dev(f), 1.0, corr=True), ud, 10.0, 10.0, 1.0))
        np.testing.assert_allclose(got, two, rtol=0, atol=1e-37)


# ----------------------------------------------------------------------- spike_grad_shift
@pytest.mark.parametrize("shape,Ts", [((1, 1, 1, 1, 1), 1.0), ((2, 3, 1, 1, 7), 1.0), ((5, 10, 4, 3, 500), 0.1),
                                      ((3, 16, 1, 1, 300), 1.0), ((4, 8, 2, 1, 301), 0.5), ((2, 6, 1, 1, 1450), 1.0),
                                      ((3, 5, 1, 1, 33), 2.0), ((7, 37, 1, 1, 1450), 1.0), ((5, 51, 1, 1, 6), 1.0),
                                      ((3, 11, 1, 1, 2), 1.0), ((13, 67, 1, 1, 45), 1.0), ((1, 3, 1, 1, 5001), 1.0)])
def test_spike_grad_shift_equals_shift_then_spike_grad(shape, Ts):
    """The fused backward pass gives the bits of the two operators it replaces, and of the oracle."""
    rng = np.random.RandomState(sum(shape) + 1)
    n_neurons = int(np.prod(shape[1:-1]))
    g = rng.randn(*shape).astype(np.float32)
    u = (rng.randn(*shape) * 30).astype(np.float32)
    lut = ((rng.rand(n_neurons) * 2 - 1) * min(shape[-1] + 2, 12) * Ts).astype(np.float32)
    lut[0] = 0.0
    gd, ud, ld = G.dev(g), G.dev(u), G.dev(lut)
    for theta, tau, scale in ((10.0, 10.0, 1.0), (5120.0, 5120.0, 1 / 195.0)):
        got = G.host(G.c_spike_grad_shift(gd, ud, ld, theta, tau, scale, Ts))
        two = G.host(G.c_spike_grad(G.c_shift_lut(gd, ld, Ts), ud, theta, tau, scale))
        assert_same_floats(got, two)
        want = co.spike_grad(co.shift(g, lut, Ts), u, theta, tau, scale)
        np.testing.assert_allclose(got, want, rtol=REL, atol=1e-37)
        for sv in (0.0, 3.0 * Ts, -2.0 * Ts, 1e9):
            got = G.host(G.c_spike_grad_shift(gd, ud, None, theta, tau, scale, Ts, scalar=sv))
            two = G.host(G.c_spike_grad(G.c_shift_scalar(gd, sv, Ts), ud, theta, tau, scale))
            assert_same_floats(got, two)


def test_spike_grad_shift_unaligned_buffers():
    rng = np.random.RandomState(77)
    n = 3 * 4 * 300
    g, u = rng.randn(n + 1).astype(np.float32), (rng.randn(n + 1) * 20).astype(np.float32)
    lut = (rng.rand(4) * 6 - 3).astype(np.float32)
    gd, ud = G.dev(g)[1:].view(3, 4, 300), G.dev(u)[1:].view(3, 4, 300)
    got = G.host(G.c_spike_grad_shift(gd, ud, G.dev(lut), 10.0, 10.0, 1.0, 1.0))
    want = co.spike_grad(co.shift(g[1:].reshape(3, 4, 300), lut, 1.0), u[1:].reshape(3, 4, 300), 10.0, 10.0, 1.0)
    np.testing.assert_allclose(got, want, rtol=REL, atol=1e-37)


# ---------------------------------------------------------------------------- delay_grad
@pytest.mark.parametrize("shape,Ts", [((1, 1, 1, 1, 1), 1.0), ((2, 3, 1, 1, 7), 1.0), ((9, 5, 2, 1, 300), 1.0),
                                      ((4, 16, 3, 3, 301), 0.5), ((64, 10, 1, 1, 300), 1.0),
                                      ((3, 2, 1, 1, 1450), 0.1), ((17, 4, 1, 1, 2000), 2.0)])
def test_delay_grad(shape, Ts):
    rng = np.random.RandomState(sum(shape))
    g = rng.randn(*shape).astype(np.float32)
    out = (rng.randn(*shape) * (rng.rand(*shape) < 0.4)).astype(np.float32)
    got = G.host(G.c_delay_grad(G.dev(g), G.dev(out), Ts))
    want = co.delay_grad(g, out, Ts).ravel()          # double-precision sum
    scale = np.abs(want).max() + 1e-30
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-5 * scale * np.sqrt(shape[0] * shape[-1]) / 10)
    # and against the composition it replaces (src/slayer.py:950-954) on the same device
    gt, ot = G.dev(g), G.dev(out)
    diff = torch.tensor([-1.0, 1.0], device="cuda") / Ts
    ref = torch.sum(gt * G.c_conv(ot, diff, 1.0), [0, -1]).reshape(-1) * Ts
    np.testing.assert_allclose(got, G.host(ref), rtol=0, atol=2e-5 * scale * np.sqrt(shape[0] * shape[-1]) / 10)
    # determinism: a second call returns the same bits
    again = G.host(G.c_delay_grad(gt, ot, Ts))
    np.testing.assert_array_equal(got, again)


def test_delay_grad_unaligned_and_empty():
    rng = np.random.RandomState(5)
    g = rng.randn(3 * 4 * 300 + 1).astype(np.float32)
    o = rng.randn(3 * 4 * 300 + 1).astype(np.float32)
    gd, od = G.dev(g)[1:].view(3, 4, 300), G.dev(o)[1:].view(3, 4, 300)
    got = G.host(G.c_delay_grad(gd, od, 1.0))
    want = co.delay_grad(g[1:].reshape(3, 4, 300), o[1:].reshape(3, 4, 300), 1.0).ravel()
    np.testing.assert_allclose(got, want, rtol=0, atol=1e-4 * np.abs(want).max())
    assert G.c_delay_grad(torch.empty(0, 4, 300, device="cuda"), torch.empty(0, 4, 300, device="cuda"), 1.0).eq(0).all()
    assert G.c_delay_grad(torch.empty(2, 0, 300, device="cuda"), torch.empty(2, 0, 300, device="cuda"), 1.0).numel() == 0


# ------------------------------------------- full-size runs checked on a random row sample
def sample_rows(rows, n, seed):
    return np.sort(np.random.RandomState(seed).choice(rows, size=min(n, rows), replace=False))


def test_full_size_config2_chain_rows_match_oracle(golden_dir):
    """The hidden layer of the SRM MLP workload (64 x 512 neurons x 300 steps): psp -> getSpikes ->
    per-neuron shift, then shift^-1 -> surrogate -> corr, run at full size on the GPU and
    checked exactly on 1500 random rows (rows are independent)."""
    g = np.load(golden_dir + "/ref_python.npz")
    srm_k, ref_k = g["srm_Ts1_srmKernel"], g["srm_Ts1_refKernel"]
    gen = torch.Generator().manual_seed(1002)
    N, C, T = 64, 512, 300
    a = (torch.randn(N, C, 1, 1, T, generator=gen).abs() * 2.5 * (torch.rand(N, C, 1, 1, T, generator=gen) < 0.3)).float()
    delay = (torch.rand(C, generator=gen) * 5).float()
    grad = torch.randn(N, C, 1, 1, T, generator=gen).float()
    ad, kd, rd, dd, gd = a.cuda(), G.dev(srm_k), G.dev(ref_k), delay.cuda(), grad.cuda()
    u = G.c_conv(ad, kd, 1.0)
    u_pre = u.clone()
    s = G.c_srm(u, rd, 10.0, 1.0)
    out = G.c_shift_lut(s, dd, 1.0)
    g1 = G.c_shift_lut(gd, -dd, 1.0)
    g2 = G.c_spike_grad(g1, u, 10.0, 10.0, 1.0)
    g3 = G.c_conv(g2, kd, 1.0, corr=True)
    rows = sample_rows(N * C, 1500, 1)
    pick = lambda t: G.host(t).reshape(N * C, T)[rows]
    an, gn = a.numpy().reshape(N * C, T)[rows], grad.numpy().reshape(N * C, T)[rows]
    dn = delay.numpy()[rows % C]
    u0 = co.conv(an, srm_k, 1.0)
    assert_close_or_equal(pick(u_pre), u0)
    s_w, u_w = co.srm_get_spikes(u0, ref_k, 10.0, 1.0)
    np.testing.assert_array_equal(pick(s), s_w)
    np.testing.assert_array_equal(pick(u), u_w)
    assert 0.001 < s_w.mean() < 0.5
    out_w = np.stack([co.shift(s_w[i:i + 1], dn[i], 1.0)[0] for i in range(len(rows))])
    np.testing.assert_array_equal(pick(out), out_w)
    g1_w = np.stack([co.shift(gn[i:i + 1], -dn[i], 1.0)[0] for i in range(len(rows))])
    np.testing.assert_array_equal(pick(g1), g1_w)
    g2_w = co.spike_grad(g1_w, u_w, 10.0, 10.0, 1.0)
    np.testing.assert_allclose(pick(g2), g2_w, rtol=REL, atol=1e-37)
    assert_close_or_equal(pick(g3), co.corr(pick(g2), srm_k, 1.0))
    # size-independent properties over the whole tensors
    assert torch.all((s == 0) | (s == 1.0))
    back = G.c_shift_lut(out, -dd, 1.0)                         # shift then un-shift: head survives
    dsteps = dd.floor().long().view(1, C, 1, 1, 1)
    tt = torch.arange(T, device="cuda").view(1, 1, 1, 1, T)
    keep = tt < (T - dsteps)
    assert torch.equal(back * keep, s * keep)


def test_full_size_loihi_layer_rows_match_oracle():
    """A config-5-like Loihi layer (8 x 32 x 16 x 16 neurons x 1450 steps, T % 4 != 0)."""
    gen = torch.Generator().manual_seed(1005)
    shape = (8, 32, 16, 16, 1450)
    w = (torch.randint(-128, 128, shape, generator=gen) * (torch.rand(shape, generator=gen) < 0.08)).float()
    s, v, u = G.c_loihi(w.cuda(), 0, 5120, 1024, 128, 1)
    rows_total = 8 * 32 * 16 * 16
    rows = sample_rows(rows_total, 1000, 2)
    wn = w.numpy().reshape(rows_total, 1450)[rows]
    want = co.loihi_get_spikes(wn, 0, 5120, 1024, 128, 1)
    for a, b in zip((s, v, u), want):
        np.testing.assert_array_equal(G.host(a).reshape(rows_total, 1450)[rows], b)
    assert 0.0005 < want[0].mean() < 0.5
    sh = G.c_shift_scalar(s, 1, 1)
    assert torch.equal(sh[..., 1:], s[..., :-1]) and not sh[..., 0].any()


def test_linearity_and_adjointness_at_full_size():
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(4096, 2000, generator=gen).cuda()
    y = torch.randn(4096, 2000, generator=gen).cuda()
    f = torch.randn(77, generator=gen).cuda()
    cx = G.c_conv(x, f, 1.0)
    lhs = (cx.double() * y.double()).sum()
    rhs = (x.double() * G.c_conv(y, f, 1.0, corr=True).double()).sum()
    assert abs(lhs - rhs) < 1e-6 * max(1.0, abs(lhs))
    two = G.c_conv(2 * x, f, 1.0)
    assert torch.equal(two, 2 * cx)        # scaling by a power of two is exact


# ------------------------------------------------ both data-movement paths of SRM getSpikes
@pytest.mark.parametrize("T,nus", [(16, 11), (300, 11), (304, 3), (2000, 34), (500, 160)])
def test_srm_bulk_tensor_and_cp_async_paths_agree(T, nus):
    """T % 4 == 0 and aligned buffers take the bulk-tensor-copy kernel; with it switched off the
    cp.async kernel runs.  Both must reproduce the oracle bit for bit."""
    from slayerpytorch_b200 import capi
    rng = np.random.RandomState(T + nus)
    u, nu = srm_case(rng, (3, 5, 1, 7, T), nus)
    s_want, u_want = co.srm_get_spikes(u, nu, 10.0, 1.0)
    try:
        for enable in (True, False):
            capi.set_tma(enable)
            ud = G.dev(u)
            s = G.host(G.c_srm(ud, G.dev(nu), 10.0, 1.0))
            np.testing.assert_array_equal(s, s_want, err_msg="tma=%s" % enable)
            assert_same_floats(G.host(ud), u_want)
    finally:
        capi.set_tma(True)
    assert capi.device_status() == 0


def test_device_status_word_is_clear_after_the_suite_so_far():
    from slayerpytorch_b200 import capi
    assert capi.device_status() == 0


def test_a_wait_that_runs_out_is_reported_and_leaves_the_device_usable():
    """The give-up branch of the bounded barrier waits, made to run out on purpose: a one-thread
    kernel polls a barrier that nothing completes 1000 times, records the status code and
    returns.  The code is read and cleared by device_status, and the next launch is clean."""
    from slayerpytorch_b200 import capi
    assert capi.device_status() == 0
    capi.call("slayer_b200_selftest_bounded_wait", 1000, G.stream())
    assert capi.device_status() == 0x5101
    assert capi.device_status() == 0                     # reading cleared it
    rng = np.random.RandomState(3)
    u, nu = srm_case(rng, (2, 3, 1, 7, 300), 11)
    ud = G.dev(u)
    s = G.host(G.c_srm(ud, G.dev(nu), 10.0, 1.0))
    np.testing.assert_array_equal(s, co.srm_get_spikes(u, nu, 10.0, 1.0)[0])
    assert capi.device_status() == 0
