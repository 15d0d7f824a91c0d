"""GPU: address events -> spike tensor against the reference's own event.toSpikeTensor (fixtures
in tests/golden/events_ref.npz) and against the NumPy oracle on cases the fixtures do not hold
(time shift, batches, packed output)."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import numpy_loops as nl
from slayerpytorch_b200 import capi
from tests import gpu_util as G

pytestmark = pytest.mark.gpu


def dev_i32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).cuda()


def dev_f64(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float64)).cuda()


def c_bin(start, x, y, p, t, Ts, t_start, mode, n=None):
    """Through the C ABI; start is [C,H,W,T] or [N,C,H,W,T] float32 (host array)."""
    base = G.dev(start)
    out = base.clone()
    shape = start.shape if start.ndim == 5 else (1,) + start.shape
    xs, ps, ts = dev_i32(x), dev_i32(p), dev_f64(t)
    ys = None if y is None else dev_i32(y)
    ns = None if n is None else dev_i32(n)
    capi.call("slayer_b200_bin_events", G.ptr(out), G.ptr(base) if mode == "SUM" else None,
              None if ns is None else G.ptr(ns), G.ptr(xs), None if ys is None else G.ptr(ys), G.ptr(ps), G.ptr(ts),
              len(x), *shape, ctypes.c_double(Ts), int(t_start), 1 if mode == "SUM" else 0, G.stream())
    return G.host(out)


def test_binning_equals_the_reference_fixtures(golden_dir):
    g = np.load(golden_dir + "/events_ref.npz")
    for case in g["cases"]:
        tag, mode = str(case).split(":")
        y = g[tag + "_y"] if tag + "_y" in g else None
        got = c_bin(g[tag + "_start"], g[tag + "_x"], y, g[tag + "_p"], g[tag + "_t"], float(g[tag + "_Ts"]), 0, mode)
        np.testing.assert_array_equal(got, g[tag + "_out"], err_msg=tag)
        assert (got != 0).sum() > 50


def test_event_class_mirrors_the_reference_interface(golden_dir):
    from slayerpytorch_b200 import spikeio
    g = np.load(golden_dir + "/events_ref.npz")
    for case in g["cases"]:
        tag, mode = str(case).split(":")
        y = g[tag + "_y"] if tag + "_y" in g else None
        td = spikeio.event(g[tag + "_x"], y, g[tag + "_p"], g[tag + "_t"])
        start = G.dev(g[tag + "_start"])
        got = td.toSpikeTensor(start, samplingTime=float(g[tag + "_Ts"]), binningMode=mode)
        np.testing.assert_array_equal(G.host(got), g[tag + "_out"], err_msg=tag)
        if mode == "OR":
            assert got.data_ptr() == start.data_ptr()              # filled in place, like the reference
            packed = td.toPackedSpikes(g[tag + "_out"].shape, samplingTime=float(g[tag + "_Ts"]))
            np.testing.assert_array_equal(G.host(packed.dense()), g[tag + "_out"], err_msg=tag + " packed")
    with pytest.raises(Exception, match="Unsupported binningMode"):
        td.toSpikeTensor(start, binningMode="XOR")
    with pytest.raises(RuntimeError):
        td.toSpikeTensor(torch.zeros(2, 2, 2, 2))


@pytest.mark.parametrize("Ts,t_start", [(1.0, 0), (1.0, 17), (0.5, 40), (2.0, -3)])
def test_binning_with_time_shift_and_batches_against_the_oracle(Ts, t_start):
    rng = np.random.RandomState(int(Ts * 10) + t_start)
    N, C, H, W, T = 3, 2, 6, 7, 70
    n_ev = 5000
    x, y, p = rng.randint(-1, W + 1, n_ev), rng.randint(-1, H + 1, n_ev), rng.randint(0, C + 1, n_ev)
    n = rng.randint(-1, N + 1, n_ev)
    t = rng.rand(n_ev) * (T + 30) * Ts
    t[:20] = (np.arange(20) + 0.5) * Ts                        # ties: rounded to even
    t[20] = np.nan
    for mode in ("OR", "SUM"):
        start = (rng.rand(N, C, H, W, T) < 0.05).astype(np.float32) * 2.5 if mode == "SUM" else np.zeros((N, C, H, W, T), np.float32)
        want = nl.bin_events(start, x, y, p, np.nan_to_num(t, nan=-1e9), Ts, t_start, mode, n=n)
        got = c_bin(start, x, y, p, t, Ts, t_start, mode, n=n)
        np.testing.assert_array_equal(got, want)
        assert (got != start).sum() > 500


def test_empty_inputs():
    z = np.zeros((2, 3, 4, 5), np.float32)
    e = np.zeros(0, np.int32)
    np.testing.assert_array_equal(c_bin(z, e, e, e, np.zeros(0), 1.0, 0, "OR"), z)
    lib = capi.load()
    assert lib.slayer_b200_bin_events(None, None, None, None, None, None, None, 5, 1, 0, 4, 4, 4,
                                      ctypes.c_double(1.0), 0, 0, None) == 0
    assert lib.slayer_b200_bin_events(None, None, None, None, None, None, None, 5, 1, 2, 4, 4, 4,
                                      ctypes.c_double(0.0), 0, 0, None) == -1
