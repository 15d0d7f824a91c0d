"""ctypes front end of the C oracle (``slayer_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, the smoke check and the benchmark's CPU legs import this module; the
shipped package never does.  All functions take and return NumPy ``float32`` arrays laid out
``[..., T]`` with time last; rows are every leading index flattened.

Reference files each function restates are cited in ``slayer_oracle.c``.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "slayer_oracle.c")
LIB = os.path.join(HERE, "libslayer_oracle.so")

_lib = None


def build(force=False):
    """Compile the C oracle with gcc (OpenMP, hardware FMA, no implicit contraction)."""
    if not force and os.path.isfile(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["gcc", "-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fno-fast-math",
           "-fopenmp", "-shared", "-fPIC", "-o", LIB, SRC, "-lm"]
    subprocess.check_call(cmd)
    return LIB


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(LIB)
        f32p = ctypes.c_void_p
        i64 = ctypes.c_int64
        u32 = ctypes.c_uint32
        fl = ctypes.c_float
        L.oracle_conv.argtypes = [f32p, f32p, f32p, i64, i64, i64, fl]
        L.oracle_corr.argtypes = [f32p, f32p, f32p, i64, i64, i64, fl]
        L.oracle_shift_scalar.argtypes = [f32p, f32p, fl, i64, i64, fl]
        L.oracle_shift_lut.argtypes = [f32p, f32p, f32p, i64, i64, i64, fl]
        L.oracle_srm_get_spikes.argtypes = [f32p, f32p, f32p, i64, i64, i64, fl, fl]
        L.oracle_loihi_get_spikes.argtypes = [f32p, f32p, f32p, f32p, i64, i64,
                                              u32, u32, u32, u32, u32]
        L.oracle_spike_grad.argtypes = [f32p, f32p, f32p, i64, fl, fl, fl]
        L.oracle_delay_grad.argtypes = [f32p, f32p, f32p, i64, i64, i64, fl]
        L.oracle_delay_grad.restype = None
        L.oracle_set_ftz.argtypes = [ctypes.c_int]
        L.oracle_set_threads.argtypes = [ctypes.c_int]
        L.oracle_max_threads.restype = ctypes.c_int
        for name in ("oracle_conv", "oracle_corr", "oracle_shift_scalar", "oracle_shift_lut",
                     "oracle_srm_get_spikes", "oracle_loihi_get_spikes", "oracle_spike_grad",
                     "oracle_set_ftz", "oracle_set_threads"):
            getattr(L, name).restype = None
        _lib = L
    return _lib


def set_threads(n):
    lib().oracle_set_threads(int(n))


def max_threads():
    return int(lib().oracle_max_threads())


def set_ftz(on):
    """Flush denormals like the reference's -use_fast_math GPU build (default: off)."""
    lib().oracle_set_ftz(1 if on else 0)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _rows_T(x):
    T = x.shape[-1] if x.ndim else 1
    return (x.size // T if T else 0), T


def conv(x, f, Ts=1.0):
    x, f = _f32(x), _f32(f).ravel()
    out = np.empty_like(x)
    rows, T = _rows_T(x)
    if x.size:
        lib().oracle_conv(_p(out), _p(x), _p(f), rows, T, f.size, float(Ts))
    return out


def corr(x, f, Ts=1.0):
    x, f = _f32(x), _f32(f).ravel()
    out = np.empty_like(x)
    rows, T = _rows_T(x)
    if x.size:
        lib().oracle_corr(_p(out), _p(x), _p(f), rows, T, f.size, float(Ts))
    return out


def shift(x, shift_value, Ts=1.0):
    """Scalar or per-neuron shift; dispatch as shiftCuda does (src/cuda/slayerKernels.cu:77-108)."""
    x = _f32(x)
    out = np.empty_like(x)
    rows, T = _rows_T(x)
    if np.ndim(shift_value) == 0 or np.size(shift_value) == 1:
        sv = float(np.asarray(shift_value, dtype=np.float32).reshape(-1)[0])
        if x.size:
            lib().oracle_shift_scalar(_p(out), _p(x), sv, rows, T, float(Ts))
        return out
    lut = _f32(shift_value).ravel()
    n_batch = x.shape[0]
    n_neurons = rows // n_batch if n_batch else 0
    if lut.size != n_neurons:
        raise ValueError("shift and number of neurons must be same")
    if x.size:
        lib().oracle_shift_lut(_p(out), _p(x), _p(lut), n_batch, n_neurons, T, float(Ts))
    return out


def srm_get_spikes(u, nu, theta, Ts=1.0):
    """Returns (spikes, u_after); the input array is not modified."""
    u = _f32(u).copy()
    nu = _f32(nu).ravel()
    s = np.empty_like(u)
    rows, T = _rows_T(u)
    if u.size:
        lib().oracle_srm_get_spikes(_p(s), _p(u), _p(nu), rows, nu.size, T, float(theta), float(Ts))
    return s, u


def loihi_get_spikes(w, wgtExp, theta, iDecay, vDecay, refDelay):
    """Returns (spike, voltage, current) like slayerLoihiCuda.getSpikes."""
    w = _f32(w)
    s, v, u = np.empty_like(w), np.empty_like(w), np.empty_like(w)
    rows, T = _rows_T(w)
    if refDelay < 1:
        raise ValueError("refDelay must be >= 1")
    if w.size:
        lib().oracle_loihi_get_spikes(_p(s), _p(v), _p(u), _p(w), rows, T,
                                      int(wgtExp), int(theta), int(iDecay), int(vDecay), int(refDelay))
    return s, v, u


def spike_grad(g, u, theta, tau, scale):
    g, u = _f32(g), _f32(u)
    out = np.empty_like(g)
    if g.size:
        lib().oracle_spike_grad(_p(out), _p(g), _p(u), g.size, float(theta), float(tau), float(scale))
    return out


def delay_grad(g, out, Ts=1.0):
    """gradDelay of shape g.shape[1:-1] (one value per neuron), as _delayFunction.backward."""
    g, out = _f32(g), _f32(out)
    n_batch, T = g.shape[0], g.shape[-1]
    n_neurons = g.size // (n_batch * T) if n_batch * T else 0
    res = np.zeros(n_neurons, np.float32)
    if n_neurons:
        lib().oracle_delay_grad(_p(res), _p(g), _p(out), n_batch, n_neurons, T, float(Ts))
    return res.reshape(g.shape[1:-1])
