"""Helpers for the GPU parity tests: device buffers through torch, calls through the C ABI."""
import ctypes

import numpy as np
import torch

from slayerpytorch_b200 import capi


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.detach().cpu().numpy()


def ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def rows_T(t):
    T = t.shape[-1]
    return (t.numel() // T if T else 0), T


def c_conv(x, f, Ts, corr=False):
    out = torch.empty_like(x)
    rows, T = rows_T(x)
    capi.call("slayer_b200_corr" if corr else "slayer_b200_conv",
              ptr(out), ptr(x), ptr(f), rows, T, f.numel(), float(Ts), stream())
    return out


def c_shift_scalar(x, d, Ts):
    out = torch.empty_like(x)
    rows, T = rows_T(x)
    capi.call("slayer_b200_shift_scalar", ptr(out), ptr(x), float(d), rows, T, float(Ts), stream())
    return out


def c_shift_lut(x, lut, Ts):
    out = torch.empty_like(x)
    rows, T = rows_T(x)
    nb = x.shape[0]
    capi.call("slayer_b200_shift_lut", ptr(out), ptr(x), ptr(lut), nb, rows // nb, T, float(Ts), stream())
    return out


def c_srm(u, nu, theta, Ts):
    """In place on u; returns s."""
    s = torch.empty_like(u)
    rows, T = rows_T(u)
    capi.call("slayer_b200_srm_get_spikes", ptr(s), ptr(u), ptr(nu), rows, nu.numel(), T,
              float(theta), float(Ts), stream())
    return s


def c_loihi(w, wgtExp, theta, iDecay, vDecay, refDelay):
    s, v, u = torch.empty_like(w), torch.empty_like(w), torch.empty_like(w)
    rows, T = rows_T(w)
    capi.call("slayer_b200_loihi_get_spikes", ptr(s), ptr(v), ptr(u), ptr(w), rows, T,
              int(wgtExp), int(theta), int(iDecay), int(vDecay), int(refDelay), stream())
    return s, v, u


def c_spike_grad(g, u, theta, tau, scale):
    out = torch.empty_like(g)
    capi.call("slayer_b200_spike_grad", ptr(out), ptr(g), ptr(u), g.numel(),
              float(theta), float(tau), float(scale), stream())
    return out


def c_delay_grad(g, out, Ts):
    nb, T = g.shape[0], g.shape[-1]
    nn = g.numel() // (nb * T) if nb * T else 0
    res = torch.full((max(nn, 1),), float("nan"), device=g.device, dtype=torch.float32)
    capi.call("slayer_b200_delay_grad", ptr(res), ptr(g), ptr(out), nb, nn, T, float(Ts), stream())
    return res[:nn]


def c_corr_spike_grad(g, f, u, theta, tau, scale, Ts):
    out = torch.full_like(g, float("nan"))
    rows, T = rows_T(g)
    capi.call("slayer_b200_corr_spike_grad", ptr(out), ptr(g), ptr(f), ptr(u), rows, T, f.numel(), float(Ts),
              float(theta), float(tau), float(scale), stream())
    return out


def c_spike_grad_shift(g, u, lut, theta, tau, scale, Ts, scalar=None):
    out = torch.empty_like(g)
    nb, T = g.shape[0], g.shape[-1]
    rows = g.numel() // T if T else 0
    if lut is None:
        capi.call("slayer_b200_spike_grad_shift", ptr(out), ptr(g), ptr(u), None, float(scalar), rows, 1, T,
                  float(Ts), float(theta), float(tau), float(scale), stream())
    else:
        capi.call("slayer_b200_spike_grad_shift", ptr(out), ptr(g), ptr(u), ptr(lut), 0.0, nb, rows // nb, T,
                  float(Ts), float(theta), float(tau), float(scale), stream())
    return out


def c_srm_delayed(u, nu, lut, theta, Ts, scalar=None, scratch=False):
    """In place on u; returns the delayed spikes.  scratch=True passes a buffer for the unfused path."""
    d = torch.full_like(u, float("nan"))
    sc = torch.empty_like(u) if scratch else None
    nb, T = u.shape[0], u.shape[-1]
    rows = u.numel() // T if T else 0
    if lut is None:
        capi.call("slayer_b200_srm_get_spikes_delayed", ptr(d), ptr(sc) if scratch else None, ptr(u), ptr(nu), None,
                  float(scalar), rows, 1, nu.numel(), T, float(theta), float(Ts), stream())
    else:
        capi.call("slayer_b200_srm_get_spikes_delayed", ptr(d), ptr(sc) if scratch else None, ptr(u), ptr(nu), ptr(lut),
                  0.0, nb, rows // nb, nu.numel(), T, float(theta), float(Ts), stream())
    return d


def words_of(T):
    return (T + 31) // 32


def c_pack(s):
    rows, T = rows_T(s)
    bits = torch.empty(s.shape[:-1] + (words_of(T),), dtype=torch.int32, device=s.device)
    capi.call("slayer_b200_pack_spikes", ptr(bits), ptr(s), rows, T, stream())
    return bits


def c_unpack(bits, T, value):
    s = torch.empty(bits.shape[:-1] + (T,), dtype=torch.float32, device=bits.device)
    capi.call("slayer_b200_unpack_spikes", ptr(s), ptr(bits), s.numel() // T if T else 0, T, float(value), stream())
    return s


def c_srm_packed(u, nu, theta):
    """In place on u; returns the packed spikes."""
    rows, T = rows_T(u)
    bits = torch.full(u.shape[:-1] + (words_of(T),), -1, dtype=torch.int32, device=u.device)
    capi.call("slayer_b200_srm_get_spikes_packed", ptr(bits), ptr(u), ptr(nu), rows, nu.numel(), T, float(theta), stream())
    return bits


def c_conv_packed(bits, T, f, value, Ts):
    out = torch.empty(bits.shape[:-1] + (T,), dtype=torch.float32, device=bits.device)
    capi.call("slayer_b200_conv_packed", ptr(out), ptr(bits), ptr(f), out.numel() // T if T else 0, T, f.numel(),
              float(value), float(Ts), stream())
    return out


def c_loihi_delayed(w, wgtExp, theta, iDecay, vDecay, refDelay, delay, current=True):
    d, v = torch.full_like(w, float("nan")), torch.full_like(w, float("nan"))
    u = torch.full_like(w, float("nan")) if current else None
    rows, T = rows_T(w)
    capi.call("slayer_b200_loihi_get_spikes_delayed", ptr(d), ptr(v), ptr(u) if current else None, ptr(w), rows, T,
              int(wgtExp), int(theta), int(iDecay), int(vDecay), int(refDelay), int(delay), stream())
    return d, v, u
