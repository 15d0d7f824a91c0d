"""NumPy time-loop restatement of the same operators.  TEST INFRASTRUCTURE ONLY.

A second, independently written statement of the algorithms (one Python iteration per time
step, vectorised across rows) used to cross-check the C oracle on small cases.  It follows
the explicit time-loop models in the reference's own tests:

* SRM spikes:   test/test_slayer002.py:153-167
* Loihi neuron: test/test_slayerLoihi002.py:30-82 (``Neuron.run``), but with the C++ integer
  promotion rules of src/cuda/spikeLoihiKernels.h:44-70 (uint32 products, logical shift)
* shift:        test/test_slayer009.py:29-43 (``checkShift``) with ``int(delay / Ts)`` (:57)
* conv / corr:  src/cuda/convKernels.h:28-33, :55-60 (tap loop; no fused multiply-add here,
  so values agree with the C oracle to rounding, not bit for bit)
* surrogate:    src/slayer.py:862
* event binning: src/spikeFileIO.py:66-144 (``event.toSpikeTensor``), one Python iteration per
  event
"""
import numpy as np


def conv(x, f, Ts=1.0):
    x = np.asarray(x, np.float32)
    f = np.asarray(f, np.float32).ravel()
    T = x.shape[-1]
    acc = np.zeros_like(x)
    for i in range(min(f.size, T)):
        acc[..., i:] = acc[..., i:] + x[..., :T - i] * f[i]
    return acc * np.float32(Ts)


def corr(x, f, Ts=1.0):
    x = np.asarray(x, np.float32)
    f = np.asarray(f, np.float32).ravel()
    T = x.shape[-1]
    acc = np.zeros_like(x)
    for i in range(min(f.size, T)):
        acc[..., :T - i] = acc[..., :T - i] + x[..., i:] * f[i]
    return acc * np.float32(Ts)


def shift_steps(shift, Ts):
    return int(np.float32(shift) / np.float32(Ts))


def shift(x, shift_value, Ts=1.0):
    x = np.asarray(x, np.float32)
    T = x.shape[-1]
    out = np.zeros_like(x)

    def one(dst, src, d):
        if d == 0:
            dst[...] = src
        elif 0 < d < T:
            dst[..., d:] = src[..., :T - d]
        elif -T < d < 0:
            dst[..., :T + d] = src[..., -d:]

    if np.size(shift_value) == 1:
        one(out, x, shift_steps(np.asarray(shift_value).reshape(-1)[0], Ts))
        return out
    lut = np.asarray(shift_value, np.float32).ravel()
    xb = x.reshape(x.shape[0], -1, T)
    ob = out.reshape(x.shape[0], -1, T)
    assert lut.size == xb.shape[1], "shift and number of neurons must be same"
    for n in range(lut.size):
        one(ob[:, n], xb[:, n], shift_steps(lut[n], Ts))
    return out


def srm_get_spikes(u, nu, theta, Ts=1.0):
    u = np.array(u, np.float32, copy=True)
    nu = np.asarray(nu, np.float32).ravel()
    shape = u.shape
    T = shape[-1]
    u = u.reshape(-1, T)
    s = np.zeros_like(u)
    theta = np.float32(theta)
    spike = np.float32(1.0) / np.float32(Ts)
    for t in range(T):
        fired = u[:, t] >= theta
        if fired.any():
            s[fired, t] = spike
            n = min(nu.size, T - t)
            u[fired, t:t + n] += nu[:n]
    return s.reshape(shape), u.reshape(shape)


def loihi_get_spikes(w, wgtExp, theta, iDecay, vDecay, refDelay):
    w = np.asarray(w, np.float32)
    shape = w.shape
    T = shape[-1]
    w = w.reshape(-1, T)
    rows = w.shape[0]
    M = np.uint64(0xFFFFFFFF)

    def u32(a):
        return np.asarray(a).astype(np.int64).astype(np.uint64) & M

    def i32(a):  # reinterpret the low 32 bits as signed
        a = (np.asarray(a, np.uint64) & M).astype(np.int64)
        return np.where(a >= 2 ** 31, a - 2 ** 32, a)

    s = np.zeros((rows, T), np.int64)
    v = np.zeros((rows, T), np.int64)
    u = np.zeros((rows, T), np.int64)
    uOld = np.zeros(rows, np.int64)
    vOld = np.zeros(rows, np.int64)
    ref = np.zeros(rows, np.int64)
    scale = np.uint64(1 << (6 + wgtExp))
    for t in range(1, T):
        uSign = np.where(uOld >= 0, 1, -1)
        vSign = np.where(vOld >= 0, 1, -1)
        wi = np.trunc(w[:, t]).astype(np.int64)
        uMag = ((u32(uSign * uOld) * np.uint64(4096 - iDecay)) & M) >> np.uint64(12)
        uT = i32(u32(uSign) * uMag + scale * u32(wi))
        vMag = ((u32(vSign * vOld) * np.uint64(4096 - vDecay)) & M) >> np.uint64(12)
        vT = i32(u32(vSign) * vMag + u32(uT))
        if t >= refDelay:
            ref = ref - s[:, t - refDelay]
        spike = ((vT > theta) & (ref == 0)).astype(np.int64)
        vOld = np.where((ref == 0) & (spike == 0), vT, 0)
        ref = ref + spike
        s[:, t] = spike
        u[:, t] = uOld = uT
        v[:, t] = np.where(spike > 0, vDecay, vOld)
    f = lambda a: a.astype(np.float32).reshape(shape)
    return f(s), f(v), f(u)


def spike_grad(g, u, theta, tau, scale):
    g = np.asarray(g, np.float32)
    u = np.asarray(u, np.float32)
    theta, tau, scale = np.float32(theta), np.float32(tau), np.float32(scale)
    return g * (scale / tau * np.exp(-np.abs(u - theta) / tau))


def bin_events(tensor, x, y, p, t, sampling_time=1.0, t_start=0, mode="OR", n=None):
    """Address events into a spike tensor, following event.toSpikeTensor
    (src/spikeFileIO.py:66-144): indices are rounded (:95-97, :120), events with any index
    outside the tensor are dropped (:102-107, :121-128), 'OR' sets the bin to 1/samplingTime
    (:108-112) and 'SUM' is an indexed "+=" (:113-117), which NumPy evaluates from the original
    tensor and assigns once per distinct index.  ``tensor`` is [C, H, W, T], or [N, C, H, W, T]
    with a sample index ``n`` per event; ``y`` may be None (one spatial dimension: y = 0).
    Returns a new array."""
    base = np.array(tensor, copy=True)
    out = np.array(tensor, copy=True)
    batched = out.ndim == 5
    shape = out.shape if batched else (1,) + out.shape
    view = out.reshape(shape)
    orig = base.reshape(shape)
    value = out.dtype.type(1.0 / sampling_time)
    xs = np.round(np.asarray(x)).astype(np.int64)
    ps = np.round(np.asarray(p)).astype(np.int64)
    ys = np.zeros_like(xs) if y is None else np.round(np.asarray(y)).astype(np.int64)
    ts = np.round(np.asarray(t, np.float64) / sampling_time).astype(np.int64) - int(t_start)
    ns = np.zeros_like(xs) if n is None else np.asarray(n, np.int64)
    N, C, H, W, T = shape
    for e in range(xs.size):
        if not (0 <= ns[e] < N and 0 <= ps[e] < C and 0 <= ys[e] < H and 0 <= xs[e] < W and 0 <= ts[e] < T):
            continue
        if mode.upper() == "OR":
            view[ns[e], ps[e], ys[e], xs[e], ts[e]] = value
        elif mode.upper() == "SUM":
            view[ns[e], ps[e], ys[e], xs[e], ts[e]] = orig[ns[e], ps[e], ys[e], xs[e], ts[e]] + value
        else:
            raise ValueError("Unsupported binningMode. It was {}".format(mode))
    return out
